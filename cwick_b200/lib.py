"""ctypes binding of libcwk_attn.so -- the only way this package computes.

There is no CPU or eager fallback: if the shared library is missing or the
process has no CUDA device, `load()` / `Context()` raise.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcwk_attn.so")

OK, ERR_MEMORY, ERR_STATE, ERR_ARGUMENT, ERR_UNSUPPORTED, ERR_CUDA = 0, 4, 5, 6, 7, 100

vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float

# name -> (restype, argtypes); mirrors include/cwk_attn.h one to one
SIGNATURES = {
    "cwk_ctx_create": (i32, [i32, C.POINTER(vp)]),
    "cwk_ctx_destroy": (None, [vp]),
    "cwk_ctx_set_stream": (i32, [vp, vp]),
    "cwk_ctx_sync": (i32, [vp]),
    "cwk_last_error": (C.c_char_p, [vp]),
    "cwk_ctx_launch_count": (C.c_uint64, [vp]),
    "cwk_ctx_sm_count": (i32, [vp]),
    "cwk_ctx_profile": (i32, [vp, i32]),
    "cwk_ctx_profile_read": (i32, [vp, C.POINTER(C.c_double), C.POINTER(i32)]),
    "cwk_ctx_set_wait_limit": (i32, [vp, C.c_uint32]),
    "cwk_ctx_weight_cache": (i32, [vp, C.c_size_t]),
    "cwk_mla_decode_path": (i32, [vp, i32, i32, i32]),
    "cwk_ctx_force_mla_path": (i32, [vp, i32]),
    "cwk_mla_decode_parked_records": (i32, [vp, C.POINTER(C.c_uint64)]),
    "cwk_mla_decode": (i32, [vp, vp, vp, i64, i64, vp, i32, vp, i64, i32, i32, i32, i32, f32, vp, i32]),
    "cwk_mla_decode_host": (i32, [vp, vp, vp, i64, i64, vp, vp, i64, i32, i32, i32, i32, f32, vp, i32]),
    "cwk_mla_decode_noalloc": (i32, [vp, vp, vp, i64, i64, vp, i32, i32, i32, f32, vp, C.c_char_p, C.c_size_t]),
    "cwk_mla_decode_partial": (i32, [vp, vp, vp, i64, i64, i64, i32, i32, i32, f32, vp]),
    "cwk_lse_combine": (i32, [vp, vp, i32, i32, i32, vp]),
    "cwk_xchg_create": (i32, [vp, i32, i32, i32, C.POINTER(vp), C.POINTER(C.c_size_t)]),
    "cwk_xchg_export": (i32, [vp, vp, vp]),
    "cwk_xchg_open": (i32, [vp, vp, C.POINTER(vp)]),
    "cwk_xchg_close": (i32, [vp, vp]),
    "cwk_xchg_destroy": (i32, [vp, vp]),
    "cwk_mla_decode_kv_split": (i32, [vp, vp, vp, i64, i64, i32, i32, i32, f32, C.POINTER(vp), i32, i32, C.c_uint32, vp]),
    "cwk_indexer_scores_fp8": (i32, [vp, vp, vp, i64, vp, vp, vp, i32, i32, i32, i32, vp]),
    "cwk_topk_select": (i32, [vp, vp, i64, vp, i32, i32, i32, i32, vp, i64, vp]),
    "cwk_dsa_select": (i32, [vp, vp, vp, i64, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, i64, vp, vp]),
    "cwk_gqa_decode": (i32, [vp, vp, vp, vp, i64, vp, i32, i32, i32, i32, i32, f32, vp, i32]),
    "cwk_gqa_prefill": (i32, [vp, vp, vp, vp, i64, i32, i32, i32, i32, f32, vp]),
    "cwk_gqa_qk_prep": (i32, [vp, vp, vp, vp, vp, vp, f32, i32, C.c_double, i64, i32, i32, i32, i32, vp, vp, vp]),
    "cwk_gqa_gate": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "cwk_indexer_pool_compress": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, vp]),
    "cwk_ds_sparse_attn": (i32, [vp, vp, vp, vp, i32, i32, i32, vp, f32, vp]),
    "cwk_ds_indexer_scores": (i32, [vp, vp, vp, vp, i32, i32, i32, vp]),
    "cwk_ds_topk": (i32, [vp, vp, i64, vp, i32, i32, vp, i64, vp]),
    "cwk_ds_lin_q": (i32, [vp, vp, vp, vp, i64, i64, vp]),
    "cwk_mla_unabsorb": (i32, [vp, vp, vp, i64, i32, i32, vp]),
    "cwk_cache_export_f32": (i32, [vp, vp, i64, i64, i32, vp]),
    "cwk_cache_import_f32": (i32, [vp, vp, i64, i32, vp, i64, i32]),
    "cwk_cache_copy_bf16": (i32, [vp, i32, vp, vp, i64, i64, i32]),
    "cwk_ds_state_bytes": (C.c_size_t, [vp, i64]),
    "cwk_ds_state_pack": (i32, [vp, vp, i64, vp, C.c_size_t]),
    "cwk_ds_state_apply": (i32, [vp, vp, vp, C.c_size_t, C.POINTER(i64)]),
    "cwk_q35_prefix_bytes": (C.c_size_t, [vp, i64]),
    "cwk_q35_prefix_pack": (i32, [vp, vp, i64, vp, C.c_size_t]),
    "cwk_q35_prefix_apply": (i32, [vp, vp, vp, C.c_size_t, i64, C.POINTER(i64)]),
    "cwk_gdn_scan": (i32, [vp, i32, i32, i32, i32, i32, i32] + [vp] * 7 + [f32, vp, vp]),
    "cwk_mm_index_scores": (i32, [vp, vp, i64, i32, vp, i32, vp]),
    "cwk_mm_select_blocks": (i32, [vp, vp, i64, i32, i32, i32, vp, vp, vp, vp]),
    "cwk_gqa_decode_sel": (i32, [vp, vp, vp, vp, i64, vp, i32, vp, i64, i32, i32, i32, i32, f32, vp, i32]),
    "cwk_kda_step": (i32, [vp, i32, i32, i32, f32, f32] + [vp] * 15),
    "cwk_ds_pool_norm": (i32, [vp, vp, vp, i32, i32, i32, vp, f32, vp]),
    "cwk_ds_rmsnorm_bf16w": (i32, [vp, vp, vp, i32, i32, f32, vp]),
    "cwk_ds_rope_round_qdq": (i32, [vp, vp, i32, i32, vp, i32, i64, i32, i32]),
    "cwk_ds_kv_row_store": (i32, [vp, vp, i32, vp, i32, i64, vp, i32]),
    "cwk_ds_out_unrope": (i32, [vp, vp, i32, i32, vp, i32, i64]),
    "cwk_ds_candidates": (i32, [vp, vp, i32, i32, i32, vp]),
    "cwk_ds_mask_candidates": (i32, [vp, vp, vp, i32]),
    "cwk_mla_prefill": (i32, [vp] * 12 + [i64] + [i32] * 7 + [f32, f32, f32, vp]),
    "cwk_fp8_linear": (i32, [vp, vp, vp, vp, i64, i64, i64, vp, i32]),
}

# reference-named entry points (include/cwick_compat.h); bound separately because their
# arguments are the reference's structs
COMPAT_SYMBOLS = ["cwick_attention_mla_decode", "cwick_mla_latent_enabled", "cwick_indexer_active",
                  "cwick_latent_bf16_enabled", "cwick_latent_elem_bytes", "cwk_dropin_reset",
                  "cwick_indexer_bytes", "cwick_indexer_reset", "cwick_mla_chunk_supported",
                  "cwick_attention_mla_prefill_chunk", "cwick_attention_kda_decode"]

_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m cwick_b200.build` "
                "(there is no fallback implementation)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError if the header and the library drift
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class CwkError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"cwk status {status}: {msg}")
        self.status = status


class Context:
    """One cwk_ctx: a device, a stream, split scratch."""

    def __init__(self, device=0, stream=None):
        self.lib = load()
        h = vp()
        st = self.lib.cwk_ctx_create(device, C.byref(h))
        if st != OK:
            raise CwkError(st, "cwk_ctx_create failed (no CUDA device, or not an sm_100 part)")
        self.h = h
        if stream is not None:
            self.check(self.lib.cwk_ctx_set_stream(self.h, vp(stream)))

    def check(self, st):
        if st != OK:
            raise CwkError(st, self.lib.cwk_last_error(self.h).decode())

    def sync(self):
        self.check(self.lib.cwk_ctx_sync(self.h))

    @property
    def launches(self):
        return int(self.lib.cwk_ctx_launch_count(self.h))

    @property
    def sm_count(self):
        return int(self.lib.cwk_ctx_sm_count(self.h))

    def profile(self, on):
        self.check(self.lib.cwk_ctx_profile(self.h, 1 if on else 0))

    def profile_read(self):
        """(summed main-kernel milliseconds, bracketed launches) since the last read."""
        ms, n = C.c_double(0.0), i32(0)
        self.check(self.lib.cwk_ctx_profile_read(self.h, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def close(self):
        if getattr(self, "h", None):
            self.lib.cwk_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
