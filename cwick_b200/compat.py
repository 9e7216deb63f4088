"""ctypes mirrors of the reference's structs as the reference-named entry points take them (include/cwick_compat.h,
src/cwick.h:864-938): a weight tensor, the error record, and a model spec as a raw buffer with the fields the attention
entry points read poked at their offsets. Used by the drop-in tests and by bench.py's drop-in timing."""
import ctypes as C


class Tensor(C.Structure):
    _fields_ = [("rows", C.c_int64), ("cols", C.c_int64), ("kind", C.c_int), ("data", C.c_void_p),
                ("scales", C.c_void_p), ("data_bytes", C.c_size_t), ("scale_bytes", C.c_size_t), ("name", C.c_char * 128)]


class Err(C.Structure):
    _fields_ = [("status", C.c_int), ("message", C.c_char * 512)]


SPEC_BYTES = 1024   # larger than the reference struct; fields are poked at their offsets


def spec_offsets():
    """Offsets of the fields the entry point reads, from the mirrored header's member order."""
    # model_type[64] dtype[16] bos eos eos_ids[8] n_eos(+pad) pad_token | hidden ...
    off = {}
    o = 64 + 16 + 8 + 8 + 64 + 8 + 8
    for name in ("hidden_size", "intermediate_size", "num_hidden_layers", "vocab_size", "max_position_embeddings",
                 "rms_norm_eps", "num_attention_heads", "num_key_value_heads", "head_dim", "q_lora_rank", "kv_lora_rank",
                 "qk_nope_head_dim", "qk_rope_head_dim", "value_head_dim"):
        off[name] = o
        o += 8
    o += 8                      # bool mla_use_output_gate + padding
    o += 8 * 3 + 8 + 8 * 7      # linear_*, attn_res_block_size, MoE geometry
    o += 4                      # two bools + padding to float alignment
    o += 4 * 5
    off["rms_norm_eps_f"] = o
    return off


def make_spec(H, nh, nope, vdim, q_lora, kv_lora, eps):
    buf = (C.c_uint8 * SPEC_BYTES)()
    off = spec_offsets()
    for k, v in dict(hidden_size=H, num_attention_heads=nh, num_key_value_heads=nh, q_lora_rank=q_lora,
                     kv_lora_rank=kv_lora, qk_nope_head_dim=nope, qk_rope_head_dim=0, value_head_dim=vdim).items():
        C.c_int64.from_buffer(buf, off[k]).value = v
    C.c_float.from_buffer(buf, off["rms_norm_eps_f"]).value = eps
    return buf


def tensor(arr, rows, cols):
    t = Tensor()
    t.rows, t.cols, t.kind, t.data = rows, cols, 1, arr.ctypes.data
    t.data_bytes = arr.nbytes
    return t


def tensor_fp8(codes, scales, rows, cols):
    """An FP8-E4M3 weight: uint8 codes [rows][cols] and one f32 multiplier per 128 x 128 block [rows/128][cols/128]."""
    t = Tensor()
    t.rows, t.cols, t.kind, t.data, t.scales = rows, cols, 4, codes.ctypes.data, scales.ctypes.data
    t.data_bytes, t.scale_bytes = codes.nbytes, scales.nbytes
    return t

