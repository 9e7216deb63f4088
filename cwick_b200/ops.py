"""Tensor-level mirror of the C entry points, for tests and the benchmark.

torch is used for device memory and streams only; every computation is a call
into libcwk_attn.so through `lib.Context`. Argument names and meanings follow
include/cwk_attn.h.
"""
import math

import torch

from . import lib as _lib


def _p(t):
    return None if t is None else _lib.vp(t.data_ptr())


def _bf16(t):
    assert t.dtype == torch.bfloat16 and t.is_cuda and t.is_contiguous()
    return t


class Attn:
    def __init__(self, device=0):
        torch.cuda.set_device(device)
        self.device = device
        self.ctx = _lib.Context(device, stream=torch.cuda.current_stream(device).cuda_stream)
        self.lib = self.ctx.lib

    # ---- MLA ---------------------------------------------------------------
    def mla_decode(self, q, cache, kv_len, max_kv_len=None, sel=None, scale=None, seq_stride=None,
                   n_splits=0, out=None):
        """q [B][nh][L+R] bf16; cache [B][rows][ld] or [rows][ld] bf16 (then seq_stride 0);
        kv_len int32 [B] cuda; sel optional int32 [B][sel_ld] cuda. Returns [B][nh][L] bf16."""
        _bf16(q), _bf16(cache)
        B, nh, dk = q.shape
        ld = cache.shape[-1]
        R = 64 if dk == 576 else 0
        L = dk - R
        if seq_stride is None:
            seq_stride = cache.shape[-2] * ld if cache.dim() == 3 else 0
        if max_kv_len is None:
            max_kv_len = int(kv_len.max().item())
        if scale is None:
            scale = 1.0 / math.sqrt(192.0 if R else L)
        if out is None:
            out = torch.empty(B, nh, L, dtype=torch.bfloat16, device=q.device)
        sel_ld = sel.shape[-1] if sel is not None else 0
        self.ctx.check(self.lib.cwk_mla_decode(self.ctx.h, _p(q), _p(cache), seq_stride, ld, _p(kv_len),
                                               max_kv_len, _p(sel), sel_ld, B, nh, L, R, scale, _p(out),
                                               n_splits))
        return out

    def mla_decode_dims(self, q, cache, kv_len, L, R, scale, max_kv_len=None, sel=None, seq_stride=None,
                        n_splits=0):
        """As mla_decode with explicit (L, R)."""
        _bf16(q), _bf16(cache)
        B, nh, dk = q.shape
        assert dk == L + R
        ld = cache.shape[-1]
        if seq_stride is None:
            seq_stride = cache.shape[-2] * ld if cache.dim() == 3 else 0
        if max_kv_len is None:
            max_kv_len = int(kv_len.max().item())
        out = torch.empty(B, nh, L, dtype=torch.bfloat16, device=q.device)
        sel_ld = sel.shape[-1] if sel is not None else 0
        self.ctx.check(self.lib.cwk_mla_decode(self.ctx.h, _p(q), _p(cache), seq_stride, ld, _p(kv_len),
                                               max_kv_len, _p(sel), sel_ld, B, nh, L, R, scale, _p(out),
                                               n_splits))
        return out

    def mla_decode_host(self, q_host, cache, kv_len_host, L, R, scale, out_host, sel_host=None, seq_stride=None,
                        n_splits=0):
        """q_host/out_host/kv_len_host: CPU tensors (any memory); cache: cuda bf16."""
        B, nh, dk = q_host.shape
        ld = cache.shape[-1]
        if seq_stride is None:
            seq_stride = cache.shape[-2] * ld if cache.dim() == 3 else 0
        sel_ld = sel_host.shape[-1] if sel_host is not None else 0
        self.ctx.check(self.lib.cwk_mla_decode_host(
            self.ctx.h, _p(q_host), _p(cache), seq_stride, ld, _p(kv_len_host), _p(sel_host), sel_ld, B, nh,
            L, R, scale, _p(out_host), n_splits))
        return out_host

    def mla_decode_partial(self, q, cache, row0, rows, L, R, scale, partial=None):
        """q [nh][L+R] bf16, cache [rows_total][ld] bf16 -> f32 [nh*(L+2)] un-normalised record."""
        nh = q.shape[-2]
        if partial is None:
            partial = torch.empty(nh * (L + 2), dtype=torch.float32, device=q.device)
        self.ctx.check(self.lib.cwk_mla_decode_partial(self.ctx.h, _p(q), _p(cache), cache.shape[-1], row0,
                                                       rows, nh, L, R, scale, _p(partial)))
        return partial

    def lse_combine(self, partials, nh, L):
        G = partials.shape[0]
        out = torch.empty(nh, L, dtype=torch.bfloat16, device=partials.device)
        self.ctx.check(self.lib.cwk_lse_combine(self.ctx.h, _p(partials), G, nh, L, _p(out)))
        return out

    # ---- DSA -----------------------------------------------------------------
    def indexer_scores_fp8(self, keys, kscale, q, wt, n, max_n=None):
        """keys uint8 [B][T][hd]; kscale f32 [B][T]; q f32 [B][ih][hd]; wt f32 [B][ih]; n int32 [B]."""
        B, T, hd = keys.shape
        ih = q.shape[1]
        if max_n is None:
            max_n = int(n.max().item())
        sc = torch.zeros(B, T, dtype=torch.float32, device=keys.device)
        self.ctx.check(self.lib.cwk_indexer_scores_fp8(self.ctx.h, _p(keys), _p(kscale), T, _p(q), _p(wt), _p(n),
                                                       max_n, B, ih, hd, _p(sc)))
        return sc

    def topk_select(self, sc, n, want, keep_self=False, max_n=None):
        B, T = sc.shape
        sel = torch.full((B, want + 1), -1, dtype=torch.int32, device=sc.device)
        nsel = torch.zeros(B, dtype=torch.int32, device=sc.device)
        self.ctx.check(self.lib.cwk_topk_select(self.ctx.h, _p(sc), T, _p(n), max_n or T, B, want,
                                                1 if keep_self else 0, _p(sel), want + 1, _p(nsel)))
        return sel, nsel

    def dsa_select(self, keys, kscale, q, wt, n, want, keep_self=False, max_n=None, return_scores=False):
        """Indexer scores and exact top-`want` in one call (tensor-core scores, exact re-scoring around
        the threshold). Returns (sel int32 [B][want+1], nsel int32 [B]) and, on request, the refined
        score array."""
        B, T, hd = keys.shape
        ih = q.shape[1]
        if max_n is None:
            max_n = int(n.max().item())
        sel = torch.full((B, want + 1), -1, dtype=torch.int32, device=keys.device)
        nsel = torch.zeros(B, dtype=torch.int32, device=keys.device)
        sc = torch.zeros(B, T, dtype=torch.float32, device=keys.device) if return_scores else None
        self.ctx.check(self.lib.cwk_dsa_select(self.ctx.h, _p(keys), _p(kscale), T, _p(q), _p(wt), _p(n), max_n, B, ih, hd,
                                               want, 1 if keep_self else 0, _p(sel), want + 1, _p(nsel),
                                               _p(sc) if sc is not None else None))
        return (sel, nsel, sc) if return_scores else (sel, nsel)

    # ---- GQA -----------------------------------------------------------------
    def gqa_decode(self, q, K, V, kv_len, scale=None, max_kv_len=None, n_splits=0, out=None):
        """q [B][nh][hd]; K,V [B][T][nkv][hd] bf16; kv_len int32 [B]."""
        _bf16(q), _bf16(K), _bf16(V)
        B, nh, hd = q.shape
        T, nkv = K.shape[1], K.shape[2]
        if scale is None:
            scale = 1.0 / math.sqrt(hd)
        if max_kv_len is None:
            max_kv_len = int(kv_len.max().item())
        if out is None:
            out = torch.empty(B, nh, hd, dtype=torch.bfloat16, device=q.device)
        self.ctx.check(self.lib.cwk_gqa_decode(self.ctx.h, _p(q), _p(K), _p(V), T * nkv * hd, _p(kv_len),
                                               max_kv_len, B, nh, nkv, hd, scale, _p(out), n_splits))
        return out

    def gqa_prefill(self, Q, K, V, pos, scale=None):
        """Q [n][nh][hd]; K,V [pos+n][nkv][hd] bf16."""
        _bf16(Q), _bf16(K), _bf16(V)
        n, nh, hd = Q.shape
        nkv = K.shape[1]
        if scale is None:
            scale = 1.0 / math.sqrt(hd)
        out = torch.empty(n, nh, hd, dtype=torch.bfloat16, device=Q.device)
        self.ctx.check(self.lib.cwk_gqa_prefill(self.ctx.h, _p(Q), _p(K), _p(V), pos, n, nh, nkv, hd, scale,
                                                _p(out)))
        return out

    # ---- FP8 projection ------------------------------------------------------------
    def fp8_linear(self, X, W, scale_inv, out_bf16=False):
        """X [n][k] bf16; W uint8 [cols][k] (E4M3 codes); scale_inv f32 [cols/128][k/128]."""
        n, k = X.shape
        cols = W.shape[0]
        Y = torch.empty(n, cols, dtype=torch.bfloat16 if out_bf16 else torch.float32, device=X.device)
        self.ctx.check(self.lib.cwk_fp8_linear(self.ctx.h, _p(X), _p(W), _p(scale_inv), n, k, cols, _p(Y),
                                               1 if out_bf16 else 0))
        return Y

    def mla_unabsorb(self, attn_out, Wv, head_rows=128):
        """attn_out bf16 [n][nh][512]; Wv bf16, head h's [128][512] at row h * head_rows. Returns bf16 [n][nh*128]
        (src/attention.c:812-815 batched over tokens: the input rows of o_proj)."""
        _bf16(attn_out), _bf16(Wv)
        n, nh, _ = attn_out.shape
        out = torch.empty(n, nh * 128, dtype=torch.bfloat16, device=attn_out.device)
        self.ctx.check(self.lib.cwk_mla_unabsorb(self.ctx.h, _p(attn_out), _p(Wv), head_rows, n, nh, _p(out)))
        return out

    # ---- MLA prefill -----------------------------------------------------------------
    def mla_prefill(self, X, Wqa, Sqa, Wqb, Sqb, Wkva, Skva, qa_norm, kva_norm, Wuk, cache, pos0, nh,
                    nope=128, rope=64, kv_lora=512, eps=1e-6, rope_base=10000.0, scale=None):
        """X bf16 [n][H]; weights uint8 E4M3 + f32 scales; norms bf16; Wuk bf16 [nh][nope][kv_lora];
        cache bf16 [rows][kv_lora+rope] (rows pos0..pos0+n-1 written). Returns bf16 [n][nh][kv_lora]."""
        n, H = X.shape
        q_lora = Wqa.shape[0]
        if scale is None:
            scale = 1.0 / math.sqrt(nope + rope)
        out = torch.empty(n, nh, kv_lora, dtype=torch.bfloat16, device=X.device)
        self.ctx.check(self.lib.cwk_mla_prefill(
            self.ctx.h, _p(X), _p(Wqa), _p(Sqa), _p(Wqb), _p(Sqb), _p(Wkva), _p(Skva), _p(qa_norm), _p(kva_norm),
            _p(Wuk), _p(cache), pos0, n, H, q_lora, nh, nope, rope, kv_lora, eps, rope_base, scale, _p(out)))
        return out

    # ---- linear-attention layers and the sparse variants next to the MLA path ------------
    def kda_step(self, q, k, v, q_conv, k_conv, v_conv, conv, gate_raw, dt_bias, a_log, beta_raw, gate, o_norm, rec,
                 lower, rms_eps):
        """One KDA decode step for B slots (cwk_kda_step): q, k, v, gate_raw, gate f32 [B][nh*hd]; beta_raw f32 [B][nh];
        conv f32 [B][3][nh*hd][3] and rec f32 [B][nh][hd][hd] are updated in place. Returns core f32 [B][nh*hd]."""
        B, nh, hd, _ = rec.shape
        core = torch.empty(B, nh * hd, dtype=torch.float32, device=q.device)
        self.ctx.check(self.lib.cwk_kda_step(self.ctx.h, B, nh, hd, lower, rms_eps, _p(q), _p(k), _p(v), _p(q_conv), _p(k_conv),
                                             _p(v_conv), _p(conv), _p(gate_raw), _p(dt_bias), _p(a_log), _p(beta_raw), _p(gate),
                                             _p(o_norm), _p(rec), _p(core)))
        return core

    def gdn_scan(self, up, gdec, beta, gate, a_log, dt_bias, norm, S, kv_group, rms_eps):
        """Gated DeltaNet scan (cwk_gdn_scan): up f32 [B][n][2*key_dim + val_dim]; gdec, beta f32 [B][n][nh]; gate f32
        [B][n][val_dim]; S f32 [B][nh][head_v][head_k] updated in place. Returns f32 [B][n][val_dim]."""
        B, n, _ = up.shape
        _, nh, hv, hk = S.shape
        out = torch.empty(B, n, nh * hv, dtype=torch.float32, device=up.device)
        self.ctx.check(self.lib.cwk_gdn_scan(self.ctx.h, B, n, nh, hk, hv, kv_group, _p(up), _p(gdec), _p(beta), _p(gate), _p(a_log),
                                             _p(dt_bias), _p(norm), rms_eps, _p(S), _p(out)))
        return out

    def mm_select(self, index_keys, iq, limit, block_size, topk_blocks, cap=4096):
        """MiniMax indexer for one query: index scores over bf16 keys [rows][id] (the first `limit` rows), then the
        positions of the selected blocks. Returns (sel int32 [cap], nsel int32 [1])."""
        _bf16(index_keys)
        ih, idim = iq.shape
        sc = torch.empty(limit, dtype=torch.float32, device=iq.device)
        self.ctx.check(self.lib.cwk_mm_index_scores(self.ctx.h, _p(index_keys), limit, idim, _p(iq), ih, _p(sc)))
        sel = torch.full((cap,), -1, dtype=torch.int32, device=iq.device)
        nsel = torch.zeros(1, dtype=torch.int32, device=iq.device)
        self.ctx.check(self.lib.cwk_mm_select_blocks(self.ctx.h, _p(sc), limit, block_size, topk_blocks, cap, _p(sel), _p(nsel), None, None))
        return sel, nsel

    def gqa_decode_sel(self, q, K, V, sel, nsel, max_nsel, scale=None, n_splits=0):
        """GQA decode over the rows sel[b][0:nsel[b]] of each sequence's cache (cwk_gqa_decode_sel)."""
        _bf16(q), _bf16(K), _bf16(V)
        B, nh, hd = q.shape
        T, nkv = K.shape[1], K.shape[2]
        if scale is None:
            scale = 1.0 / math.sqrt(hd)
        out = torch.empty_like(q)
        self.ctx.check(self.lib.cwk_gqa_decode_sel(self.ctx.h, _p(q), _p(K), _p(V), T * nkv * hd, _p(nsel), max_nsel, _p(sel),
                                                   sel.shape[-1], B, nh, nkv, hd, scale, _p(out), n_splits))
        return out

