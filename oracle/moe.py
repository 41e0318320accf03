"""MoE block oracle: int8 W8A8 and fp8 block-scaled routed + shared experts, and the combine.

Test infrastructure only (see oracle/__init__.py).

Slot convention (i8x_decode.py:297,442): routed pair (token t, pick j) has slot t*K + j, the
shared expert's row for token t has slot T*K + t.  `cache[slot]` holds the bf16 down-projection
row already multiplied by its routing weight (i8x_decode.py:420-422); the combine adds the K
routed rows in slot order and the sigmoid-gated shared row (i8x_decode.py:425-443).
"""
from __future__ import annotations

import numpy as np

from .numerics import (F32, bf16_round, e4m3_decode, quant_fp8_groups, quant_int8_rows,
                       silu_mul_bf16)


def _expert_rows(ids: np.ndarray, valid):
    T, K = ids.shape
    ok = np.ones(T, dtype=bool) if valid is None else np.asarray(valid, dtype=bool)
    by = {}
    for t in range(T):
        if not ok[t]:
            continue
        for j in range(K):
            by.setdefault(int(ids[t, j]), []).append((t, t * K + j))
    return by


# ----------------------------------------------------------------------------------------------
# int8 W8A8  (per-token activation scale x per-output-channel weight scale)
# ----------------------------------------------------------------------------------------------
def mlp_int8(xq, xs, w13q, s13, w2q, s2, want_acc=False):
    """One expert's MLP on already-quantised rows.

    acc = int32 sum over the whole K (exact); value = (float(acc) * xs[row]) * ws[col], the
    reference's W8A8 epilogue order (qwen36_lmhead8/w8a8.py:64-70; qk_moe_prefill_i8.cu:3646-3655
    for the MoE twin).  SwiGLU rounds g, u and h to bf16 (i8x_decode.py:151-156).  h is
    re-quantised per row before the down GEMM (qk_moe_prefill_i8.cu:4061-4066).
    Returns y fp32 [rows, H] (not yet weighted / rounded), h (bf16 values), acc13 (int32) if asked.
    """
    I = w13q.shape[0] // 2
    acc13 = (xq.astype(np.float64) @ w13q.astype(np.float64).T)  # exact: |sum| < 2^53
    gu = ((acc13.astype(F32) * xs[:, None]).astype(F32) * s13[None, :]).astype(F32)
    h = silu_mul_bf16(gu[:, :I], gu[:, I:])
    hq, hs = quant_int8_rows(h)
    acc2 = hq.astype(np.float64) @ w2q.astype(np.float64).T
    y = ((acc2.astype(F32) * hs[:, None]).astype(F32) * s2[None, :]).astype(F32)
    if want_acc:
        return y, h, acc13.astype(np.int64).astype(np.int32), acc2.astype(np.int64).astype(np.int32)
    return y, h


def moe_int8(x, ids, wts, w13q, s13, w2q, s2, sh13q, shs13, sh2q, shs2, gate_w, valid=None,
             want_debug=False):
    """Whole int8 MoE block.  x: bf16 values [T, H]; ids/wts from the router; w13q int8 [E, 2I, H],
    s13 fp32 [E, 2I]; w2q int8 [E, H, I], s2 fp32 [E, H]; shared expert likewise without the E
    axis; gate_w bf16 values [H].  Returns out (bf16 values, fp32 array [T, H]) and, if asked,
    dict(h, cache, acc13, xq, xs)."""
    x = np.asarray(x, dtype=F32)
    T, H = x.shape
    K = ids.shape[1]
    I = w2q.shape[-1]
    xq, xs = quant_int8_rows(x)
    cache = np.zeros((T * (K + 1), H), dtype=F32)
    hbuf = np.zeros((T * (K + 1), I), dtype=F32)
    accbuf = np.zeros((T * (K + 1), 2 * I), dtype=np.int32) if want_debug else None
    flatw = np.asarray(wts, dtype=F32).reshape(-1)
    for e, rows in sorted(_expert_rows(np.asarray(ids), valid).items()):
        tok = np.array([r[0] for r in rows])
        slot = np.array([r[1] for r in rows])
        res = mlp_int8(xq[tok], xs[tok], w13q[e], s13[e], w2q[e], s2[e], want_acc=want_debug)
        y, h = res[0], res[1]
        cache[slot] = bf16_round((y * flatw[slot][:, None]).astype(F32))
        hbuf[slot] = h
        if want_debug:
            accbuf[slot] = res[2]
    ok = np.ones(T, dtype=bool) if valid is None else np.asarray(valid, dtype=bool)
    tok = np.nonzero(ok)[0]
    res = mlp_int8(xq[tok], xs[tok], sh13q, shs13, sh2q, shs2, want_acc=want_debug)
    cache[T * K + tok] = bf16_round(res[0])
    hbuf[T * K + tok] = res[1]
    if want_debug:
        accbuf[T * K + tok] = res[2]
    out = combine(cache, x, gate_w, K, valid)
    if want_debug:
        return out, dict(h=hbuf, cache=cache, acc13=accbuf, xq=xq, xs=xs)
    return out


# ----------------------------------------------------------------------------------------------
# fp8 e4m3, 128 x 128 weight blocks, per-(token, 128-channel) activation scales
# ----------------------------------------------------------------------------------------------
def gemm_fp8_blocks(aq, a_s, wq, w_s):
    """out[m, n] = sum over 128-k blocks g, in increasing g, of fma(partial_g[m, n], a_s[m, g] *
    w_s[n // 128, g], acc), acc starting at 0; partial_g is the block's own dot product started from
    zero.  This is the promotion order the reference documents for its scaled GEMMs ("per 128-k
    block a chain from zero, fp32 adds in k order": qk_lt.cu:361-364; the int8 twin
    `acc = fmaf(float(s32), sa[row,g]*sb[col,g], acc)`: qk_moe_prefill_i8.cu:3649-3651).
    The tensor core forms partial_g with its own internal accumulation, so the block dot is
    taken in float64 and rounded once to fp32 here; comparisons use the bf16 tolerance.
    aq uint8 e4m3 codes [M, K], a_s fp32 [M, K/128]; wq uint8 [N, K], w_s fp32 [N/128, K/128]."""
    M, K = aq.shape
    N = wq.shape[0]
    a = e4m3_decode(aq).astype(np.float64).reshape(M, K // 128, 128)
    w = e4m3_decode(wq).astype(np.float64).reshape(N, K // 128, 128)
    acc = np.zeros((M, N), dtype=F32)
    ws_full = np.repeat(np.asarray(w_s, dtype=F32), 128, axis=0)[:N]  # [N, K/128]; N may end inside a block
    for g in range(K // 128):
        part = (a[:, g, :] @ w[:, g, :].T).astype(F32)
        sc = (a_s[:, g][:, None] * ws_full[:, g][None, :]).astype(F32)
        acc = (part.astype(np.float64) * sc.astype(np.float64) + acc.astype(np.float64)).astype(F32)
    return acc


def mlp_fp8(xq, xs, w13q, s13, w2q, s2):
    I = w13q.shape[0] // 2
    gu = gemm_fp8_blocks(xq, xs, w13q, s13)
    h = silu_mul_bf16(gu[:, :I], gu[:, I:])
    hq, hs = quant_fp8_groups(h)
    y = gemm_fp8_blocks(hq, hs, w2q, s2)
    return y, h


def moe_fp8(x, ids, wts, w13q, s13, w2q, s2, sh13q, shs13, sh2q, shs2, gate_w, valid=None,
            want_debug=False):
    """Whole fp8 MoE block.  w13q uint8 e4m3 codes [E, 2I, H], s13 fp32 [E, 2I/128, H/128];
    w2q [E, H, I], s2 [E, H/128, I/128]; shared expert likewise without E."""
    x = np.asarray(x, dtype=F32)
    T, H = x.shape
    K = ids.shape[1]
    I = w2q.shape[-1]
    xq, xs = quant_fp8_groups(x)
    cache = np.zeros((T * (K + 1), H), dtype=F32)
    hbuf = np.zeros((T * (K + 1), I), dtype=F32)
    flatw = np.asarray(wts, dtype=F32).reshape(-1)
    for e, rows in sorted(_expert_rows(np.asarray(ids), valid).items()):
        tok = np.array([r[0] for r in rows])
        slot = np.array([r[1] for r in rows])
        y, h = mlp_fp8(xq[tok], xs[tok], w13q[e], s13[e], w2q[e], s2[e])
        cache[slot] = bf16_round((y * flatw[slot][:, None]).astype(F32))
        hbuf[slot] = h
    ok = np.ones(T, dtype=bool) if valid is None else np.asarray(valid, dtype=bool)
    tok = np.nonzero(ok)[0]
    y, h = mlp_fp8(xq[tok], xs[tok], sh13q, shs13, sh2q, shs2)
    cache[T * K + tok] = bf16_round(y)
    hbuf[T * K + tok] = h
    out = combine(cache, x, gate_w, K, valid)
    if want_debug:
        return out, dict(h=hbuf, cache=cache, xq=xq, xs=xs)
    return out


# ----------------------------------------------------------------------------------------------
# combine
# ----------------------------------------------------------------------------------------------
def combine(cache, x, gate_w, top_k, valid=None):
    """out[t] = bf16(sum_{j<K} cache[t*K + j] (fp32, slot order) + sigmoid(x[t] . gate_w) *
    cache[T*K + t]); padding rows give zeros (`i8x_dec_combine`, i8x_decode.py:425-443)."""
    x = np.asarray(x, dtype=F32)
    T, H = x.shape
    dot = (x.astype(np.float64) @ np.asarray(gate_w, dtype=np.float64)).astype(F32)
    gate = (F32(1.0) / (F32(1.0) + np.exp(-dot, dtype=F32))).astype(F32)
    acc = np.zeros((T, H), dtype=F32)
    for j in range(top_k):
        acc = (acc + cache[np.arange(T) * top_k + j]).astype(F32)
    acc = (acc + gate[:, None] * cache[T * top_k + np.arange(T)]).astype(F32)
    out = bf16_round(acc)
    if valid is not None:
        out = np.where(np.asarray(valid, dtype=bool)[:, None], out, F32(0.0))
    return out
