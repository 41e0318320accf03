"""Oracles for the fused gated-attention projection front and the vocab-sharded LM head.

Test infrastructure only (see oracle/__init__.py).  PARITY UNPINNED by the reference for the
fp8 128x128 block-scaled GEMM and for the argmax (the reference has neither); the norm / RoPE /
e4m3 front follows the reference's kernel line by line.
"""
from __future__ import annotations

import numpy as np

from .moe import gemm_fp8_blocks
from .numerics import F32, bf16_round, e4m3_encode, quant_fp8_groups

HQ, HKV, HD, ROT = 16, 2, 256, 64
QG_COLS = HQ * 2 * HD          # 8192: per head [q 256 | gate 256]  (qk_attn_verify.cu:25,443,450)
K_COL0 = QG_COLS               # 8192
V_COL0 = QG_COLS + HKV * HD    # 8704
N_COLS = QG_COLS + 2 * HKV * HD  # 9216


def rope_table(max_pos: int, theta: float = 1e7, rot: int = ROT) -> np.ndarray:
    """[max_pos, rot] fp32 laid out [cos_0..cos_{rot/2-1} | sin_0..sin_{rot/2-1}], the cache layout
    the reference reads (qk_attn_verify.cu:167-175); angle(pos, i) = pos * theta^(-2i/rot)."""
    half = rot // 2
    inv = np.power(np.float64(theta), -2.0 * np.arange(half, dtype=np.float64) / rot)
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * inv[None, :]
    return np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(F32)


def norm_rope(xh, w, cs, eps):
    """One head row block: xh [T, 256] bf16 values, w [256] bf16 values, cs [T, 64] fp32.
    inv = rsqrt(sum x^2 / 256 + eps); x = bf16(x * inv * (w + 1)); neox rotation of dims (i, i+32),
    i < 32: bf16(x_i c - x_{i+32} s), bf16(x_{i+32} c + x_i s); dims 64..255 pass through
    (`norm_rope_e4m3`, qk_attn_verify.cu:180-208)."""
    ss = np.sum(xh * xh, axis=-1, keepdims=True, dtype=F32)
    inv = (F32(1.0) / np.sqrt(ss / F32(HD) + F32(eps))).astype(F32)
    y = bf16_round(((xh * inv).astype(F32) * (w[None, :] + F32(1.0))).astype(F32))
    half = ROT // 2
    c, s = cs[:, :half], cs[:, half:]
    lo, hi = y[:, :half].copy(), y[:, half:ROT].copy()
    y[:, :half] = bf16_round(((lo * c).astype(F32) - (hi * s).astype(F32)).astype(F32))
    y[:, half:ROT] = bf16_round(((hi * c).astype(F32) + (lo * s).astype(F32)).astype(F32))
    return y


def attn_front(x, wq, w_s, q_norm_w, k_norm_w, positions, cos_sin, eps=1e-6, out_fp8=True):
    """Fused QKV + gate projection with q/k RMSNorm and partial RoPE.

    x bf16 values [T, 2048] is quantised per token per 128 channels; W e4m3 codes [9216, 2048]
    with block scales [72, 16]; the GEMM result is rounded to bf16 (the reference's projection
    writes bf16 before its front kernel reads it: qk_lt.cu:361-364, qk_attn_verify.cu:765-800).
    Column layout per q head h: q at h*512, gate at h*512 + 256; K at 8192, V at 8704.
    Returns q [T, 16, 256], gate [T, 16, 256] (bf16 values), k, v [T, 2, 256]; q, k, v are e4m3
    codes (uint8, cvt.rn.satfinite: qk_attn_verify.cu:142-146,207,793) when out_fp8 else bf16 values.
    """
    x = np.asarray(x, dtype=F32)
    T = x.shape[0]
    xq, xs = quant_fp8_groups(x)
    y = bf16_round(gemm_fp8_blocks(xq, xs, wq, w_s))
    cs = np.asarray(cos_sin, dtype=F32)[np.asarray(positions)]
    qg = y[:, :QG_COLS].reshape(T, HQ, 2, HD)
    gate = qg[:, :, 1, :].copy()
    q = np.empty((T, HQ, HD), dtype=F32)
    for h in range(HQ):
        q[:, h] = norm_rope(qg[:, h, 0, :].copy(), np.asarray(q_norm_w, dtype=F32), cs, eps)
    kk = y[:, K_COL0:V_COL0].reshape(T, HKV, HD)
    k = np.empty((T, HKV, HD), dtype=F32)
    for h in range(HKV):
        k[:, h] = norm_rope(kk[:, h].copy(), np.asarray(k_norm_w, dtype=F32), cs, eps)
    v = y[:, V_COL0:].reshape(T, HKV, HD).copy()
    if out_fp8:
        return e4m3_encode(q), gate, e4m3_encode(k), e4m3_encode(v)
    return q, gate, k, v


def lmhead_logits(x, wq, w_s):
    """fp32 logits [T, V_shard] of one vocab shard: activations e4m3 per (token, 128), weights e4m3
    with 128x128 block scales, promotion per 128-k block (see gemm_fp8_blocks).  The reference's
    LM head is the same swap-AB weight-streaming GEMM in int8 (qwen36_lmhead8/lmhead8.py:56-91,
    w8a8.py:38-75); it scales once at the end, which a block-scaled format cannot."""
    xq, xs = quant_fp8_groups(np.asarray(x, dtype=F32))
    return gemm_fp8_blocks(xq, xs, wq, w_s)


def shard_argmax(logits, shard_lo=0):
    """(max fp32, global argmax int32) per row; ties go to the lower id; NaN never wins.
    The reference returns logits and has no argmax (qwen36_lmhead8/node.py:136-151)."""
    lg = np.where(np.isnan(logits), -np.inf, logits).astype(F32)
    idx = np.argmax(lg, axis=1)  # first occurrence = lowest id
    return lg[np.arange(lg.shape[0]), idx], (idx + shard_lo).astype(np.int32)


def merge_argmax(maxes, idxs):
    """Merge per-shard pairs [S, T]: the largest value wins, ties go to the lower global id."""
    maxes = np.asarray(maxes, dtype=F32)
    idxs = np.asarray(idxs, dtype=np.int64)
    best = np.max(maxes, axis=0)
    cand = np.where(maxes == best[None, :], idxs, np.iinfo(np.int64).max)
    return np.min(cand, axis=0).astype(np.int32)


def vocab_shards(vocab: int, world: int, block: int = 128):
    """Row ranges per rank, cut on 128-row scale-block boundaries: the first (blocks % world) ranks
    take one block more.  151936 rows / 8 ranks -> 3 x 19072 + 5 x 18944."""
    nb = (vocab + block - 1) // block
    base, extra = divmod(nb, world)
    out, lo = [], 0
    for r in range(world):
        n = (base + (1 if r < extra else 0)) * block
        hi = min(vocab, lo + n)
        out.append((lo, hi))
        lo = hi
    return out


def dense_fp8(x, wq, w_s):
    """out = bf16(x . W^T): the decode-width projections between the named kernels (gdn in_proj, qkv_proj,
    o_proj: qk_proj_decode.cu:409-470, dense8.py:317-353) at the target's fp8 block-scaled format."""
    return bf16_round(lmhead_logits(x, wq, w_s))


def add_rmsnorm(proj, residual, w, eps=1e-6):
    """r = bf16(proj + residual) (proj already bf16, fp32 add: proj.py:75-77); y = bf16(r * rsqrt(mean r^2 +
    eps) * (1 + w)) (proj.py:78-81).  Returns (y, r)."""
    r = bf16_round((np.asarray(proj, dtype=F32) + np.asarray(residual, dtype=F32)).astype(F32))
    var = np.mean(r.astype(np.float64) ** 2, axis=-1, keepdims=True)
    y = bf16_round((r * (1.0 / np.sqrt(var + eps)).astype(F32) * (F32(1.0) + np.asarray(w, dtype=F32))[None, :]).astype(F32))
    return y, r
