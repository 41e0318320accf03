"""Gated DeltaNet speculative-verify oracle (test infrastructure only, see oracle/__init__.py).

PARITY UNPINNED by the reference: its verify recurrence exists only as a CUDA kernel
(qk_gdn_verify.cu) that cannot run on a CPU, and it keeps its state as a checkpoint plus a
(d, k, g) ring instead of the explicit state used here.  This file restates the mathematics the
kernel documents, token by token in float64, with the reference's bf16 rounding points.
"""
from __future__ import annotations

import numpy as np

from .numerics import F32, bf16_round

HK, HV, DK, DV, NT = 16, 32, 128, 128, 4
QDIM = HK * DK              # 2048
CONV = 2 * QDIM + HV * DV   # 8192 channels: [q | k | v]  (qk_gdn_verify.cu:35,404-406)


def causal_conv(mixed, conv_state, conv_w):
    """Width-4 depthwise causal conv + SiLU with the carried 3-token state.

    Per channel and token s the window is [s0 s1 s2 x0 .. x3][s : s+4]; every tap product is
    rounded to bf16, the four are added in fp32 oldest first, SiLU, result stored as bf16
    (`conv_tap`, qk_gdn_verify.cu:240-247; Triton twin gdn.py:84-96).  conv_state is
    [B, C, 3] with column 2 the most recent token; conv_w is [C, 4] with tap 3 on the current
    token (qk_gdn_verify.cu:241-246,863-865).
    mixed: [B, NT, C].  Returns (y [B, NT, C] bf16 values, window [B, C, 7])."""
    B = mixed.shape[0]
    win = np.concatenate([np.asarray(conv_state, dtype=F32),
                          np.transpose(np.asarray(mixed, dtype=F32), (0, 2, 1))], axis=2)  # [B, C, 7]
    w = np.asarray(conv_w, dtype=F32)
    y = np.empty((B, NT, win.shape[1]), dtype=F32)
    for s in range(NT):
        acc = np.zeros(win.shape[:2], dtype=F32)
        for tap in range(4):
            acc = (acc + bf16_round((win[:, :, s + tap] * w[None, :, tap]).astype(F32))).astype(F32)
        with np.errstate(over="ignore"):
            y[:, s] = bf16_round((acc / (F32(1.0) + np.exp(-acc, dtype=F32))).astype(F32))
    return y, win


def gdn_verify(mixed, z, a, b, conv_state, conv_w, a_log, dt_bias, state, accepted, norm_w, eps=1e-6):
    """One verify step over NT = 4 draft tokens for B sequences.

    mixed [B*NT, 8192], z [B*NT, 4096], a, b [B*NT, 32] (bf16 values); conv_state [B, 8192, 3];
    conv_w [8192, 4]; a_log, dt_bias fp32 [32]; state fp32 [B, 32, 128 (v), 128 (k)], orientation
    S[v][k], o[v] = sum_k S[v][k] q[k], update S[v][k] += d[v] k[k] (qk_gdn_verify.cu:297,742-750);
    accepted int [B] in 0..NT; norm_w [128].

    q, k: conv -> fp32 L2 normalisation y / sqrt(sum y^2 + 1e-6), q also times d_k^-0.5
    (qk_gdn_verify.cu:576-581).  Gates: g = -exp(A_log) * softplus(a + dt_bias) with softplus the
    identity above 20, beta = sigmoid(b) (qk_gdn_verify.cu:616-631).  Value heads 2*hk and 2*hk+1
    share key head hk (qk_gdn_verify.cu:9-11,520).  Recurrence per value head, token s:
        S <- e^{g_s} S;  d = beta_s (v_s - S k_s);  S <- S + d k_s^T;  o_s = S q_s
    which is what the reference evaluates in closed form over the window
    (R, (I + A)^-1, F: qk_gdn_verify.cu:633-762).  o is rounded to bf16 before the gated RMSNorm
    (qk_gdn_verify.cu:761), out = bf16(o * rsqrt(mean o^2 + eps) * w * z * sigmoid(z))
    (qk_gdn_verify.cu:763-791).

    The state written back is the state after `accepted[b]` tokens (rollback = the tokens past
    it are discarded) and the conv state becomes the last three inputs of
    [s0 s1 s2 x0 .. x_{accepted-1}].
    Returns (out [B*NT, 4096] bf16 values, new_state fp32, new_conv_state bf16 values).
    """
    B = state.shape[0]
    mixed = np.asarray(mixed, dtype=F32).reshape(B, NT, CONV)
    z = np.asarray(z, dtype=F32).reshape(B, NT, HV, DV)
    a = np.asarray(a, dtype=F32).reshape(B, NT, HV)
    b = np.asarray(b, dtype=F32).reshape(B, NT, HV)
    y, win = causal_conv(mixed, conv_state, conv_w)
    q = y[:, :, :QDIM].reshape(B, NT, HK, DK)
    k = y[:, :, QDIM:2 * QDIM].reshape(B, NT, HK, DK)
    v = y[:, :, 2 * QDIM:].reshape(B, NT, HV, DV).astype(np.float64)
    qn = (q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True, dtype=F32) + F32(1e-6))).astype(F32)
    qn = (qn * F32(DK ** -0.5)).astype(np.float64)
    kn = (k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True, dtype=F32) + F32(1e-6))).astype(F32)
    kn = kn.astype(np.float64)

    xg = (a + np.asarray(dt_bias, dtype=F32)[None, None, :]).astype(np.float64)
    sp = np.where(xg <= 20.0, np.log1p(np.exp(np.minimum(xg, 20.0))), xg)
    g = -np.exp(np.asarray(a_log, dtype=np.float64))[None, None, :] * sp   # [B, NT, HV]
    beta = 1.0 / (1.0 + np.exp(-b.astype(np.float64)))

    S = np.asarray(state, dtype=np.float64).copy()          # [B, HV, DV, DK]
    new_state = np.asarray(state, dtype=F32).copy()
    o = np.empty((B, NT, HV, DV), dtype=np.float64)
    acc = np.asarray(accepted).astype(np.int64)
    hk_of = np.arange(HV) // 2
    for s in range(NT):
        ks = kn[:, s, hk_of]                                # [B, HV, DK]
        qs = qn[:, s, hk_of]
        S = S * np.exp(g[:, s])[:, :, None, None]
        d = beta[:, s][:, :, None] * (v[:, s] - np.einsum("bhvk,bhk->bhv", S, ks))
        S = S + d[:, :, :, None] * ks[:, :, None, :]
        o[:, s] = np.einsum("bhvk,bhk->bhv", S, qs)
        hit = acc == s + 1
        if np.any(hit):
            new_state[hit] = S[hit].astype(F32)

    ob = bf16_round(o.astype(F32))
    var = np.mean(ob * ob, axis=-1, keepdims=True, dtype=F32)
    rstd = (F32(1.0) / np.sqrt(var + F32(eps))).astype(F32)
    with np.errstate(over="ignore"):
        gate = (z * (F32(1.0) / (F32(1.0) + np.exp(-z, dtype=F32)))).astype(F32)
    out = bf16_round((ob * rstd * np.asarray(norm_w, dtype=F32)[None, None, None, :] * gate).astype(F32))

    new_conv = np.empty((B, CONV, 3), dtype=F32)
    for bi in range(B):
        n = int(acc[bi])
        new_conv[bi] = win[bi, :, n:n + 3]
    return out.reshape(B * NT, HV * DV), new_state, new_conv


RING = 16


def ring_state(checkpoint, d_ring, k_ring, g_ring, write_pos, cache_base):
    """The state a checkpoint plus the committed ring entries stand for, in float64:
        S = e^{total} H0 + sum_{c < wp} e^{total - pre_c} d_c k_c^T,  pre_c = g_0 + .. + g_c, total = pre_{wp-1}
    with logical entry c at physical entry (cache_base + c) & 15 (qk_gdn_verify.cu:597-604,633-647,706-717).
    checkpoint [32, 128, 128]; d_ring [32, 16, 128]; k_ring [16, 16, 128]; g_ring [32, 16] (one request)."""
    wp = int(min(max(write_pos, 0), RING))
    S = np.asarray(checkpoint, dtype=np.float64).copy()
    phys = [(int(cache_base) + c) & (RING - 1) for c in range(wp)]
    for hv in range(HV):
        g = np.asarray(g_ring[hv], dtype=np.float64)[phys] if wp else np.zeros(0)
        pre = np.cumsum(g)
        total = pre[-1] if wp else 0.0
        S[hv] *= np.exp(total)
        for c in range(wp):
            d = np.asarray(d_ring[hv, phys[c]], dtype=np.float64)
            k = np.asarray(k_ring[hv // 2, phys[c]], dtype=np.float64)
            S[hv] += np.exp(total - pre[c]) * d[:, None] * k[None, :]
    return S


def gdn_verify_replay(mixed, z, a, b, conv_state, conv_w, a_log, dt_bias, checkpoint, d_ring, k_ring, g_ring,
                      state_idx, ring_idx, write_pos, cache_base, norm_w, eps=1e-6):
    """The verify step on the checkpoint + (d, k, g) ring layout (qk_gdn_verify.cu:293-793, gdn_fused.py:37-57).

    checkpoint fp32 [slots, 32, 128, 128] and conv_state [slots, 8192, 3] are indexed by state_idx[b]
    (< 0: padded request, zero output); d_ring [rslots, 32, 16, 128], k_ring [rslots, 16, 16, 128] (bf16 high
    parts, the only parts the kernel reads: qk_gdn_verify.cu:63-64), g_ring fp32 [rslots, 32, 16],
    write_pos / cache_base int [rslots], indexed by ring_idx[b].

    The window runs on the state `ring_state` reconstructs; the recurrence, rounding points and the gated
    norm are those of `gdn_verify`.  The per-token deltas d_s of the sequential recurrence are the D_s of the
    reference's closed form (S_n = e^{G_{n-1}} S + sum_{i<n} e^{G_{n-1} - G_i} D_i k_i^T,
    qk_gdn_verify.cu:686-752), so the appended entries are (d_s, unit key k_s, g_s).

    Returns a dict: out [B*4, 4096] bf16 values; per request the appended entries
    d_hi, d_lo [B, 4, 32, 128], k_hi, k_lo [B, 4, 16, 128] (bf16 values; low = bf16(value - high),
    qk_gdn_verify.cu:588-593,776-778), g [B, 4, 32] fp32; `slots` [B, 4] the physical entry of draft s or -1
    when write_pos + s >= 16 (qk_gdn_verify.cu:586,631,774); new_conv [B, 8192, 3] = [x1 x2 x3] and
    window [B, 8192, 6] = [s1 s2 x0 x1 x2 x3] (Conv4::store, qk_gdn_verify.cu:277-289)."""
    B = len(state_idx)
    mixed = np.asarray(mixed, dtype=F32).reshape(B, NT, CONV)
    z = np.asarray(z, dtype=F32).reshape(B, NT, HV, DV)
    a = np.asarray(a, dtype=F32).reshape(B, NT, HV)
    b = np.asarray(b, dtype=F32).reshape(B, NT, HV)
    sidx = np.asarray(state_idx).astype(np.int64)
    ridx = np.asarray(ring_idx).astype(np.int64)
    live = sidx >= 0
    cs = np.zeros((B, CONV, 3), dtype=F32)
    cs[live] = np.asarray(conv_state, dtype=F32)[sidx[live]]
    y, win = causal_conv(mixed, cs, conv_w)
    q = y[:, :, :QDIM].reshape(B, NT, HK, DK)
    k = y[:, :, QDIM:2 * QDIM].reshape(B, NT, HK, DK)
    v = y[:, :, 2 * QDIM:].reshape(B, NT, HV, DV).astype(np.float64)
    qn = (q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True, dtype=F32) + F32(1e-6))).astype(F32)
    qn = (qn * F32(DK ** -0.5)).astype(np.float64)
    kn32 = (k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True, dtype=F32) + F32(1e-6))).astype(F32)
    kn = kn32.astype(np.float64)
    xg = (a + np.asarray(dt_bias, dtype=F32)[None, None, :]).astype(np.float64)
    sp = np.where(xg <= 20.0, np.log1p(np.exp(np.minimum(xg, 20.0))), xg)
    g = -np.exp(np.asarray(a_log, dtype=np.float64))[None, None, :] * sp
    beta = 1.0 / (1.0 + np.exp(-b.astype(np.float64)))

    S = np.zeros((B, HV, DV, DK), dtype=np.float64)
    slots = -np.ones((B, NT), dtype=np.int64)
    for bi in range(B):
        if not live[bi]:
            continue
        r = ridx[bi]
        S[bi] = ring_state(checkpoint[sidx[bi]], d_ring[r], k_ring[r], g_ring[r], write_pos[r], cache_base[r])
        wp = int(min(max(write_pos[r], 0), RING))
        for s in range(NT):
            if wp + s < RING:
                slots[bi, s] = (int(cache_base[r]) + wp + s) & (RING - 1)
    o = np.empty((B, NT, HV, DV), dtype=np.float64)
    dd = np.empty((B, NT, HV, DV), dtype=np.float64)
    hk_of = np.arange(HV) // 2
    for s in range(NT):
        ks = kn[:, s, hk_of]
        qs = qn[:, s, hk_of]
        S = S * np.exp(g[:, s])[:, :, None, None]
        d = beta[:, s][:, :, None] * (v[:, s] - np.einsum("bhvk,bhk->bhv", S, ks))
        S = S + d[:, :, :, None] * ks[:, :, None, :]
        o[:, s] = np.einsum("bhvk,bhk->bhv", S, qs)
        dd[:, s] = d
    ob = bf16_round(o.astype(F32))
    var = np.mean(ob * ob, axis=-1, keepdims=True, dtype=F32)
    rstd = (F32(1.0) / np.sqrt(var + F32(eps))).astype(F32)
    with np.errstate(over="ignore"):
        gate = (z * (F32(1.0) / (F32(1.0) + np.exp(-z, dtype=F32)))).astype(F32)
    out = bf16_round((ob * rstd * np.asarray(norm_w, dtype=F32)[None, None, None, :] * gate).astype(F32))
    out[~live] = 0
    d32 = dd.astype(F32)
    d_hi = bf16_round(d32)
    d_lo = bf16_round((d32 - d_hi).astype(F32))
    k_hi = bf16_round(kn32)
    k_lo = bf16_round((kn32 - k_hi).astype(F32))
    return dict(out=out.reshape(B * NT, HV * DV), d_hi=d_hi, d_lo=d_lo, k_hi=k_hi, k_lo=k_lo, g=g.astype(F32),
                slots=slots, new_conv=win[:, :, 4:7].copy(), window=win[:, :, 1:7].copy(), live=live,
                state_after=S)
