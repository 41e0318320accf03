"""Oracle for the attention-verify core (4 draft tokens over a paged e4m3 KV cache).

Test infrastructure only (see oracle/__init__.py).  PARITY UNPINNED: the reference's kernel is CUDA only
(qk_attn_verify.cu:354-744); this restates its arithmetic in float64 with its rounding points: q, k, v are
e4m3 values (exact in f16 / fp32), scores are exact products summed in fp32 on the GPU (float64 here),
probabilities are rounded to f16 before the P . V product (qk_attn_verify.cu:297-301), the normalised
output is rounded to bf16 and then multiplied by sigmoid(gate) (:559-562).  The running-maximum policy
(:264-267) and the split order change only which power of two scales P before its f16 rounding; the oracle
uses the row maximum, the comparison uses a bf16-level tolerance.
"""
from __future__ import annotations

import numpy as np

from .numerics import F32, bf16_round, e4m3_decode

HQ, HKV, GQ, D, NT, PAGE = 16, 2, 8, 256, 4, 128


def append_kv(kcache, vcache, k_new, v_new, page_table, seqlens):
    """Write the drafts' K rows and (transposed) V columns at positions seqlens-4 .. seqlens-1.
    kcache uint8 [P,2,128,256]; vcache uint8 [P,2,256,128]; k_new, v_new uint8 [4B,2,256]."""
    kc, vc = kcache.copy(), vcache.copy()
    for r, n in enumerate(seqlens):
        for t in range(NT):
            pos = int(n) - NT + t
            page = int(page_table[r, pos // PAGE])
            for h in range(HKV):
                kc[page, h, pos % PAGE, :] = k_new[r * NT + t, h]
                vc[page, h, :, pos % PAGE] = v_new[r * NT + t, h]
    return kc, vc


def attn_verify(q, gate, k_new, v_new, kcache, vcache, page_table, seqlens, scale=1.0 / 16.0):
    """q uint8 [4B,16,256] e4m3 codes; gate bf16 values [4B,16,256]; returns (out bf16 values [4B,4096],
    kcache', vcache')."""
    kc, vc = append_kv(kcache, vcache, k_new, v_new, page_table, seqlens)
    B = len(seqlens)
    out = np.zeros((B * NT, HQ * D), dtype=F32)
    qf = e4m3_decode(q).astype(np.float64)
    for r in range(B):
        n = int(seqlens[r])
        npages = (n + PAGE - 1) // PAGE
        pages = [int(page_table[r, i]) for i in range(npages)]
        for h in range(HKV):
            K = np.concatenate([e4m3_decode(kc[pg, h]) for pg in pages], axis=0)[:n].astype(np.float64)      # [n,256]
            V = np.concatenate([e4m3_decode(vc[pg, h]).T for pg in pages], axis=0)[:n].astype(np.float64)    # [n,256]
            for t in range(NT):
                lim = n - NT + t  # keys 0..lim
                for g in range(GQ):
                    hq = h * GQ + g
                    s = (K[:lim + 1] @ qf[r * NT + t, hq]).astype(F32) * F32(scale * 1.4426950408889634)
                    m = s.max()
                    p = np.exp2((s - m).astype(np.float64))
                    p16 = p.astype(np.float16).astype(np.float64)
                    o = (p16 @ V[:lim + 1]) / p.sum()  # the row sum takes the unrounded probabilities (:290-302)
                    ob = bf16_round(o.astype(F32))
                    gv = np.asarray(gate[r * NT + t, hq], dtype=F32)
                    sig = (F32(1.0) / (F32(1.0) + np.exp(-gv, dtype=F32))).astype(F32)
                    out[r * NT + t, hq * D:(hq + 1) * D] = bf16_round((ob * sig).astype(F32))
    return out, kc, vc
