"""Router oracle: gate logits, softmax, top-k with renormalisation, routing lists.

Test infrastructure only (see oracle/__init__.py).
"""
from __future__ import annotations

import numpy as np

from .numerics import F32, bf16_round, fma32

SLICE = 128


def gate_logits(x: np.ndarray, wr: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    """logits[t, e] = sum_k x[t, k] * wr[e, k] (+ bias[e]) in fp32 with ONE fixed summation tree.

    The reference fixes the tree of its gate GEMM so that its CUDA and Triton routers agree bit
    for bit (split-K 4, k16 MMA chains in increasing k, partials added in order
    (((0 + p0) + p1) + p2) + p3: qk_route.cu:3-4,125-133; i8x_decode.py:226-247).  The target keeps
    that discipline with fp32 weights and FMA chains:
      p_s   = fma chain from 0 over k = 128 s .. 128 s + 127, ascending, s = 0 .. H/128 - 1;
      logit = ((p_0 + p_1) + p_2) + ... (slice order);  bias (skew / correction bias) added last.
    x holds bf16 values (as fp32), wr is fp32 [E, H].
    """
    x = np.asarray(x, dtype=F32)
    wr = np.asarray(wr, dtype=F32)
    T, H = x.shape
    E = wr.shape[0]
    assert H % SLICE == 0
    ns = H // SLICE
    xs = x.reshape(T, ns, SLICE)
    ws = wr.reshape(E, ns, SLICE)
    out = np.empty((T, E), dtype=F32)
    chunk = max(1, (1 << 22) // (E * ns))
    for t0 in range(0, T, chunk):
        xa = xs[t0:t0 + chunk]
        acc = np.zeros((xa.shape[0], E, ns), dtype=F32)
        for k in range(SLICE):
            acc = fma32(xa[:, None, :, k], ws[None, :, :, k], acc)
        tot = acc[..., 0]
        for s in range(1, ns):
            tot = (tot + acc[..., s]).astype(F32)
        out[t0:t0 + chunk] = tot
    if bias is not None:
        out = (out + np.asarray(bias, dtype=F32)[None, :]).astype(F32)
    return out


def topk_softmax(logits: np.ndarray, top_k: int, round_bf16: bool = False):
    """Softmax over all experts, top-k, renormalise (`_top8`, i8x_decode.py:99-117).

    x = logits (optionally rounded to bf16 first, as the reference does: i8x_decode.py:100);
    prob = exp(x - max) / sum; pick k times the largest x, ties to the SMALLEST expert id
    (i8x_decode.py:108-109; qk_route.cu:71-75,142: -0 == +0, NaN ranks lowest);
    w = prob[picked] / sum(picked), the divisor replaced by 1 when the sum is not positive
    (i8x_decode.py:115-116).  Returns (ids int32 [T, k] in pick order, w fp32 [T, k]).
    """
    x = np.asarray(logits, dtype=F32)
    if round_bf16:
        x = bf16_round(x)
    T, E = x.shape
    key = np.where(np.isnan(x), -np.inf, x).astype(F32)
    key = key + F32(0.0)  # -0 -> +0
    mx = np.max(key, axis=1, keepdims=True)
    ex = np.exp((key - mx).astype(F32), dtype=F32)
    ex = np.where(np.isnan(x), F32(0.0), ex)
    prob = (ex / np.sum(ex, axis=1, keepdims=True, dtype=F32)).astype(F32)
    # stable argsort on -key: equal keys keep ascending id order
    order = np.argsort(-key, axis=1, kind="stable")[:, :top_k]
    ids = order.astype(np.int32)
    w = np.take_along_axis(prob, order, axis=1)
    tot = np.zeros(T, dtype=F32)
    for j in range(top_k):  # sequential sum in pick order
        tot = (tot + w[:, j]).astype(F32)
    w = (w / np.where(tot > 0, tot, F32(1.0))[:, None]).astype(F32)
    return ids, w


def route(x, wr, top_k, bias=None, round_bf16=False):
    logits = gate_logits(x, wr, bias)
    ids, w = topk_softmax(logits, top_k, round_bf16)
    return logits, ids, w


def routing_lists(ids: np.ndarray, n_experts: int, valid: np.ndarray | None = None, block: int = 128):
    """Per-expert token lists (`i8x_dec_lists`, i8x_decode.py:264-289; tail of `route_kernel`,
    qk_route.cu:297-357).

    A routed pair p = t * top_k + j (the reference's slot id, i8x_decode.py:297) lands in the
    sorted row offsets[e] + rank, rank = number of earlier valid pairs with the same expert.
    Rows of tokens whose `valid` flag is false (graph padding, position == 0 in the reference:
    qk_route.cu:229,307) get row -1 and are not counted.  Each expert's rows are cut into `block`-row
    pieces (the reference cuts at 16; the target's MMA N tile is up to 128); the block list is ordered
    heaviest first (see below), the reference's walks experts in ascending order.
    Returns dict(counts, offsets [E+1], row_of_pair [T*k], pair_of_row [sum counts],
                 blk_expert, blk_row0, blk_rows).
    """
    ids = np.asarray(ids, dtype=np.int64)
    T, K = ids.shape
    flat = ids.reshape(-1)
    ok = np.ones(T, dtype=bool) if valid is None else np.asarray(valid, dtype=bool)
    okp = np.repeat(ok, K)
    counts = np.bincount(flat[okp], minlength=n_experts).astype(np.int32)
    offsets = np.zeros(n_experts + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    row_of_pair = np.full(T * K, -1, dtype=np.int32)
    fill = offsets[:-1].copy()
    for p in range(T * K):
        if okp[p]:
            e = flat[p]
            row_of_pair[p] = fill[e]
            fill[e] += 1
    pair_of_row = np.full(int(offsets[-1]), -1, dtype=np.int32)
    sel = row_of_pair >= 0
    pair_of_row[row_of_pair[sel]] = np.nonzero(sel)[0]
    # heaviest first: full blocks, then partial blocks by quarter of the block size (>= 3/4, >= 1/2, >= 1/4, less),
    # each class in expert order (the GEMMs deal tiles to their CTAs round-robin; the reference's list is in expert order)
    classes = ([], [], [], [], [])
    for e in range(n_experts):
        c = int(counts[e])
        for r0 in range(0, c, block):
            n = min(block, c - r0)
            cls = 0 if (n == block or block != 128) else 4 - min(3, (4 * n) // block)  # only 128-row lists are reordered
            classes[cls].append((e, int(offsets[e]) + r0, n))
    be = [t[0] for cl in classes for t in cl]
    b0 = [t[1] for cl in classes for t in cl]
    bn = [t[2] for cl in classes for t in cl]
    return dict(counts=counts, offsets=offsets, row_of_pair=row_of_pair, pair_of_row=pair_of_row,
                blk_expert=np.asarray(be, dtype=np.int32), blk_row0=np.asarray(b0, dtype=np.int32),
                blk_rows=np.asarray(bn, dtype=np.int32))
