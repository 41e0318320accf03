"""Registers the hot-path operators as torch custom ops (`torch.ops.b200nodes.*`) so that an engine
that dispatches through the torch op registry (SGLang does) can load them.  The implementations call
the C-ABI library through `bundles_b200.ops`; only the CUDA dispatch key is registered: on any other
device the ops raise (there is no fallback)."""
from __future__ import annotations

import torch

from . import ops

_lib = torch.library.Library("b200nodes", "DEF")
_lib.define("router(Tensor x, Tensor wr, Tensor? bias, int top_k, bool round_bf16) -> (Tensor, Tensor)")
_lib.define("gdn_verify(Tensor mixed, Tensor z, Tensor a, Tensor b, Tensor(a!) conv_state, Tensor conv_w, "
            "Tensor a_log, Tensor dt_bias, Tensor(b!) state, Tensor accepted, Tensor norm_w, float eps) -> Tensor")
_lib.define("gdn_verify_replay(Tensor mixed, Tensor z, Tensor a, Tensor b, Tensor(a!) conv_state, Tensor conv_w, "
            "Tensor(b!) window, Tensor a_log, Tensor dt_bias, Tensor checkpoint, Tensor(c!) d_ring, Tensor(d!) dlo_ring, "
            "Tensor(e!) k_ring, Tensor(f!) klo_ring, Tensor(g!) g_ring, Tensor state_idx, Tensor ring_idx, Tensor win_idx, "
            "Tensor write_pos, Tensor cache_base, Tensor norm_w, float eps) -> Tensor")
_lib.define("attn_front(Tensor x, Tensor w, Tensor w_s, Tensor q_norm_w, Tensor k_norm_w, Tensor positions, "
            "Tensor cos_sin, float eps, bool out_fp8) -> (Tensor, Tensor, Tensor, Tensor)")
_lib.define("attn_verify(Tensor q, Tensor gate, Tensor k_new, Tensor v_new, Tensor(a!) kcache, Tensor(b!) vcache, "
            "Tensor page_table, Tensor seqlens, float scale) -> Tensor")
_lib.define("lmhead_argmax(Tensor x, Tensor w, Tensor w_s, int shard_lo) -> (Tensor, Tensor)")
_lib.define("moe_combine(Tensor cache, Tensor x, Tensor? gate_w, int top_k, Tensor? pos) -> Tensor")
_lib.define("moe_combine_norm(Tensor cache, Tensor x, Tensor? gate_w, int top_k, Tensor(a!) residual, Tensor norm_w, "
            "float eps, Tensor? pos) -> (Tensor, Tensor)")
# The routing lists travel as one int32 tensor and one fp32 tensor (the C ABI's nine device arrays laid end to end,
# see `lists_pack`), so that the three MoE ops below compose through the registry without Python objects.
_lib.define("build_lists(Tensor ids, Tensor wts, Tensor? pos, int e_lo, int n_local, int block_rows, bool with_shared) "
            "-> (Tensor, Tensor)")
_lib.define("moe_w8a8(Tensor x, Tensor w13, Tensor s13, Tensor w2, Tensor s2, Tensor? sh13, Tensor? shs13, Tensor? sh2, "
            "Tensor? shs2, Tensor lists_i, Tensor lists_f, int top_k, int block_rows) -> Tensor")
_lib.define("moe_fp8(Tensor x, Tensor w13, Tensor s13, Tensor w2, Tensor s2, Tensor? sh13, Tensor? shs13, Tensor? sh2, "
            "Tensor? shs2, Tensor lists_i, Tensor lists_f, int top_k, int block_rows) -> Tensor")
_lib.define("dense_fp8(Tensor x, Tensor w, Tensor w_s) -> Tensor")
_lib.define("add_rmsnorm(Tensor proj, Tensor(a!) residual, Tensor w, float eps) -> Tensor")
_lib.define("argmax_merge(Tensor maxes, Tensor idxs) -> Tensor")
_lib.define("gdn_ring_fold(Tensor(a!) checkpoint, Tensor d_ring, Tensor dlo_ring, Tensor k_ring, Tensor klo_ring, "
            "Tensor g_ring, Tensor state_idx, Tensor ring_idx, Tensor write_pos, Tensor cache_base) -> ()")


def _router(x, wr, bias, top_k, round_bf16):
    _, ids, wts = ops.router(x, wr, top_k, bias, round_bf16, want_logits=False)
    return ids, wts


def _gdn(mixed, z, a, b, conv_state, conv_w, a_log, dt_bias, state, accepted, norm_w, eps):
    return ops.gdn_verify(mixed, z, a, b, conv_state, conv_w, a_log, dt_bias, state, accepted, norm_w, eps)


def _gdn_replay(mixed, z, a, b, conv_state, conv_w, window, a_log, dt_bias, checkpoint, d_ring, dlo_ring, k_ring,
                klo_ring, g_ring, state_idx, ring_idx, win_idx, write_pos, cache_base, norm_w, eps):
    return ops.gdn_verify_replay(mixed, z, a, b, conv_state, conv_w, window, a_log, dt_bias, checkpoint, d_ring, dlo_ring,
                                 k_ring, klo_ring, g_ring, state_idx, ring_idx, win_idx, write_pos, cache_base, norm_w, eps)


def _attn(x, w, w_s, qw, kw, positions, cos_sin, eps, out_fp8):
    return ops.attn_front(x, w, w_s, qw, kw, positions, cos_sin, eps, out_fp8)


def _attn_verify(q, gate, k_new, v_new, kcache, vcache, page_table, seqlens, scale):
    return ops.attn_verify(q, gate, k_new, v_new, kcache, vcache, page_table, seqlens, scale)


def _lmhead(x, w, w_s, shard_lo):
    mx, idx, _ = ops.lmhead_argmax(x, w, w_s, shard_lo)
    return mx, idx


def _combine(cache, x, gate_w, top_k, pos):
    return ops.moe_combine(cache, x, gate_w, top_k, pos)


def _combine_norm(cache, x, gate_w, top_k, residual, norm_w, eps, pos):
    return ops.moe_combine_norm(cache, x, gate_w, top_k, residual, norm_w, eps, pos)


def lists_pack(T, K, n_local, block_rows, device):
    """RoutingLists whose nine arrays are views into one int32 and one fp32 tensor."""
    mb = ops._lib.lib().b200_moe_max_blocks(T, K, n_local, block_rows)
    sizes = [n_local + 1, n_local + 2, T * K, T * (K + 1), mb, mb, mb, 1]
    li = torch.zeros(sum(sizes), dtype=torch.int32, device=device)
    lf = torch.zeros(T * (K + 1), dtype=torch.float32, device=device)
    return _lists_view(li, lf, T, K, n_local, block_rows), li, lf


def _lists_view(li, lf, T, K, n_local, block_rows):
    mb = ops._lib.lib().b200_moe_max_blocks(T, K, n_local, block_rows)
    sizes = [n_local + 1, n_local + 2, T * K, T * (K + 1), mb, mb, mb, 1]
    if li.numel() != sum(sizes) or lf.numel() != T * (K + 1):
        raise ops.B200Error("routing-list tensors do not match (T, K, n_local, block_rows)")
    parts = torch.split(li, sizes)
    L = ops.RoutingLists.__new__(ops.RoutingLists)
    L.T, L.K, L.E_local, L.block_rows, L.max_blocks = T, K, n_local, block_rows, mb
    (L.counts, L.offsets, L.row_of_pair, L.slot_of_row, L.blk_expert, L.blk_row0, L.blk_rows, L.nblocks) = parts
    L.wt_of_row = lf
    L.c = ops.MoeLists(*[t.data_ptr() for t in (L.counts, L.offsets, L.row_of_pair, L.slot_of_row, L.wt_of_row,
                                                 L.blk_expert, L.blk_row0, L.blk_rows, L.nblocks)])
    return L


def _build_lists(ids, wts, pos, e_lo, n_local, block_rows, with_shared):
    T, K = ids.shape
    L, li, lf = lists_pack(T, K, n_local, block_rows, ids.device)
    ops.build_lists(ids, wts, L, pos, e_lo=e_lo, with_shared=with_shared)
    return li, lf


def _weights(w13, s13, w2, s2, sh13, shs13, sh2, shs2):
    return ops.MoeW8A8Weights(w13, s13, w2, s2, sh13, shs13, sh2, shs2)


def _moe_w8a8(x, w13, s13, w2, s2, sh13, shs13, sh2, shs2, lists_i, lists_f, top_k, block_rows):
    L = _lists_view(lists_i, lists_f, x.shape[0], top_k, w13.shape[0], block_rows)
    return ops.moe_w8a8(x, _weights(w13, s13, w2, s2, sh13, shs13, sh2, shs2), L)


def _moe_fp8(x, w13, s13, w2, s2, sh13, shs13, sh2, shs2, lists_i, lists_f, top_k, block_rows):
    L = _lists_view(lists_i, lists_f, x.shape[0], top_k, w13.shape[0], block_rows)
    return ops.moe_fp8(x, _weights(w13, s13, w2, s2, sh13, shs13, sh2, shs2), L)


def _dense(x, w, w_s):
    return ops.dense_fp8(x, w, w_s)


def _add_norm(proj, residual, w, eps):
    return ops.add_rmsnorm(proj, residual, w, eps)


def _merge(maxes, idxs):
    return ops.argmax_merge(maxes, idxs)


def _fold(checkpoint, d_ring, dlo_ring, k_ring, klo_ring, g_ring, state_idx, ring_idx, write_pos, cache_base):
    ops.gdn_ring_fold(checkpoint, d_ring, dlo_ring, k_ring, klo_ring, g_ring, state_idx, ring_idx, write_pos, cache_base)


_lib.impl("router", _router, "CUDA")
_lib.impl("moe_combine_norm", _combine_norm, "CUDA")
_lib.impl("build_lists", _build_lists, "CUDA")
_lib.impl("moe_w8a8", _moe_w8a8, "CUDA")
_lib.impl("moe_fp8", _moe_fp8, "CUDA")
_lib.impl("dense_fp8", _dense, "CUDA")
_lib.impl("add_rmsnorm", _add_norm, "CUDA")
_lib.impl("argmax_merge", _merge, "CUDA")
_lib.impl("gdn_ring_fold", _fold, "CUDA")
_lib.impl("gdn_verify", _gdn, "CUDA")
_lib.impl("gdn_verify_replay", _gdn_replay, "CUDA")
_lib.impl("attn_front", _attn, "CUDA")
_lib.impl("attn_verify", _attn_verify, "CUDA")
_lib.impl("lmhead_argmax", _lmhead, "CUDA")
_lib.impl("moe_combine", _combine, "CUDA")
