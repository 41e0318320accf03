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


_lib.impl("router", _router, "CUDA")
_lib.impl("gdn_verify", _gdn, "CUDA")
_lib.impl("gdn_verify_replay", _gdn_replay, "CUDA")
_lib.impl("attn_front", _attn, "CUDA")
_lib.impl("attn_verify", _attn_verify, "CUDA")
_lib.impl("lmhead_argmax", _lmhead, "CUDA")
_lib.impl("moe_combine", _combine, "CUDA")
