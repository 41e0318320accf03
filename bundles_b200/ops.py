"""Host-side operators: torch tensors in, C-ABI calls out.

torch is used for device memory and the current stream only; every computation happens in
libb200nodes.so.  Each function mirrors the reference operator it replaces (names in the
docstrings) and raises `B200Error` on a non-zero return code, as the reference's TORCH_CHECKs
raise RuntimeError (qk_route.cu:1128-1133).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import B200Error, MoeLists, MoeWeights, check

__all__ = ["router", "RoutingLists", "build_lists", "MoeW8A8Weights", "moe_w8a8", "moe_w8a8_ep", "ep_push", "ep_put",
           "ep_barrier", "moe_fp8", "moe_fp8_ep", "moe_combine", "moe_combine_norm", "attn_front", "attn_verify",
           "dense_fp8", "dense_fp8_split", "dense_fp8_add_rmsnorm", "add_rmsnorm", "lmhead_argmax", "argmax_merge", "gdn_verify",
           "gdn_verify_replay", "gdn_ring_fold", "set_wait_budget_ns", "selftest_wait_expiry", "new_status",
           "read_status", "B200Error"]


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t, dtype, name, dims=None):
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == dtype and t.is_contiguous()):
        raise B200Error(f"{name} must be a contiguous CUDA tensor of {dtype}")
    if dims is not None and t.dim() != dims:
        raise B200Error(f"{name} must have {dims} dimensions, got {tuple(t.shape)}")


def new_status(device) -> torch.Tensor:
    """A zeroed device status word for kernels with bounded waits (see include/b200nodes.h)."""
    return torch.zeros(4, dtype=torch.int32, device=device)


def read_status(status: torch.Tensor) -> int:
    return int(status[0].item())


# ---------------------------------------------------------------------------------------------------
def router_scratch(T, H, E, device):
    n = _lib.lib().b200_router_scratch_bytes(T, H, E)
    return torch.empty(max(n, 16), dtype=torch.uint8, device=device)


def router(x, wr, top_k, bias=None, round_bf16=False, logits=None, scratch=None, want_logits=True, ids=None,
           wts=None):
    """Gate logits + softmax top-k + renormalise (reference: qk_route.route / i8x_dec_topk).
    Returns (logits fp32 [T,E] or None, ids int32 [T,K], wts fp32 [T,K])."""
    _need(x, torch.bfloat16, "x", 2)
    _need(wr, torch.float32, "wr", 2)
    T, H = x.shape
    E = wr.shape[0]
    if bias is not None:
        _need(bias, torch.float32, "bias", 1)
    if logits is None and want_logits:
        logits = torch.empty(T, E, dtype=torch.float32, device=x.device)
    if scratch is None:
        scratch = router_scratch(T, H, E, x.device)
    if ids is None:
        ids = torch.empty(T, top_k, dtype=torch.int32, device=x.device)
    if wts is None:
        wts = torch.empty(T, top_k, dtype=torch.float32, device=x.device)
    check(_lib.lib().b200_router(_p(x), _p(wr), _p(bias), T, H, E, top_k, 1 if round_bf16 else 0, _p(logits),
                                 _p(ids), _p(wts), _p(scratch), scratch.numel(), _stream()), "b200_router")
    return logits, ids, wts


class RoutingLists:
    """Device buffers of the routing lists (reference: `Workspace`, i8x_decode.py:495-518)."""

    def __init__(self, T, K, E_local, block_rows, device):
        self.T, self.K, self.E_local, self.block_rows = T, K, E_local, block_rows
        self.max_blocks = _lib.lib().b200_moe_max_blocks(T, K, E_local, block_rows)
        i32 = dict(dtype=torch.int32, device=device)
        self.counts = torch.zeros(E_local + 1, **i32)
        self.offsets = torch.zeros(E_local + 2, **i32)
        self.row_of_pair = torch.zeros(T * K, **i32)
        self.slot_of_row = torch.zeros(T * (K + 1), **i32)
        self.wt_of_row = torch.zeros(T * (K + 1), dtype=torch.float32, device=device)
        self.blk_expert = torch.zeros(self.max_blocks, **i32)
        self.blk_row0 = torch.zeros(self.max_blocks, **i32)
        self.blk_rows = torch.zeros(self.max_blocks, **i32)
        self.nblocks = torch.zeros(1, **i32)
        self.c = MoeLists(*[t.data_ptr() for t in (self.counts, self.offsets, self.row_of_pair, self.slot_of_row,
                                                   self.wt_of_row, self.blk_expert, self.blk_row0, self.blk_rows,
                                                   self.nblocks)])


def build_lists(ids, wts, lists: RoutingLists, pos=None, e_lo=0, with_shared=True, shared_range=None):
    """Per-expert sorted rows + GEMM block list (reference: i8x_dec_lists).  `shared_range` = (first token, count):
    only these tokens get a shared-expert row (an expert-parallel rank's own tokens among the gathered ones)."""
    _need(ids, torch.int32, "ids", 2)
    _need(wts, torch.float32, "wts", 2)
    if pos is not None:
        _need(pos, torch.int64, "pos", 1)
    T, K = ids.shape
    if (T, K) != (lists.T, lists.K):
        raise B200Error("routing lists were sized for another (T, K)")
    if shared_range is not None:
        lo, n = shared_range
        check(_lib.lib().b200_moe_build_lists_range(_p(ids), _p(wts), _p(pos), T, K, e_lo, lists.E_local,
                                                    lists.block_rows, int(lo), int(n), C.byref(lists.c), _stream()),
              "b200_moe_build_lists_range")
        return lists
    check(_lib.lib().b200_moe_build_lists(_p(ids), _p(wts), _p(pos), T, K, e_lo, lists.E_local, lists.block_rows,
                                          1 if with_shared else 0, C.byref(lists.c), _stream()),
          "b200_moe_build_lists")
    return lists


@dataclass
class MoeW8A8Weights:
    """Private int8 copy of one layer's experts (reference: `Copy`, i8x_kernels.py:69-110)."""
    w13: torch.Tensor       # int8 [E, 2I, H]
    s13: torch.Tensor       # fp32 [E, 2I]
    w2: torch.Tensor        # int8 [E, H, I]
    s2: torch.Tensor        # fp32 [E, H]
    sh13: torch.Tensor | None = None   # int8 [2I, H]
    shs13: torch.Tensor | None = None
    sh2: torch.Tensor | None = None    # int8 [H, I]
    shs2: torch.Tensor | None = None

    def c_struct(self):
        return MoeWeights(*[0 if t is None else t.data_ptr() for t in (self.w13, self.s13, self.w2, self.s2,
                                                                        self.sh13, self.shs13, self.sh2, self.shs2)])


def moe_w8a8_workspace(T, H, I, K, device):
    n = _lib.lib().b200_moe_w8a8_workspace_bytes(T, H, I, K)
    buf = torch.empty(n + 1024, dtype=torch.uint8, device=device)
    off = (-buf.data_ptr()) % 1024
    return buf[off:off + n]


STAGE_QUANT, STAGE_UP, STAGE_HQUANT, STAGE_DOWN = 1, 2, 4, 8
TEST_STARVE = 16     # B200_MOE_TEST_STARVE: self-test of the wait-expiry path, see include/b200nodes.h


def moe_w8a8(x, w: MoeW8A8Weights, lists: RoutingLists, cache=None, ws=None, status=None, dbg_acc13=None,
             dbg_h=None, stages=0):
    """Routed + shared expert MLPs in int8 W8A8 (reference: i8x_decode.moe_row_batch up/down).
    Returns cache bf16 [T*(K+1), H] indexed by slot."""
    _need(x, torch.bfloat16, "x", 2)
    _need(w.w13, torch.int8, "w13", 3)
    _need(w.w2, torch.int8, "w2", 3)
    T, H = x.shape
    E, twoI, _ = w.w13.shape
    I = twoI // 2
    K = lists.K
    if cache is None:
        cache = torch.zeros(T * (K + 1), H, dtype=torch.bfloat16, device=x.device)
    if ws is None:
        ws = moe_w8a8_workspace(T, H, I, K, x.device)
    wc = w.c_struct()
    check(_lib.lib().b200_moe_w8a8(_p(x), T, H, I, K, E, C.byref(wc), C.byref(lists.c), _p(cache), _p(ws),
                                   ws.numel(), _p(dbg_acc13), _p(dbg_h), int(stages), _p(status), _stream()),
          "b200_moe_w8a8")
    return cache


def moe_fp8_workspace(T, H, I, K, device):
    n = _lib.lib().b200_moe_fp8_workspace_bytes(T, H, I, K)
    buf = torch.empty(n + 1024, dtype=torch.uint8, device=device)
    off = (-buf.data_ptr()) % 1024
    return buf[off:off + n]


def moe_fp8(x, w: MoeW8A8Weights, lists: RoutingLists, cache=None, ws=None, status=None, dbg_h=None, stages=0):
    """Routed + shared expert MLPs in fp8 e4m3 with 128 x 128 block scales (weights as uint8 codes in
    the same container as the int8 block; scales [E, rows/128, K/128]).  Lists need block_rows <= 32.
    Returns cache bf16 [T*(K+1), H] indexed by slot."""
    _need(x, torch.bfloat16, "x", 2)
    _need(w.w13, torch.uint8, "w13", 3)
    _need(w.w2, torch.uint8, "w2", 3)
    if lists.block_rows > 32:
        raise B200Error("moe_fp8 needs routing lists built with block_rows <= 32")
    T, H = x.shape
    E, twoI, _ = w.w13.shape
    I = twoI // 2
    K = lists.K
    if cache is None:
        cache = torch.zeros(T * (K + 1), H, dtype=torch.bfloat16, device=x.device)
    if ws is None:
        ws = moe_fp8_workspace(T, H, I, K, x.device)
    wc = w.c_struct()
    check(_lib.lib().b200_moe_fp8(_p(x), T, H, I, K, E, C.byref(wc), C.byref(lists.c), _p(cache), _p(ws), ws.numel(),
                                  _p(dbg_h), int(stages), _p(status), _stream()), "b200_moe_fp8")
    return cache


def moe_w8a8_ep(x_all, w: MoeW8A8Weights, lists: RoutingLists, peer_ptrs, rank, tokens_per_rank, ws=None,
                status=None):
    """Expert-parallel int8 experts: this rank's experts over the gathered tokens, the weighted down rows
    stored straight into every home rank's routed cache (`peer_ptrs`: device pointers, one per rank)."""
    _need(x_all, torch.bfloat16, "x_all", 2)
    T, H = x_all.shape
    E, twoI, _ = w.w13.shape
    I = twoI // 2
    K = lists.K
    if ws is None:
        ws = moe_w8a8_workspace(T, H, I, K, x_all.device)
    world = len(peer_ptrs)
    arr = _ptr_array(peer_ptrs)
    wc = w.c_struct()
    check(_lib.lib().b200_moe_w8a8_ep(_p(x_all), T, H, I, K, E, C.byref(wc), C.byref(lists.c), arr, world,
                                      int(rank), int(tokens_per_rank), _p(ws), ws.numel(), _p(status), _stream()),
          "b200_moe_w8a8_ep")


def ep_push(x, ids, wts, rank, peer_x, peer_ids, peer_wts):
    """Store this rank's token rows and routing into every rank's gathered buffers (peer pointers as ints)."""
    _need(x, torch.bfloat16, "x", 2)
    _need(ids, torch.int32, "ids", 2)
    _need(wts, torch.float32, "wts", 2)
    T, H = x.shape
    world = len(peer_x)
    arr = lambda ptrs: (C.c_void_p * world)(*[C.c_void_p(int(p)) for p in ptrs])
    check(_lib.lib().b200_ep_push(_p(x), _p(ids), _p(wts), T, H, ids.shape[1], int(rank), world, arr(peer_x),
                                  arr(peer_ids), arr(peer_wts), _stream()), "b200_ep_push")


def _ptr_array(ptrs):
    return (C.c_void_p * len(ptrs))(*[C.c_void_p(int(p)) for p in ptrs])


def moe_fp8_ep(x_all, w: MoeW8A8Weights, lists: RoutingLists, peer_ptrs, rank, tokens_per_rank, ws=None, status=None):
    """Expert-parallel fp8 experts: this rank's experts over the gathered tokens, the weighted down rows stored
    straight into every home rank's routed cache (`peer_ptrs`: device pointers, one per rank)."""
    _need(x_all, torch.bfloat16, "x_all", 2)
    _need(w.w13, torch.uint8, "w13", 3)
    if lists.block_rows > 32:
        raise B200Error("moe_fp8_ep needs routing lists built with block_rows <= 32")
    T, H = x_all.shape
    E, twoI, _ = w.w13.shape
    I = twoI // 2
    K = lists.K
    if ws is None:
        ws = moe_fp8_workspace(T, H, I, K, x_all.device)
    wc = w.c_struct()
    check(_lib.lib().b200_moe_fp8_ep(_p(x_all), T, H, I, K, E, C.byref(wc), C.byref(lists.c), _ptr_array(peer_ptrs),
                                     len(peer_ptrs), int(rank), int(tokens_per_rank), _p(ws), ws.numel(), _p(status),
                                     _stream()), "b200_moe_fp8_ep")


def ep_put(src, dst_offset_bytes, peer_ptrs):
    """Store the bytes of `src` into every rank's buffer at `dst_offset_bytes` (an all-gather by peer stores)."""
    if not (isinstance(src, torch.Tensor) and src.is_cuda and src.is_contiguous()):
        raise B200Error("ep_put: src must be a contiguous CUDA tensor")
    check(_lib.lib().b200_ep_put(_p(src), src.numel() * src.element_size(), int(dst_offset_bytes), _ptr_array(peer_ptrs),
                                 len(peer_ptrs), _stream()), "b200_ep_put")


def ep_barrier(peer_flags, epochs, rank, channel, timeout_ns=200_000_000, status=None):
    """Barrier among the ranks of an expert-parallel group as one small kernel with a bounded wait (`peer_flags`:
    device pointers of every rank's flag array; `epochs`: this rank's private uint64 counters)."""
    _need(epochs, torch.int64, "epochs", 1)
    check(_lib.lib().b200_ep_barrier(_ptr_array(peer_flags), _p(epochs), len(peer_flags), int(rank), int(channel),
                                     int(timeout_ns), _p(status), _stream()), "b200_ep_barrier")


def set_wait_budget_ns(ns: int) -> None:
    """Budget of the device-side waits of kernels launched on the current device from now on (0: the default, 1 s)."""
    check(_lib.lib().b200_set_wait_budget_ns(int(ns)), "b200_set_wait_budget_ns")


def selftest_wait_expiry(status) -> None:
    """Launches a one-CTA kernel whose wait can never succeed; `status` reads B200_ST_WAIT_FULL (101) afterwards."""
    check(_lib.lib().b200_selftest_wait_expiry(_p(status), _stream()), "b200_selftest_wait_expiry")


def moe_combine(cache, x, gate_w, top_k, pos=None, out=None):
    """Sum of the routed rows + sigmoid-gated shared row (reference: i8x_dec_combine)."""
    _need(cache, torch.bfloat16, "cache", 2)
    _need(x, torch.bfloat16, "x", 2)
    T, H = x.shape
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    check(_lib.lib().b200_moe_combine(_p(cache), _p(x), _p(gate_w), _p(pos), T, H, top_k, _p(out), _stream()),
          "b200_moe_combine")
    return out


def gdn_ring_fold(checkpoint, d_ring, dlo_ring, k_ring, klo_ring, g_ring, state_idx, ring_idx, write_pos, cache_base):
    """Folds the committed ring entries into the checkpoints in place (the engine-side step of the ring layout,
    gdn_fused.py:24); the caller resets `write_pos` afterwards."""
    _need(checkpoint, torch.float32, "checkpoint", 4)
    for name, t in (("d_ring", d_ring), ("dlo_ring", dlo_ring), ("k_ring", k_ring), ("klo_ring", klo_ring)):
        _need(t, torch.bfloat16, name, 4)
    _need(g_ring, torch.float32, "g_ring", 3)
    for name, t in (("state_idx", state_idx), ("ring_idx", ring_idx), ("write_pos", write_pos), ("cache_base", cache_base)):
        _need(t, torch.int32, name, 1)
    check(_lib.lib().b200_gdn_ring_fold(_p(checkpoint), _p(d_ring), _p(dlo_ring), _p(k_ring), _p(klo_ring), _p(g_ring),
                                        _p(state_idx), _p(ring_idx), _p(write_pos), _p(cache_base), state_idx.shape[0],
                                        _stream()), "b200_gdn_ring_fold")


def attn_front(x, w, w_s, q_norm_w, k_norm_w, positions, cos_sin, eps=1e-6, out_fp8=True, ws=None, status=None,
               quantised=None):
    """Fused QKV + gate projection with q/k RMSNorm and partial RoPE (reference: fp8.linear_q followed by
    qk_attn_verify.attn_prefill_front).  Returns (q [T,16,256], gate bf16 [T,16,256], k, v [T,2,256]);
    q, k, v are uint8 e4m3 codes when out_fp8 else bf16.  `quantised` = (xq, xs) of the same rows as left by
    `moe_combine_norm(quantised=...)`: the activation quantiser launch is skipped."""
    _need(x, torch.bfloat16, "x", 2)
    _need(w, torch.uint8, "w", 2)
    _need(w_s, torch.float32, "w_s", 2)
    _need(positions, torch.int64, "positions", 1)
    _need(cos_sin, torch.float32, "cos_sin", 2)
    T = x.shape[0]
    if x.shape[1] != 2048 or tuple(w.shape) != (9216, 2048) or tuple(w_s.shape) != (72, 16) or cos_sin.shape[1] != 64:
        raise B200Error("attn_front: expected x [T,2048], w [9216,2048], w_s [72,16], cos_sin [max_pos,64]")
    dt = torch.uint8 if out_fp8 else torch.bfloat16
    q = torch.empty(T, 16, 256, dtype=dt, device=x.device)
    k = torch.empty(T, 2, 256, dtype=dt, device=x.device)
    v = torch.empty(T, 2, 256, dtype=dt, device=x.device)
    gate = torch.empty(T, 16, 256, dtype=torch.bfloat16, device=x.device)
    if quantised is not None:
        xq, xs = quantised
        _need(xq, torch.uint8, "xq", 2)
        _need(xs, torch.float32, "xs", 2)
        if tuple(xq.shape) != (T, 2048) or tuple(xs.shape) != (T, 16):
            raise B200Error("attn_front: quantised rows must be [T, 2048] and [T, 16]")
        check(_lib.lib().b200_attn_front_q(_p(xq), _p(xs), T, _p(w), _p(w_s), _p(q_norm_w), _p(k_norm_w), _p(positions),
                                           _p(cos_sin), cos_sin.shape[0], float(eps), 1 if out_fp8 else 0, _p(q), _p(gate),
                                           _p(k), _p(v), _p(status), _stream()), "b200_attn_front_q")
        return q, gate, k, v
    if ws is None:
        n = _lib.lib().b200_attn_front_workspace_bytes(T)
        buf = torch.empty(n + 1024, dtype=torch.uint8, device=x.device)
        off = (-buf.data_ptr()) % 1024
        ws = buf[off:off + n]
    check(_lib.lib().b200_attn_front(_p(x), T, _p(w), _p(w_s), _p(q_norm_w), _p(k_norm_w), _p(positions), _p(cos_sin),
                                     cos_sin.shape[0], float(eps), 1 if out_fp8 else 0, _p(q), _p(gate), _p(k), _p(v),
                                     _p(ws), ws.numel(), _p(status), _stream()), "b200_attn_front")
    return q, gate, k, v


def moe_combine_norm(cache, x, gate_w, top_k, residual, norm_w, eps=1e-6, pos=None, out=None, normed=None, quantised=None):
    """Combine with the next layer's input norm folded in (reference: qk_route.combine_norm): `residual` is updated
    in place to bf16(out + residual); returns (out, normed).  `quantised` = (xq uint8 [T, H], xs fp32 [T, H/128]):
    the normed rows are also written there in the e4m3 form that `dense_fp8_split_q` / `attn_front_q` read."""
    _need(cache, torch.bfloat16, "cache", 2)
    _need(x, torch.bfloat16, "x", 2)
    _need(residual, torch.bfloat16, "residual", 2)
    _need(norm_w, torch.bfloat16, "norm_w", 1)
    T, H = x.shape
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    if normed is None:
        normed = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    if quantised is not None:
        xq, xs = quantised
        _need(xq, torch.uint8, "xq", 2)
        _need(xs, torch.float32, "xs", 2)
        if tuple(xq.shape) != (T, H) or tuple(xs.shape) != (T, H // 128):
            raise B200Error("moe_combine_norm: quantised outputs must be [T, H] and [T, H/128]")
        check(_lib.lib().b200_moe_combine_norm_q(_p(cache), _p(x), _p(gate_w), _p(pos), T, H, int(top_k), _p(out),
                                                 _p(residual), _p(norm_w), float(eps), _p(normed), _p(xq), _p(xs),
                                                 _stream()), "b200_moe_combine_norm_q")
        return out, normed
    check(_lib.lib().b200_moe_combine_norm(_p(cache), _p(x), _p(gate_w), _p(pos), T, H, int(top_k), _p(out), _p(residual),
                                           _p(norm_w), float(eps), _p(normed), _stream()), "b200_moe_combine_norm")
    return out, normed


def attn_verify(q, gate, k_new, v_new, kcache, vcache, page_table, seqlens, scale=None, splits=None, out=None, ws=None,
                status=None):
    """Attention verify core over paged e4m3 KV (reference: qk_attn_verify.attn_verify_fused).  q uint8 [4B,16,256],
    gate bf16 [4B,16,256], k_new / v_new uint8 [4B,2,256]; kcache uint8 [P,2,128,256], vcache uint8 [P,2,256,128]
    (both updated in place with the new tokens); page_table int32 [B,n]; seqlens int32 [B] including the 4
    drafts.  Returns out bf16 [4B, 4096]."""
    _need(q, torch.uint8, "q", 3)
    _need(gate, torch.bfloat16, "gate", 3)
    _need(k_new, torch.uint8, "k_new", 3)
    _need(v_new, torch.uint8, "v_new", 3)
    _need(kcache, torch.uint8, "kcache", 4)
    _need(vcache, torch.uint8, "vcache", 4)
    _need(page_table, torch.int32, "page_table", 2)
    _need(seqlens, torch.int32, "seqlens", 1)
    B = seqlens.shape[0]
    if scale is None:
        scale = 1.0 / 16.0
    if splits is None:
        splits = _lib.lib().b200_attn_verify_splits(B)
    if out is None:
        out = torch.empty(4 * B, 4096, dtype=torch.bfloat16, device=q.device)
    if ws is None:
        n = _lib.lib().b200_attn_verify_workspace_bytes(B, splits)
        ws = torch.empty(n, dtype=torch.uint8, device=q.device)
    check(_lib.lib().b200_attn_verify(_p(q), _p(gate), _p(k_new), _p(v_new), _p(kcache), _p(vcache), kcache.shape[0],
                                      _p(page_table), page_table.shape[1], _p(seqlens), B, float(scale), int(splits),
                                      _p(out), _p(ws), ws.numel(), _p(status), _stream()), "b200_attn_verify")
    return out


def dense_fp8_workspace(T, H, device):
    n = _lib.lib().b200_dense_fp8_workspace_bytes(T, H)
    buf = torch.empty(n + 1024, dtype=torch.uint8, device=device)
    off = (-buf.data_ptr()) % 1024
    return buf[off:off + n]


def dense_fp8(x, w, w_s, out=None, ws=None, status=None):
    """Decode-width projection out = bf16(x . W^T) with an fp8 block-scaled weight, any number of rows (reference: qk_proj_decode gdn_in_proj / qkv_proj / dense8)."""
    _need(x, torch.bfloat16, "x", 2)
    _need(w, torch.uint8, "w", 2)
    _need(w_s, torch.float32, "w_s", 2)
    T, H = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    if ws is None:
        ws = dense_fp8_workspace(T, H, x.device)
    check(_lib.lib().b200_dense_fp8(_p(x), T, H, _p(w), _p(w_s), N, _p(out), _p(ws), ws.numel(), _p(status),
                                    _stream()), "b200_dense_fp8")
    return out


def dense_fp8_split(x, w, w_s, widths, outs=None, ws=None, status=None, quantised=None):
    """dense_fp8 with the N output features cut into up to four consecutive segments (`widths`), each written to
    its own contiguous tensor [T, width] (the GDN in_proj's [q k v | z | b | a], dense8.py:64-68)."""
    _need(x, torch.bfloat16, "x", 2)
    _need(w, torch.uint8, "w", 2)
    _need(w_s, torch.float32, "w_s", 2)
    T, H = x.shape
    N = w.shape[0]
    n = len(widths)
    if outs is None:
        outs = [torch.empty(T, wd, dtype=torch.bfloat16, device=x.device) for wd in widths]
    for o, wd in zip(outs, widths):
        _need(o, torch.bfloat16, "segment output", 2)
        if tuple(o.shape) != (T, wd):
            raise B200Error("dense_fp8_split: a segment output must be [T, width]")
    cols = (C.c_int * n)(*[int(v) for v in widths])
    lds = (C.c_int * n)(*[int(v) for v in widths])
    if quantised is not None:   # the rows as left by moe_combine_norm(quantised=...): no activation quantiser launch
        xq, xs = quantised
        _need(xq, torch.uint8, "xq", 2)
        _need(xs, torch.float32, "xs", 2)
        if tuple(xq.shape) != (T, H) or tuple(xs.shape) != (T, H // 128):
            raise B200Error("dense_fp8_split: quantised rows must be [T, H] and [T, H/128]")
        check(_lib.lib().b200_dense_fp8_split_q(_p(xq), _p(xs), T, H, _p(w), _p(w_s), N, n, cols,
                                                _ptr_array([o.data_ptr() for o in outs]), lds, _p(status), _stream()),
              "b200_dense_fp8_split_q")
        return outs
    if ws is None:
        ws = dense_fp8_workspace(T, H, x.device)
    check(_lib.lib().b200_dense_fp8_split(_p(x), T, H, _p(w), _p(w_s), N, n, cols, _ptr_array([o.data_ptr() for o in outs]),
                                          lds, _p(ws), ws.numel(), _p(status), _stream()), "b200_dense_fp8_split")
    return outs


def dense_fp8_add_rmsnorm_workspace(T, K, N, device):
    n = _lib.lib().b200_dense_fp8_add_rmsnorm_workspace_bytes(T, K, N)
    buf = torch.empty(n + 1024, dtype=torch.uint8, device=device)
    off = (-buf.data_ptr()) % 1024
    return buf[off:off + n]


def dense_fp8_add_rmsnorm(x, w, w_s, residual, norm_w, eps=1e-6, out=None, proj_out=None, ws=None, status=None):
    """A mixer's output projection fused with the residual add and the norm behind it (reference:
    proj.project_add_norm): split-K fp8 GEMM into fp32 partials, then one kernel that sums them, rounds the projection
    to bf16, adds it to `residual` in place and norms.  Returns the normed rows bf16 [T, N]."""
    _need(x, torch.bfloat16, "x", 2)
    _need(w, torch.uint8, "w", 2)
    _need(w_s, torch.float32, "w_s", 2)
    _need(residual, torch.bfloat16, "residual", 2)
    _need(norm_w, torch.bfloat16, "norm_w", 1)
    T, K = x.shape
    N = w.shape[0]
    if tuple(residual.shape) != (T, N):
        raise B200Error("dense_fp8_add_rmsnorm: residual must be [T, N]")
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    if ws is None:
        ws = dense_fp8_add_rmsnorm_workspace(T, K, N, x.device)
    check(_lib.lib().b200_dense_fp8_add_rmsnorm(_p(x), T, K, _p(w), _p(w_s), N, _p(residual), _p(norm_w), float(eps), _p(out),
                                                _p(proj_out), _p(ws), ws.numel(), _p(status), _stream()),
          "b200_dense_fp8_add_rmsnorm")
    return out


def add_rmsnorm(proj, residual, w, eps=1e-6, out=None):
    """residual <- bf16(proj + residual); returns bf16(residual * rstd * (1 + w)) (reference: proj.project_add_norm)."""
    _need(proj, torch.bfloat16, "proj", 2)
    _need(residual, torch.bfloat16, "residual", 2)
    T, H = proj.shape
    if out is None:
        out = torch.empty_like(proj)
    check(_lib.lib().b200_add_rmsnorm(_p(proj), _p(residual), _p(w), float(eps), T, H, _p(out), _stream()),
          "b200_add_rmsnorm")
    return out


def lmhead_workspace(T, H, V, device):
    n = _lib.lib().b200_lmhead_workspace_bytes(T, H, V)
    buf = torch.empty(n + 1024, dtype=torch.uint8, device=device)
    off = (-buf.data_ptr()) % 1024
    return buf[off:off + n]


def lmhead_argmax(x, w, w_s, shard_lo=0, want_logits=False, ws=None, status=None):
    """One vocabulary shard of the fp8 LM head with the argmax fused in (reference: the logits GEMM of
    qwen36_lmhead8; the argmax has no counterpart there).  Returns (max fp32 [T], idx int32 [T], logits or None)."""
    _need(x, torch.bfloat16, "x", 2)
    _need(w, torch.uint8, "w", 2)
    _need(w_s, torch.float32, "w_s", 2)
    T, H = x.shape
    V = w.shape[0]
    mx = torch.empty(T, dtype=torch.float32, device=x.device)
    idx = torch.empty(T, dtype=torch.int32, device=x.device)
    logits = torch.empty(T, V, dtype=torch.float32, device=x.device) if want_logits else None
    if ws is None:
        ws = lmhead_workspace(T, H, V, x.device)
    check(_lib.lib().b200_lmhead_argmax(_p(x), T, H, _p(w), _p(w_s), V, int(shard_lo), _p(mx), _p(idx), _p(logits),
                                        _p(ws), ws.numel(), _p(status), _stream()), "b200_lmhead_argmax")
    return mx, idx, logits


def argmax_merge(maxes, idxs):
    """[S, T] shard maxima and ids -> tokens int32 [T] (largest value, ties to the lower id)."""
    _need(maxes, torch.float32, "maxes", 2)
    _need(idxs, torch.int32, "idxs", 2)
    S, T = maxes.shape
    tokens = torch.empty(T, dtype=torch.int32, device=maxes.device)
    check(_lib.lib().b200_argmax_merge(_p(maxes), _p(idxs), S, T, _p(tokens), _stream()), "b200_argmax_merge")
    return tokens


def gdn_workspace(B, device):
    n = _lib.lib().b200_gdn_workspace_bytes(B)
    buf = torch.empty(n + 128, dtype=torch.uint8, device=device)
    off = (-buf.data_ptr()) % 128
    return buf[off:off + n]


def gdn_verify(mixed, z, a, b, conv_state, conv_w, a_log, dt_bias, state, accepted, norm_w, eps=1e-6, out=None,
               status=None, ws=None):
    """Gated DeltaNet verify over 4 draft tokens; updates `state` and `conv_state` in place to the
    accepted length (reference: qk_gdn_verify.gdn_verify_fused).  Returns out bf16 [B*4, 4096]."""
    _need(mixed, torch.bfloat16, "mixed", 2)
    _need(state, torch.float32, "state", 4)
    _need(conv_state, torch.bfloat16, "conv_state", 3)
    _need(accepted, torch.int32, "accepted", 1)
    B = state.shape[0]
    if tuple(mixed.shape) != (B * 4, 8192) or tuple(state.shape) != (B, 32, 128, 128) or \
            tuple(conv_state.shape) != (B, 8192, 3):
        raise B200Error(f"gdn_verify: unexpected shapes mixed={tuple(mixed.shape)} state={tuple(state.shape)} "
                        f"conv_state={tuple(conv_state.shape)}")
    if out is None:
        out = torch.empty(B * 4, 4096, dtype=torch.bfloat16, device=mixed.device)
    if ws is None:
        ws = gdn_workspace(B, mixed.device)
    check(_lib.lib().b200_gdn_verify(_p(mixed), _p(z), _p(a), _p(b), _p(conv_state), _p(conv_w), _p(a_log),
                                     _p(dt_bias), _p(state), _p(accepted), _p(norm_w), float(eps), B, _p(out),
                                     _p(ws), ws.numel(), _p(status), _stream()), "b200_gdn_verify")
    return out


def gdn_verify_replay(mixed, z, a, b, conv_state, conv_w, window, a_log, dt_bias, checkpoint, d_ring, dlo_ring, k_ring,
                      klo_ring, g_ring, state_idx, ring_idx, win_idx, write_pos, cache_base, norm_w, eps=1e-6,
                      out=None, status=None, ws=None):
    """Gated DeltaNet verify on the checkpoint + (d, k, g) ring state layout (reference:
    qk_gdn_verify.gdn_verify_fused, gdn_fused.py:37-57): reads the checkpoint and the committed ring
    entries, appends this window's entries, rolls `conv_state` and records the draft windows in place.
    Returns out bf16 [B*4, 4096]."""
    _need(mixed, torch.bfloat16, "mixed", 2)
    _need(checkpoint, torch.float32, "checkpoint", 4)
    _need(conv_state, torch.bfloat16, "conv_state", 3)
    _need(window, torch.bfloat16, "window", 3)
    for name, t in (("d_ring", d_ring), ("dlo_ring", dlo_ring), ("k_ring", k_ring), ("klo_ring", klo_ring)):
        _need(t, torch.bfloat16, name, 4)
    _need(g_ring, torch.float32, "g_ring", 3)
    for name, t in (("state_idx", state_idx), ("ring_idx", ring_idx), ("win_idx", win_idx), ("write_pos", write_pos),
                    ("cache_base", cache_base)):
        _need(t, torch.int32, name, 1)
    B = state_idx.shape[0]
    slots, rslots = checkpoint.shape[0], g_ring.shape[0]
    if tuple(mixed.shape) != (B * 4, 8192) or tuple(checkpoint.shape) != (slots, 32, 128, 128) or \
            tuple(conv_state.shape) != (slots, 8192, 3) or tuple(window.shape[1:]) != (8192, 6) or \
            tuple(d_ring.shape) != (rslots, 32, 16, 128) or tuple(dlo_ring.shape) != (rslots, 32, 16, 128) or \
            tuple(k_ring.shape) != (rslots, 16, 16, 128) or tuple(klo_ring.shape) != (rslots, 16, 16, 128) or \
            tuple(g_ring.shape) != (rslots, 32, 16) or ring_idx.shape[0] != B or win_idx.shape[0] != B or \
            write_pos.shape[0] != rslots or cache_base.shape[0] != rslots:
        raise B200Error("gdn_verify_replay: unexpected shapes")
    if out is None:
        out = torch.empty(B * 4, 4096, dtype=torch.bfloat16, device=mixed.device)
    if ws is None:
        ws = gdn_workspace(B, mixed.device)
    check(_lib.lib().b200_gdn_verify_replay(
        _p(mixed), _p(z), _p(a), _p(b), _p(conv_state), _p(conv_w), _p(window), _p(a_log), _p(dt_bias), _p(checkpoint),
        slots, _p(d_ring), _p(dlo_ring), _p(k_ring), _p(klo_ring), _p(g_ring), _p(state_idx), _p(ring_idx), _p(win_idx),
        _p(write_pos), _p(cache_base), _p(norm_w), float(eps), B, _p(out), _p(ws), ws.numel(), _p(status), _stream()),
        "b200_gdn_verify_replay")
    return out
