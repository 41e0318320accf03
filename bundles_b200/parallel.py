"""Multi-GPU partitioning of the hot path on one node: expert-parallel MoE and the vocab-sharded
LM head.  One process per GPU, `torch.distributed` (NCCL on GPUs, gloo in the CPU tests).

The reference is single-GPU (it raises for TP != 1: layer.py:396-402) and has no collective at all,
so there is no reference call to mirror here; the partitioning is the one the target names:
experts split evenly over ranks (expert e lives on rank e // E_local), vocabulary rows split on
128-row scale-block boundaries.

Expert-parallel step, exact by construction:
  1. every rank routes its own tokens; x, ids and weights are all-gathered (a token is needed by
     up to min(K, world) ranks, so for K >= world gathering each row once moves no more bytes than a
     per-destination all-to-all would);
  2. every rank builds the routing lists of ITS experts over all tokens, runs their MLPs and writes
     bf16(y * w) into a zero-initialised cache [T_all * K, H] at the global slot t * K + j;
  3. the cache is reduce-scattered (sum): every slot is non-zero on exactly one rank and x + 0 == x,
     so each home rank receives its tokens' K rows bit-exactly, whatever the reduction order;
  4. the home rank adds the K rows in slot order and the sigmoid-gated shared-expert row (computed
     locally for its own tokens), exactly as the single-GPU combine does.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def expert_range(n_experts: int, rank: int, world: int):
    if n_experts % world:
        raise ValueError(f"{n_experts} experts do not split evenly over {world} ranks")
    per = n_experts // world
    return rank * per, per


def vocab_shards(vocab: int, world: int, block: int = 128):
    """Row ranges per rank, cut on 128-row scale-block boundaries; the first (blocks % world) ranks
    take one block more (151936 rows over 8 ranks -> 3 x 19072 + 5 x 18944)."""
    nb = (vocab + block - 1) // block
    base, extra = divmod(nb, world)
    out, lo = [], 0
    for r in range(world):
        hi = min(vocab, lo + (base + (1 if r < extra else 0)) * block)
        out.append((lo, hi))
        lo = hi
    return out


class ExpertParallelMoe:
    """Expert-parallel MoE block.  `local` is the compute backend of this rank:
        local.route(x) -> (ids int32 [T,K], wts fp32 [T,K])                      (all experts' router)
        local.experts(x_all, ids_all, wts_all, cache_all) -> None                (fills this rank's slots, routed only)
        local.shared_and_combine(x, routed_rows [T*K,H]) -> out bf16 [T,H]       (shared expert + combine, own tokens)
    On GPUs the backend wraps the C-ABI operators (`GpuMoeBackend`); the CPU tests plug the oracle in.
    """

    def __init__(self, local, top_k: int, hidden: int, group=None):
        self.local, self.K, self.H, self.group = local, top_k, hidden, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        T, H = x.shape
        W, K = self.world, self.K
        ids, wts = self.local.route(x)
        x_all = torch.empty(W * T, H, dtype=x.dtype, device=x.device)
        ids_all = torch.empty(W * T, K, dtype=ids.dtype, device=x.device)
        wts_all = torch.empty(W * T, K, dtype=wts.dtype, device=x.device)
        dist.all_gather_into_tensor(x_all, x.contiguous(), group=self.group)
        dist.all_gather_into_tensor(ids_all, ids.contiguous(), group=self.group)
        dist.all_gather_into_tensor(wts_all, wts.contiguous(), group=self.group)
        cache_all = torch.zeros(W * T * K, H, dtype=x.dtype, device=x.device)
        self.local.experts(x_all, ids_all, wts_all, cache_all)
        if dist.get_backend(self.group) == "gloo":   # gloo has no reduce-scatter: all-reduce and keep our slice
            dist.all_reduce(cache_all, op=dist.ReduceOp.SUM, group=self.group)
            mine = cache_all[self.rank * T * K:(self.rank + 1) * T * K]
        else:
            mine = torch.empty(T * K, H, dtype=x.dtype, device=x.device)
            dist.reduce_scatter_tensor(mine, cache_all, op=dist.ReduceOp.SUM, group=self.group)
        return self.local.shared_and_combine(x, mine)

    __call__ = forward


class GpuMoeBackend:
    """This rank's share of an int8 W8A8 MoE layer on its GPU, through the C-ABI operators."""

    def __init__(self, wr, weights, gate_w, top_k, e_lo, bias=None):
        from . import ops
        self.ops = ops
        self.wr, self.w, self.gate_w, self.K, self.e_lo, self.bias = wr, weights, gate_w, top_k, e_lo, bias
        self.E_local = weights.w13.shape[0]
        self.status = ops.new_status(wr.device)
        self._lists = {}
        # the shared expert runs on the home rank only: a weights view without / with only the shared expert
        self.w_routed = ops.MoeW8A8Weights(weights.w13, weights.s13, weights.w2, weights.s2)
        self.launches_per_call = 14

    def _get_lists(self, T, shared):
        key = (T, shared)
        if key not in self._lists:
            self._lists[key] = self.ops.RoutingLists(T, self.K, self.E_local, 128, self.wr.device)
        return self._lists[key]

    def route(self, x):
        _, ids, wts = self.ops.router(x, self.wr, self.K, self.bias, want_logits=False)
        return ids, wts

    def experts(self, x_all, ids_all, wts_all, cache_all):
        T = x_all.shape[0]
        lists = self._get_lists(T, False)
        self.ops.build_lists(ids_all, wts_all, lists, None, e_lo=self.e_lo, with_shared=False)
        # the kernel addresses cache rows by slot < T*(K+1); only routed slots are written here
        self.ops.moe_w8a8(x_all, self.w_routed, lists, cache=cache_all, status=self.status)

    def shared_and_combine(self, x, routed_rows):
        ops = self.ops
        T, H = x.shape
        K = self.K
        cache = torch.empty(T * (K + 1), H, dtype=x.dtype, device=x.device)
        cache[:T * K].copy_(routed_rows)
        # shared expert only: lists with no routed pair (ids outside this rank's window) + the shared rows
        lists = self._get_lists(T, True)
        none_ids = torch.full((T, K), -1, dtype=torch.int32, device=x.device)
        zero_w = torch.zeros(T, K, dtype=torch.float32, device=x.device)
        ops.build_lists(none_ids, zero_w, lists, None, e_lo=0, with_shared=True)
        w_sh = ops.MoeW8A8Weights(self.w.w13, self.w.s13, self.w.w2, self.w.s2, self.w.sh13, self.w.shs13,
                                  self.w.sh2, self.w.shs2)
        ops.moe_w8a8(x, w_sh, lists, cache=cache, status=self.status)
        return ops.moe_combine(cache, x, self.gate_w, K)


EP_CHANNELS = 4   # B200_EP_CHANNELS of the C ABI


class EpGroup:
    """Buffers that every rank of an expert-parallel group can store into, and the barrier among the ranks.
    One process per GPU; the buffers are symmetric memory (`torch.distributed._symmetric_memory`: one allocation per
    rank, each mapped into every process), the barrier is the library's own one-warp kernel (`ops.ep_barrier`):
    peer stores of an epoch counter, a poll bounded by `timeout_ns` that ends with status B200_ST_WAIT_PEER
    instead of spinning on (torch's symmetric-memory barrier spins without a limit, or traps the GPU when
    given one).  `shared()` must be called in the same order with the same shapes on every rank."""

    def __init__(self, group=None, device=None, timeout_ns=1_000_000_000):
        import torch.distributed._symmetric_memory as symm
        from . import ops
        self._symm, self._ops = symm, ops
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.timeout_ns = int(timeout_ns)
        self.flags, self.peer_flags = self.shared((EP_CHANNELS * 8,), torch.int64, zero=True)
        self.epochs = torch.zeros(EP_CHANNELS, dtype=torch.int64, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)       # nobody signals before every flag array is zero

    def shared(self, shape, dtype, zero=False):
        """(this rank's tensor, [device pointer of every rank's tensor as mapped into this process])."""
        t = self._symm.empty(*shape, dtype=dtype, device=self.device)
        if zero:
            t.zero_()
        handle = self._symm.rendezvous(t, self.group)
        return t, [int(p) for p in handle.buffer_ptrs]

    def barrier(self, channel, status=None):
        self._ops.ep_barrier(self.peer_flags, self.epochs, self.rank, channel, self.timeout_ns, status)


class VirtualEpGroup:
    """The ranks of an expert-parallel group emulated in ONE process on ONE GPU, for checking the expert-parallel
    data path (per-rank lists, peer destinations of the down GEMM, gathered buffers) where there is a single GPU:
    every virtual rank has its own buffers in the same device memory, "peer" pointers are simply the other virtual
    ranks' buffers, and the ranks' steps are run in lockstep on one stream (`run_lockstep`), phase by phase, so that
    stream order stands in for the barriers (kernels that wait on one another must never run as separate launches
    on one GPU, so the barrier kernel is not launched here)."""

    def __init__(self, world, device):
        self.world, self.device = int(world), torch.device(device)
        self._bufs = []

    def view(self, rank):
        return _VirtualRank(self, int(rank))


class _VirtualRank:
    def __init__(self, parent, rank):
        self.parent, self.rank, self.world, self.device = parent, rank, parent.world, parent.device
        self._n = 0

    def shared(self, shape, dtype, zero=False):
        i, bufs = self._n, self.parent._bufs
        self._n += 1
        if len(bufs) <= i:
            bufs.append([torch.zeros(*shape, dtype=dtype, device=self.device) for _ in range(self.world)])
        if tuple(bufs[i][0].shape) != tuple(shape) or bufs[i][0].dtype != dtype:
            raise ValueError("virtual ranks must request their shared buffers in the same order and shapes")
        return bufs[i][self.rank], [t.data_ptr() for t in bufs[i]]

    def barrier(self, channel, status=None):
        pass


class RankLost(RuntimeError):
    """A rank of the expert-parallel group did not report for a step in time."""


class StepGate:
    """Host-side roll call before an expert-parallel step.  Every rank posts the number of the step it is about to
    launch into a `torch.distributed` store and then reads its peers' entries; a peer that has not posted within
    `timeout_s` makes `sync` raise `RankLost` BEFORE this rank launches kernels that would wait for that peer on
    the device (where the wait is bounded too, but costs a whole step's worth of garbage).  A rank that leaves does
    so between steps, with none of its kernels in flight."""

    def __init__(self, store, rank, world, timeout_s=5.0, prefix="b200/step", poll_s=0.002):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.timeout_s, self.prefix, self.poll_s = float(timeout_s), prefix, float(poll_s)
        self.step = 0

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def sync(self):
        """Post the next step's number and wait for every peer to have posted it (or a later one)."""
        import time
        self.step += 1
        self.store.set(self._key(self.rank), str(self.step))
        deadline = time.monotonic() + self.timeout_s
        for r in range(self.world):
            if r == self.rank:
                continue
            while True:
                if self.store.check([self._key(r)]) and int(self.store.get(self._key(r))) >= self.step:
                    break
                if time.monotonic() > deadline:
                    raise RankLost(f"rank {r} did not report for step {self.step} within {self.timeout_s} s")
                time.sleep(self.poll_s)
        return self.step


def run_lockstep(generators):
    """Advance the per-rank step generators of a VirtualEpGroup phase by phase (every generator yields at each
    point where the real group runs a barrier); returns their return values."""
    results = [None] * len(generators)
    live = list(range(len(generators)))
    while live:
        for i in list(live):
            try:
                next(generators[i])
            except StopIteration as stop:
                results[i] = stop.value
                live.remove(i)
    return results


class FusedExpertParallelMoe:
    """Expert-parallel MoE block whose combine-side exchange is fused into the down GEMM: every rank
    stores the weighted expert rows straight into the home rank's cache over NVLink (plain peer
    stores from the GEMM epilogue, `ops.moe_w8a8_ep`), then one barrier, then the home rank adds its
    tokens' rows in slot order.  The caches are symmetric-memory buffers (one per rank, mapped into
    every process); token rows and routing reach every rank's gathered buffers by peer stores too
    (`ops.ep_push`; each token row is needed by up to min(K, world) ranks), so the step contains no NCCL
    call.  The shared expert runs in the same launches, for this rank's own tokens only.
    The whole step is captured into a CUDA graph on first use.  Bit-identical to `ExpertParallelMoe`
    and to the single-GPU block."""

    def __init__(self, backend: "GpuMoeBackend", top_k: int, hidden: int, tokens_per_rank: int, group=None,
                 use_graph=True, ep=None):
        self.b, self.K, self.H, self.T = backend, top_k, hidden, tokens_per_rank
        dev = backend.wr.device
        self.ep = ep if ep is not None else EpGroup(group, dev)
        self.world, self.rank = self.ep.world, self.ep.rank
        self.group = getattr(self.ep, "group", group)
        # rows of this rank's tokens: K routed rows per token (written by every rank) + the shared-expert row
        self.cache, self.peer_ptrs = self.ep.shared((tokens_per_rank * (top_k + 1), hidden), torch.bfloat16)
        T_all = tokens_per_rank * self.world
        # the gathered tokens and routing of all ranks: every rank stores its share into every rank's buffers
        self.x_all, self.peer_x = self.ep.shared((T_all, hidden), torch.bfloat16)
        self.ids_all, self.peer_ids = self.ep.shared((T_all, top_k), torch.int32)
        self.wts_all, self.peer_wts = self.ep.shared((T_all, top_k), torch.float32)
        self.lists = backend.ops.RoutingLists(T_all, top_k, backend.E_local, 128, dev)
        self.ws = backend.ops.moe_w8a8_workspace(T_all, hidden, backend.w.w2.shape[-1], top_k, dev)
        self.x_static = torch.empty(tokens_per_rank, hidden, dtype=torch.bfloat16, device=dev)
        self.out = torch.empty(tokens_per_rank, hidden, dtype=torch.bfloat16, device=dev)
        self.use_graph, self.graph = use_graph, None
        self._pipe = None
        self.launches_per_call = 11  # router x2, dispatch, barrier, lists, quantise, up, h-quantise, down, barrier, combine

    def _step(self):
        b, ops, K = self.b, self.b.ops, self.K
        x = self.x_static
        ids, wts = b.route(x)
        # dispatch: peer stores into every rank's gathered buffers; the barrier below makes them visible and
        # also tells that nobody still reads last step's rows when the first peer store of this step lands
        ops.ep_push(x, ids, wts, self.rank, self.peer_x, self.peer_ids, self.peer_wts)
        self.ep.barrier(0, b.status)
        ops.build_lists(self.ids_all, self.wts_all, self.lists, None, e_lo=b.e_lo,
                        shared_range=(self.rank * self.T, self.T))   # the shared expert runs for this rank's own tokens
        ops.moe_w8a8_ep(self.x_all, b.w, self.lists, self.peer_ptrs, self.rank, self.T, ws=self.ws, status=b.status)
        self.ep.barrier(1, b.status)        # every rank's rows for my tokens have landed
        ops.moe_combine(self.cache, x, b.gate_w, K, out=self.out)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self.x_static.copy_(x, non_blocking=True)
        if not self.use_graph:
            self._step()
            return self.out
        if self.graph is None:
            self._step()                    # warm-up: one-time set-up inside the operators and NCCL
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._step()
            self.graph = g
        self.graph.replay()
        return self.out

    __call__ = forward

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """Host-to-host form: this rank's pinned `x_host` in, its pinned `out_host` out, asynchronously.  The
        copy-in of call i + 1 and the copy-out of call i - 1 run on their own streams beside the step of call i
        (two staging buffers each way; the step itself keeps its single captured graph)."""
        dev = self.x_static.device
        main = torch.cuda.current_stream(dev)
        if self._pipe is None:
            mk = lambda: torch.empty_like(self.x_static)
            self._pipe = dict(i=0, s_in=torch.cuda.Stream(dev), s_out=torch.cuda.Stream(dev),
                              slots=[dict(x=mk(), out=mk(), in_ready=torch.cuda.Event(), taken=torch.cuda.Event(),
                                          done=torch.cuda.Event(), out_free=torch.cuda.Event(), used=False)
                                     for _ in range(2)])
        pipe = self._pipe
        slot = pipe["slots"][pipe["i"] & 1]
        pipe["i"] += 1
        with torch.cuda.stream(pipe["s_in"]):
            if slot["used"]:
                pipe["s_in"].wait_event(slot["taken"])     # the step two back has taken its input out of this buffer
            slot["x"].copy_(x_host, non_blocking=True)
            slot["in_ready"].record()
        main.wait_event(slot["in_ready"])
        out = self.forward(slot["x"])
        slot["taken"].record(main)
        if slot["used"]:
            main.wait_event(slot["out_free"])
        slot["out"].copy_(out, non_blocking=True)
        slot["done"].record(main)
        with torch.cuda.stream(pipe["s_out"]):
            pipe["s_out"].wait_event(slot["done"])
            out_host.copy_(slot["out"], non_blocking=True)
            slot["out_free"].record()
        slot["used"] = True

    def join_host(self) -> None:
        """Make the current stream wait for every pending copy-out of `forward_host` (no host blocking)."""
        if self._pipe is not None:
            main = torch.cuda.current_stream(self.x_static.device)
            for slot in self._pipe["slots"]:
                if slot["used"]:
                    main.wait_event(slot["out_free"])

    def close(self):
        """Drop the captured graph.  Call before `destroy_process_group`: NCCL does not finish
        destroying a communicator while a live CUDA graph still holds its kernels."""
        if self.graph is not None:
            torch.cuda.synchronize()
            self.graph = None


def sharded_argmax(x, w_shard, w_s_shard, shard_lo, group=None):
    """Vocab-sharded greedy token: per-shard (max, argmax) on this rank, all-gather of the pairs,
    merge (largest value, ties to the lower id).  Returns tokens int32 [T] (same on every rank)."""
    from . import ops
    world = dist.get_world_size(group)
    mx, idx, _ = ops.lmhead_argmax(x, w_shard, w_s_shard, shard_lo)
    T = x.shape[0]
    maxes = torch.empty(world, T, dtype=torch.float32, device=x.device)
    idxs = torch.empty(world, T, dtype=torch.int32, device=x.device)
    dist.all_gather_into_tensor(maxes, mx, group=group)
    dist.all_gather_into_tensor(idxs, idx, group=group)
    return ops.argmax_merge(maxes, idxs)
