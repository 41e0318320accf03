"""The sparse-MoE block of one decoder layer: router -> routing lists -> expert MLPs -> combine.

Host-side mirror of the reference's `moe_row_batch` (i8x_decode.py:528-576) and of the `mlp`
override its layer node installs (layer.py:434-480): same inputs (hidden states, optional
positions whose zeros mark graph-padding rows), same output (bf16 [T, H]); the workspaces are
allocated once per (device, T) and reused, as the reference's `Workspace` is (i8x_decode.py:495-526).
"""
from __future__ import annotations

from collections import OrderedDict

import torch

from . import ops


class MoeBlockW8A8:
    """int8 W8A8 experts (per-output-channel weight scales, per-token activation scales)."""
    BLOCK_ROWS = 128          # largest N tile of the int8 GEMMs
    GRAPH_MAX_T = 256         # row counts up to this are replayed from a captured CUDA graph (decode / verify batches)
    CHUNK = 2048              # larger batches (prefill / extend) run eagerly in chunks of at most this many rows
    MAX_CACHED = 6            # buffer sets / graphs kept (least recently used beyond that are dropped)

    def __init__(self, wr, weights: ops.MoeW8A8Weights, gate_w, top_k, bias=None, e_lo=0, round_bf16=False,
                 use_graph=True):
        self.wr, self.w, self.gate_w, self.bias = wr, weights, gate_w, bias
        self.top_k, self.e_lo, self.round_bf16 = top_k, e_lo, round_bf16
        self.E_local = weights.w13.shape[0]
        self.I = weights.w2.shape[-1]
        self.H = weights.w13.shape[-1]
        self._ws = OrderedDict()
        self._graphs = OrderedDict()
        self._pipes = {}
        self.use_graph = use_graph
        self.status = ops.new_status(wr.device)
        self.launches_per_call = 8  # gate, top-k, lists, quant+permute, up, h-quant, down, combine

    def _buffers(self, T, device):
        b = self._ws.get(T)
        if b is not None:
            self._ws.move_to_end(T)
        if b is None:
            while len(self._ws) >= self.MAX_CACHED:      # variable-length batches must not grow memory without bound
                self._ws.popitem(last=False)
            K = self.top_k
            b = dict(lists=ops.RoutingLists(T, K, self.E_local, self.BLOCK_ROWS, device),
                     ws=self._workspace(T, K, device),
                     cache=torch.zeros(T * (K + 1), self.H, dtype=torch.bfloat16, device=device),
                     scratch=ops.router_scratch(T, self.H, self.wr.shape[0], device),
                     ids=torch.empty(T, K, dtype=torch.int32, device=device),
                     wts=torch.empty(T, K, dtype=torch.float32, device=device),
                     out=torch.empty(T, self.H, dtype=torch.bfloat16, device=device))
            self._ws[T] = b
        return b

    def forward(self, x: torch.Tensor, positions: torch.Tensor | None = None) -> torch.Tensor:
        """One pass of the block.  With `use_graph` the eight launches of a given (T, with/without
        positions) are captured once into a CUDA graph and replayed (the reference's ops run inside the
        engine's captured decode graph as well, layer.py:174-189); the input is copied into the graph's
        static buffer and the returned tensor is the graph's static output, overwritten by the next call."""
        T = x.shape[0]
        if T > self.CHUNK:          # prefill-sized batch: chunks through one reusable buffer set per chunk size
            outs = []
            for t0 in range(0, T, self.CHUNK):
                ps = None if positions is None else positions[t0:t0 + self.CHUNK].contiguous()
                outs.append(self._forward_eager(x[t0:t0 + self.CHUNK].contiguous(), ps).clone())
            return torch.cat(outs)
        if not self.use_graph or T > self.GRAPH_MAX_T or torch.cuda.is_current_stream_capturing():
            return self._forward_eager(x, positions)
        key = (T, positions is not None)
        g = self._graphs.get(key)
        if g is not None:
            self._graphs.move_to_end(key)
        if g is None:
            while len(self._graphs) >= self.MAX_CACHED:
                self._graphs.popitem(last=False)
            dev = self.wr.device
            xs = torch.empty(x.shape, dtype=x.dtype, device=dev)
            ps = None if positions is None else torch.empty(positions.shape, dtype=positions.dtype, device=dev)
            xs.copy_(x)
            if ps is not None:
                ps.copy_(positions)
            self._forward_eager(xs, ps)                      # warm-up: one-time attribute set-up, buffers
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self._forward_eager(xs, ps)
            g = (graph, xs, ps, out)
            self._graphs[key] = g
        graph, xs, ps, out = g
        xs.copy_(x, non_blocking=True)
        if ps is not None:
            ps.copy_(positions, non_blocking=True)
        graph.replay()
        return out

    def _forward_eager(self, x: torch.Tensor, positions: torch.Tensor | None = None) -> torch.Tensor:
        T = x.shape[0]
        b = self._buffers(T, x.device)
        _, ids, wts = ops.router(x, self.wr, self.top_k, self.bias, self.round_bf16, scratch=b["scratch"],
                                 want_logits=False, ids=b["ids"], wts=b["wts"])
        ops.build_lists(ids, wts, b["lists"], positions, e_lo=self.e_lo, with_shared=self.w.sh13 is not None)
        self._experts(x, b)
        return ops.moe_combine(b["cache"], x, self.gate_w if self.w.sh13 is not None else None, self.top_k, positions,
                               out=b["out"])

    __call__ = forward

    def forward_combine_norm(self, x, positions, residual, norm_w, eps):
        """One pass of the block whose combine also does the next layer's residual add and input norm (the reference's
        combine_norm, qk_route.cu:779-819): `residual` <- bf16(out + residual) in place; returns (out, normed), both
        fresh tensors.  Runs eagerly on the current stream (inside the engine's own graph capture, if any)."""
        T = x.shape[0]
        b = self._buffers(T, x.device)
        ops.router(x, self.wr, self.top_k, self.bias, self.round_bf16, scratch=b["scratch"], want_logits=False,
                   ids=b["ids"], wts=b["wts"])
        ops.build_lists(b["ids"], b["wts"], b["lists"], positions, e_lo=self.e_lo, with_shared=self.w.sh13 is not None)
        self._experts(x, b)
        return ops.moe_combine_norm(b["cache"], x, self.gate_w if self.w.sh13 is not None else None, self.top_k, residual,
                                    norm_w, eps, positions)

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """Host-to-host form for a serving loop: `x_host` (pinned bf16 [T, H]) is copied in, the block runs, and
        the result lands in `out_host` (pinned) asynchronously.  Consecutive calls are pipelined over two sets of
        device buffers: the copy-in of call i + 1 and the copy-out of call i - 1 run on their own streams
        beside the kernels of call i.  The result of a call is complete after `synchronize_host()` (or any
        later device synchronisation); `x_host` may be reused once the call after next has been issued."""
        T = x_host.shape[0]
        pipe = self._pipes.get(T)
        dev = self.wr.device
        main = torch.cuda.current_stream(dev)
        if pipe is None:
            pipe = dict(i=0, s_in=torch.cuda.Stream(dev), s_out=torch.cuda.Stream(dev), slots=[])
            for _ in range(2):
                xs = torch.empty(T, self.H, dtype=torch.bfloat16, device=dev)
                xs.copy_(x_host)
                self._forward_eager(xs, None)              # warm-up: one-time attribute set-up, buffers
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    out = self._forward_eager(xs, None).clone()   # each slot keeps its own result buffer
                pipe["slots"].append(dict(graph=graph, xs=xs, out=out, in_ready=torch.cuda.Event(),
                                          done=torch.cuda.Event(), out_free=torch.cuda.Event(), used=False))
            self._pipes[T] = pipe
        slot = pipe["slots"][pipe["i"] & 1]
        pipe["i"] += 1
        with torch.cuda.stream(pipe["s_in"]):
            if slot["used"]:
                pipe["s_in"].wait_event(slot["done"])      # the call two back has read this input buffer
            slot["xs"].copy_(x_host, non_blocking=True)
            slot["in_ready"].record()
        main.wait_event(slot["in_ready"])
        if slot["used"]:
            main.wait_event(slot["out_free"])              # its result has left the device
        slot["graph"].replay()
        slot["done"].record(main)
        with torch.cuda.stream(pipe["s_out"]):
            pipe["s_out"].wait_event(slot["done"])
            out_host.copy_(slot["out"], non_blocking=True)
            slot["out_free"].record()
        slot["used"] = True

    def join_host(self) -> None:
        """Make the current stream wait for every pending copy-out of `forward_host` (no host blocking)."""
        main = torch.cuda.current_stream(self.wr.device)
        for pipe in self._pipes.values():
            for slot in pipe["slots"]:
                if slot["used"]:
                    main.wait_event(slot["out_free"])

    def synchronize_host(self) -> None:
        """Block until every result handed to `forward_host` has landed in its host buffer."""
        for pipe in self._pipes.values():
            pipe["s_out"].synchronize()

    def _workspace(self, T, K, device):
        return ops.moe_w8a8_workspace(T, self.H, self.I, K, device)

    def _experts(self, x, b):
        ops.moe_w8a8(x, self.w, b["lists"], cache=b["cache"], ws=b["ws"], status=self.status)


class MoeBlockFp8(MoeBlockW8A8):
    """fp8 e4m3 experts with 128 x 128 weight block scales and per-(token, 128-channel) activation scales."""
    BLOCK_ROWS = 32           # the fp8 expert GEMMs take blocks of at most 32 rows (eight partial buffers in TMEM)

    def _workspace(self, T, K, device):
        return ops.moe_fp8_workspace(T, self.H, self.I, K, device)

    def _experts(self, x, b):
        ops.moe_fp8(x, self.w, b["lists"], cache=b["cache"], ws=b["ws"], status=self.status)
