"""`logits_processor` op: prepare(module) / forward(prepared, input_ids, hidden_states, lm_head, logits_metadata).

Same contract as the reference's qwen36_lmhead8/node.py (`prepare` :169, `forward` :153-173,
`_Node.logits` :136-151): the stock LogitsProcessor keeps its own control flow and only the
lm_head GEMM is replaced, through a stand-in head whose `quant_method.apply` is ours.  The private
copy of `lm_head.weight` is e4m3 with 128 x 128 block scales, made on first use and keyed by the
weight's storage (node.py:88-107 does the same for its int8 copy).  Beyond the reference: the greedy
token (argmax fused into the GEMM, vocabulary sharded over ranks when a process group is given) is
left on the returned object as `next_token_ids`.
"""
from __future__ import annotations

import torch

from bundles_b200 import ops, parallel
from bundles_b200 import prepare as prepare_q
from bundles_b200.evidence import note

_copies = {}   # (device index, data_ptr) -> (codes uint8 [V,H], scales fp32 [V/128, H/128], shard_lo)


class UnsupportedHead(RuntimeError):
    pass


def _private_copy(weight: torch.Tensor, group=None):
    key = (weight.device.index, weight.data_ptr(), None if group is None else id(group))
    got = _copies.get(key)
    if got is None:
        if torch.cuda.is_current_stream_capturing():
            # the reference builds its private copy outside capture only (node.py:127-128): a copy made while a graph
            # is being captured would live in the graph's memory pool
            raise UnsupportedHead("qwen36_lmhead8: the private fp8 copy of lm_head.weight must exist before stream "
                                  "capture; run one forward (or `prepared.warm(lm_head)`) first")
        V, H = weight.shape
        if H % 128 or H > 4096:
            raise UnsupportedHead(f"qwen36_lmhead8: hidden size {H} is not supported")
        lo, hi = 0, V
        if group is not None:
            import torch.distributed as dist
            lo, hi = parallel.vocab_shards(V, dist.get_world_size(group))[dist.get_rank(group)]
        rows = hi - lo
        pad = (-rows) % 128
        w = weight[lo:hi].float()
        if pad:
            w = torch.cat([w, torch.zeros(pad, H, device=w.device)])
        codes, scales = prepare_q.quant_fp8_blocks(w)
        got = (codes[:rows].contiguous(), scales.contiguous(), lo)
        _copies[key] = got
    return got


class _Node:
    def __init__(self, module, group=None):
        if getattr(module, "do_tensor_parallel_all_gather", False):
            raise UnsupportedHead("qwen36_lmhead8: tensor-parallel all-gather of logits is not supported (node.py:37-38)")
        self.module, self.group = module, group
        self.last_token_ids = None

    def warm(self, lm_head):
        """Build the private copy now (call once before the engine captures its graphs)."""
        _private_copy(lm_head.weight, self.group)

    def logits(self, lm_head, hidden_states):
        """fp32 logits [T, V] over the whole vocabulary (what the stock processor goes on with) and, as a side
        effect, the greedy token ids [T] in `last_token_ids`.  With a process group every rank holds one vocabulary
        shard: the (max, argmax) pairs are gathered and merged, and the shards' logits are gathered into [T, V]."""
        x = hidden_states.to(torch.bfloat16).contiguous()
        codes, scales, lo = _private_copy(lm_head.weight, self.group)
        note("lmhead_argmax" if self.group is None else "lmhead_argmax_sharded", x.shape[0])
        mx, idx, lg = ops.lmhead_argmax(x, codes, scales, lo, True)
        if self.group is None:
            self.last_token_ids = idx
            return lg
        import torch.distributed as dist
        world = dist.get_world_size(self.group)
        T, V = x.shape[0], lm_head.weight.shape[0]
        maxes = torch.empty(world, T, dtype=torch.float32, device=x.device)
        idxs = torch.empty(world, T, dtype=torch.int32, device=x.device)
        dist.all_gather_into_tensor(maxes, mx, group=self.group)
        dist.all_gather_into_tensor(idxs, idx, group=self.group)
        self.last_token_ids = ops.argmax_merge(maxes, idxs)
        shards = parallel.vocab_shards(V, world)
        wmax = max(hi - lo_ for lo_, hi in shards)
        mine = torch.zeros(T, wmax, dtype=torch.float32, device=x.device)      # shards differ by one scale block
        mine[:, :lg.shape[1]] = lg
        parts = torch.empty(world, T, wmax, dtype=torch.float32, device=x.device)
        dist.all_gather_into_tensor(parts, mine, group=self.group)
        return torch.cat([parts[r, :, :hi - lo_] for r, (lo_, hi) in enumerate(shards)], dim=1)

    def __call__(self, input_ids, hidden_states, lm_head, logits_metadata, *args, **kwargs):
        node = self

        class _Apply:
            def apply(self, layer, x, bias=None):
                out = node.logits(lm_head, x)
                return out if bias is None else out + bias

        class _StandInHead:
            weight = lm_head.weight
            quant_method = _Apply()

        out = type(self.module).forward(self.module, input_ids, hidden_states, _StandInHead(), logits_metadata, *args,
                                        **kwargs)
        try:
            out.next_token_ids = self.last_token_ids
        except AttributeError:
            pass
        return out


def prepare(module, group=None):
    return _Node(module, group)


def forward(prepared, *args, **kwargs):
    return prepared(*args, **kwargs)
