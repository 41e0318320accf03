"""`model.layers.*` op: prepare(module) / forward(prepared, *args, **kwargs).

Same contract as the reference's qwen36_layer/layer.py (prepare :486-531, forward :762-764):
`prepare` makes a shallow replica of the stock decoder layer, reads the stock weights WITHOUT
modifying them (layer.py:16-17), builds private quantised copies and swaps the replica's sparse-MoE
block for the B200 path; `forward` calls the stock layer's own forward on the replica and returns
exactly what it returns (`(hidden_states, residual)`).  Unsupported configurations raise at
`prepare`, as the reference's do (layer.py:394-415); there is no fallback path.

Host objects read (the reference reads the same ones, layer.py:392-415):
  module.mlp.gate.weight [E,H], module.mlp.topk.topk_config.{top_k, renormalize, scoring_func,
  correction_bias}, module.mlp.experts.{w13_weight [E,2I,H], w2_weight [E,H,I]},
  module.mlp.shared_expert.{gate_up_proj.weight [2I,H], down_proj.weight [H,I]},
  module.mlp.shared_expert_gate.weight [1,H], module.mlp.tp_size.
"""
from __future__ import annotations

import copy

import torch

from bundles_b200 import moe_block, ops
from bundles_b200 import prepare as prepare_q

EXPERT_FORMAT = "w8a8"      # "w8a8": int8 per-output-channel; "fp8": e4m3 with 128 x 128 block scales
_prepared = {}              # id(module) -> replica, so that a second prepare reuses the private copy


class UnsupportedLayer(RuntimeError):
    pass


def _check_moe(mlp):
    cfg = mlp.topk.topk_config
    if getattr(mlp, "tp_size", 1) != 1:
        raise UnsupportedLayer("qwen36_layer: the MoE block must not be tensor-parallel (tp_size == 1)")
    if not getattr(cfg, "renormalize", True):
        raise UnsupportedLayer("qwen36_layer: top-k weights must be renormalised")
    if getattr(cfg, "scoring_func", "softmax") != "softmax":
        raise UnsupportedLayer("qwen36_layer: only softmax routing is supported")
    w13, w2 = mlp.experts.w13_weight, mlp.experts.w2_weight
    E, twoI, H = w13.shape
    if w2.shape != (E, H, twoI // 2) or mlp.gate.weight.shape != (E, H):
        raise UnsupportedLayer(f"qwen36_layer: unexpected expert shapes {tuple(w13.shape)} / {tuple(w2.shape)}")
    if H % 128 or (twoI // 2) % 128 or E % 64 or E > 1024:
        raise UnsupportedLayer(f"qwen36_layer: need H, I multiples of 128 and E a multiple of 64 (H={H} I={twoI // 2} E={E})")
    if cfg.top_k > 32 or cfg.top_k > E:
        raise UnsupportedLayer(f"qwen36_layer: top_k {cfg.top_k} is not supported")
    return E, twoI // 2, H, cfg.top_k


def _quantise(mlp, fmt):
    """Private quantised copy of the experts (the stock bf16 weights stay untouched)."""
    q = prepare_q.quant_int8_rows if fmt == "w8a8" else prepare_q.quant_fp8_blocks
    E = mlp.experts.w13_weight.shape[0]
    parts13, parts2 = [], []
    for e0 in range(0, E, 32):          # in slices: the fp32 staging copy stays small
        parts13.append(q(mlp.experts.w13_weight[e0:e0 + 32]))
        parts2.append(q(mlp.experts.w2_weight[e0:e0 + 32]))
    w13 = torch.cat([p[0] for p in parts13])
    s13 = torch.cat([p[1] for p in parts13])
    w2 = torch.cat([p[0] for p in parts2])
    s2 = torch.cat([p[1] for p in parts2])
    sh13 = shs13 = sh2 = shs2 = None
    if getattr(mlp, "shared_expert", None) is not None:
        sh13, shs13 = q(mlp.shared_expert.gate_up_proj.weight)
        sh2, shs2 = q(mlp.shared_expert.down_proj.weight)
    return ops.MoeW8A8Weights(w13.contiguous(), s13.contiguous(), w2.contiguous(), s2.contiguous(), sh13, shs13, sh2,
                              shs2)


class _MoeOverride(torch.nn.Module):
    """Drop-in for the stock sparse-MoE block's forward(hidden_states, forward_batch=None, ...)."""

    def __init__(self, mlp, fmt):
        super().__init__()
        E, I, H, K = _check_moe(mlp)
        if not mlp.gate.weight.is_cuda:
            raise UnsupportedLayer("qwen36_layer: weights must live on a CUDA device (there is no CPU path)")
        weights = _quantise(mlp, fmt)
        gate_w = None
        if getattr(mlp, "shared_expert_gate", None) is not None:
            gate_w = mlp.shared_expert_gate.weight.reshape(-1).to(torch.bfloat16).contiguous()
        bias = getattr(mlp.topk.topk_config, "correction_bias", None)
        wr = mlp.gate.weight.float().contiguous()          # the router runs on an fp32 copy of the gate weight
        if fmt == "w8a8":
            self.block = moe_block.MoeBlockW8A8(wr, weights, gate_w, K, bias=None if bias is None else bias.float())
        else:
            self.block = moe_block.MoeBlockFp8(wr, weights, gate_w, K, bias=None if bias is None else bias.float())
        self.hidden = H

    def forward(self, hidden_states, forward_batch=None, *args, **kwargs):
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, self.hidden)
        pos = getattr(forward_batch, "positions", None) if forward_batch is not None else None
        if pos is not None and pos.dtype != torch.int64:
            pos = pos.to(torch.int64)
        # rows whose position is 0 are graph padding and come back as zeros (layer.py:476-477)
        return self.block(x, pos).reshape(shape).clone()


def prepare(module):
    """Once per decoder layer (reference: layer.py:486-531).  Returns the callable the engine stores."""
    key = id(module)
    if key in _prepared:
        return _prepared[key]
    if not hasattr(module, "mlp") or not hasattr(module.mlp, "experts"):
        raise UnsupportedLayer("qwen36_layer: the layer has no sparse-MoE block (`mlp.experts`)")
    replica = copy.copy(module)                        # shallow: shares the stock weights, read-only
    replica._modules = dict(module._modules)
    replica._modules["mlp"] = _MoeOverride(module.mlp, EXPERT_FORMAT)

    def layer(*args, **kwargs):
        return type(module).forward(replica, *args, **kwargs)

    layer.replica = replica
    _prepared[key] = layer
    return layer


def forward(prepared, *args, **kwargs):
    return prepared(*args, **kwargs)
