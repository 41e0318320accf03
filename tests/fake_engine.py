"""Stand-ins for the serving engine's objects that the bundle's glue reads (SGLang is not installed):
a decoder layer with a Qwen-style sparse-MoE block, and a logits processor."""
from types import SimpleNamespace

import torch


class FakeMoe(torch.nn.Module):
    def __init__(self, E, H, I, K, device, seed=0, shared=True, tp_size=1, scoring="softmax", renorm=True):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        bf = torch.bfloat16
        mk = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(bf).to(device)  # noqa: E731
        self.gate = SimpleNamespace(weight=mk(E, H))
        self.topk = SimpleNamespace(topk_config=SimpleNamespace(top_k=K, renormalize=renorm, scoring_func=scoring,
                                                                correction_bias=None))
        self.experts = SimpleNamespace(w13_weight=mk(E, 2 * I, H), w2_weight=mk(E, H, I))
        if shared:
            self.shared_expert = SimpleNamespace(gate_up_proj=SimpleNamespace(weight=mk(2 * I, H)),
                                                 down_proj=SimpleNamespace(weight=mk(H, I)))
            self.shared_expert_gate = SimpleNamespace(weight=mk(1, H))
        else:
            self.shared_expert = None
            self.shared_expert_gate = None
        self.tp_size = tp_size

    def forward(self, hidden_states, forward_batch=None):
        raise AssertionError("the stock MoE forward must not run once the layer is prepared")


class FakeDecoderLayer(torch.nn.Module):
    """forward(positions, hidden_states, forward_batch, residual) -> (hidden_states, residual), like the
    stock layer: residual add, then the MoE block (attention is left out of the stand-in)."""

    def __init__(self, moe, layer_id=0):
        super().__init__()
        self.mlp = moe
        self.layer_id = layer_id

    def forward(self, positions, hidden_states, forward_batch, residual):
        residual = hidden_states if residual is None else (hidden_states + residual)
        return self.mlp(residual, forward_batch), residual


class FakeLogitsProcessor(torch.nn.Module):
    def __init__(self, vocab):
        super().__init__()
        self.vocab_size = vocab
        self.do_tensor_parallel_all_gather = False

    def forward(self, input_ids, hidden_states, lm_head, logits_metadata):
        logits = lm_head.quant_method.apply(lm_head, hidden_states)
        return SimpleNamespace(next_token_logits=logits)
