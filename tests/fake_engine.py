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


# ---------------------------------------------------------------------------------------------------------
# The hybrid decoder layer (recurrent or attention mixer + sparse MoE) with the engine objects its glue reads
# ---------------------------------------------------------------------------------------------------------
class FakeMode:
    def __init__(self, kind):
        self.kind = kind

    def is_decode(self):
        return self.kind == "decode"

    def is_target_verify(self):
        return self.kind == "target_verify"

    def is_extend(self):
        return self.kind in ("extend", "target_verify")

    def is_idle(self):
        return self.kind == "idle"


class FakeGemmaNorm(torch.nn.Module):
    """x (+ residual in fp32, rounded to bf16) -> bf16(r * rsqrt(mean r^2 + eps) * (1 + w)); returns (y, r) with a residual."""

    def __init__(self, n, device, seed, eps=1e-6):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.weight = (torch.randn(n, generator=g) * 0.1).to(torch.bfloat16).to(device)
        self.variance_epsilon = eps

    def forward(self, x, residual=None):
        r = x if residual is None else (x.float() + residual.float()).to(torch.bfloat16)
        rf = r.float()
        y = (rf * torch.rsqrt(rf.pow(2).mean(-1, keepdim=True) + self.variance_epsilon) * (1.0 + self.weight.float()))
        return y.to(torch.bfloat16) if residual is None else (y.to(torch.bfloat16), r)


class FakeLinear(torch.nn.Module):
    def __init__(self, n, k, device, seed):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.weight = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(device)
        self.bias = None
        self.tp_size = 1
        self.calls = 0

    def forward(self, x):
        self.calls += 1
        return torch.nn.functional.linear(x, self.weight), None


class FakeCommunicator:
    def __init__(self, layer):
        self.layer = layer

    def prepare_attn(self, hidden_states, residual, forward_batch):
        if residual is None:
            return self.layer.input_layernorm(hidden_states), hidden_states
        return self.layer.input_layernorm(hidden_states, residual)

    def prepare_mlp(self, hidden_states, residual, forward_batch, cache=None):
        return self.layer.post_attention_layernorm(hidden_states, residual)


class FakeGdn(torch.nn.Module):
    def __init__(self, layer_id, device, cfg):
        super().__init__()
        self.layer_id = layer_id
        self.in_proj_qkvz = FakeLinear(12288, 2048, device, 100 + layer_id)
        self.in_proj_ba = FakeLinear(64, 2048, device, 200 + layer_id)
        self.out_proj = FakeLinear(2048, 4096, device, 300 + layer_id)
        self.attn = SimpleNamespace(layer_id=layer_id, conv_weights=cfg["conv_w"].to(device), A_log=cfg["a_log"].to(device),
                                    dt_bias=cfg["dt_bias"].to(device), bias=None, activation="silu", head_k_dim=128)
        self.norm = SimpleNamespace(weight=cfg["norm_w"].to(device), eps=1e-6, norm_before_gate=True, activation="silu",
                                    group_size=None, bias=None)
        self.counters = {"stock": 0}        # a dict: shared with the shallow replicas the glue makes

    @property
    def stock_calls(self):
        return self.counters["stock"]

    def forward(self, hidden_states, forward_batch):
        if forward_batch.forward_mode.is_target_verify():
            raise AssertionError("the stock recurrent block must not run for a target-verify batch")
        self.counters["stock"] += 1
        out, _ = self.out_proj(torch.zeros(hidden_states.shape[0], 4096, dtype=torch.bfloat16, device=hidden_states.device))
        return out


class FakeHybridLayer(torch.nn.Module):
    """forward(positions, hidden_states, forward_batch, residual) in the stock order: input norm (prepare_attn), mixer,
    post-attention norm (prepare_mlp), sparse MoE."""

    def __init__(self, layer_id, moe, device, kind="gdn", gdn_cfg=None):
        super().__init__()
        self.layer_id = layer_id
        self.mlp = moe
        self.input_layernorm = FakeGemmaNorm(2048, device, 400 + layer_id)
        self.post_attention_layernorm = FakeGemmaNorm(2048, device, 500 + layer_id)
        self.layer_communicator = FakeCommunicator(self)
        if kind == "gdn":
            self.linear_attn = FakeGdn(layer_id, device, gdn_cfg)
        else:
            self.qkv_proj = FakeLinear(9216, 2048, device, 600 + layer_id)
            self.o_proj = FakeLinear(2048, 4096, device, 700 + layer_id)
            self.q_norm = FakeGemmaNorm(256, device, 800 + layer_id)
            self.k_norm = FakeGemmaNorm(256, device, 900 + layer_id)
            self.num_heads, self.num_kv_heads, self.head_dim, self.attn_output_gate = 16, 2, 256, True
            half = 32
            inv = torch.pow(torch.tensor(1e7, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / 64)
            ang = torch.arange(1024, dtype=torch.float64)[:, None] * inv[None, :]
            self.rotary_emb = SimpleNamespace(rotary_dim=64, cos_sin_cache=torch.cat([ang.cos(), ang.sin()], 1).float().to(device))
            self.attn = SimpleNamespace(layer_id=layer_id, scaling=256 ** -0.5, k_scale=None, v_scale=None)
        self.counters = {"stock_attention": 0}      # a dict: shared with the shallow replica the glue makes

    @property
    def stock_attention_calls(self):
        return self.counters["stock_attention"]

    def self_attention(self, positions, hidden_states, forward_batch):
        if forward_batch.forward_mode.is_target_verify():
            raise AssertionError("the stock attention must not run for a target-verify batch")
        self.counters["stock_attention"] += 1
        out, _ = self.o_proj(torch.zeros(hidden_states.shape[0], 4096, dtype=torch.bfloat16, device=hidden_states.device))
        return out

    def forward(self, positions, hidden_states, forward_batch, residual):
        hidden_states, residual = self.layer_communicator.prepare_attn(hidden_states, residual, forward_batch)
        if hasattr(self, "linear_attn"):
            hidden_states = self.linear_attn(hidden_states, forward_batch)
        else:
            hidden_states = self.self_attention(positions, hidden_states, forward_batch)
        hidden_states, residual = self.layer_communicator.prepare_mlp(hidden_states, residual, forward_batch)
        hidden_states = self.mlp(hidden_states, forward_batch)
        return hidden_states, residual


def fake_gdn_backend(cfg, device):
    """The linear-attention backend and pool objects of gdn_fused.py:42-57 over the tensors of `synth.gdn_replay`."""
    d = {k: v.to(device) for k, v in cfg.items()}
    params = SimpleNamespace(conv=[d["conv_state"]], intermediate_conv_window=[d["window"].view(d["window"].shape[0], -1)],
                             temporal=d["checkpoint"], replayssm_d=d["d_ring"], replayssm_rawv=d["dlo_ring"],
                             replayssm_k=d["k_ring"], replayssm_rawk=d["klo_ring"], replayssm_g=d["g_ring"])
    pool = SimpleNamespace(replayssm_spec_write_pos=d["write_pos"], replayssm_cache_base=d["cache_base"])
    lin = SimpleNamespace(forward_metadata=SimpleNamespace(mamba_cache_indices=d["state_idx"]),
                          req_to_token_pool=SimpleNamespace(mamba2_layer_cache=lambda layer_id: params, mamba_pool=pool),
                          verify_intermediate_state_indices=d["win_idx"])
    return SimpleNamespace(linear_attn_backend=lin), d


def fake_attn_backend(av, device):
    """The full-attention backend over the paged e4m3 KV cache of `synth.attn_verify` (128-token pages)."""
    d = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in av.items()}
    pool = SimpleNamespace(get_kv_buffer=lambda layer_id: (d["kcache"].view(torch.float8_e4m3fn), d["vcache"].view(torch.float8_e4m3fn)))
    full = SimpleNamespace(page_size=128, topk=1, token_to_kv_pool=pool,
                           forward_metadata=SimpleNamespace(page_table=d["page_table"], cache_seqlens_int32=d["seqlens"]))
    return SimpleNamespace(full_attn_backend=full), d
