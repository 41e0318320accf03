"""One decode / speculative-verify step through a whole stack of layers, built from the operators of this package.

The host-side loop a serving engine runs per step for the Qwen3.6-35B-A3B layout of the reference bundle
(`layer.py:486-531`: every layer = token mixer + sparse MoE; full attention every fourth layer, Gated DeltaNet
otherwise; `node.py:136-151`: LM head at the end), at the target formats: fp8 block-scaled projections and
experts, e4m3 KV pages, explicit fp32 GDN state, greedy token from the fused LM-head argmax.  Weights are
random-initialised on the device from a seed (there are no checkpoints here); every layer owns its own weights,
state and KV pages, so a step streams what a real model would stream.

Per layer (T = 4 drafts x B sequences rows, T <= 64):
    GDN layer:        in_proj (dense fp8) -> gdn_verify -> out_proj (dense fp8); with `gdn_layout="ring"` the state is
                      the engine's read-only checkpoint + 16-entry (d, k, g) ring and the step appends to the ring
    attention layer:  attn_front (projection + q/k norm + RoPE, e4m3 q/k/v) -> attn_verify -> o_proj (dense fp8)
    then              residual add + RMSNorm -> router -> lists -> fp8 experts -> combine fused with the next
                      layer's residual add + input RMSNorm
and after the last layer the vocabulary argmax.
"""
from __future__ import annotations

import math

import torch

from . import ops
from .synth import quant_fp8_blocks

H, I, E, K = 2048, 512, 512, 10
GDN_PROJ = 8192 + 4096 + 32 + 32   # q | k | v, z, b, a   (dense8.py:64-68)


def _fp8(shape, gen, device, std=0.02, chunk=64):
    """Random weight [..., rows, cols] -> (e4m3 codes, 128 x 128 block scales), generated in chunks on the device."""
    if len(shape) == 2:
        rows, cols = shape
        rp = (rows + 127) // 128 * 128   # a ragged last block row is quantised as if padded with zeros
        w = torch.zeros(rp, cols, device=device)
        w[:rows] = torch.randn(rows, cols, generator=gen, device=device) * std
        q, s = quant_fp8_blocks(w)
        return q[:rows].contiguous(), s
    n = shape[0]
    q = torch.empty(shape, dtype=torch.uint8, device=device)
    s = torch.empty(n, (shape[1] + 127) // 128, (shape[2] + 127) // 128, dtype=torch.float32, device=device)
    for e0 in range(0, n, chunk):
        m = min(chunk, n - e0)
        q[e0:e0 + m], s[e0:e0 + m] = quant_fp8_blocks(torch.randn(m, shape[1], shape[2], generator=gen, device=device) * std)
    return q, s


class DecodeStep:
    """`layers` layers (layer i is full attention iff i % 4 == 3), B sequences with `ctx` tokens of context each."""

    def __init__(self, layers=48, B=8, ctx=8192, vocab=151936, experts=E, seed=1005, device="cuda", gdn_layout="explicit",
                 ring_fill=0):
        if 4 * B > 64:
            raise ValueError("the decode-width projections take at most 64 rows: B <= 16")
        if gdn_layout not in ("explicit", "ring"):
            raise ValueError("gdn_layout is 'explicit' or 'ring'")
        self.gdn_layout = gdn_layout
        dev = torch.device(device)
        g = torch.Generator(device=dev).manual_seed(seed)
        g_ring = torch.Generator(device=dev).manual_seed(seed + 1)   # ring contents: the weights do not depend on the layout
        bf = torch.bfloat16
        self.B, self.T, self.ctx, self.n_layers, self.E = B, 4 * B, ctx, layers, experts
        self.status = ops.new_status(dev)
        rn = lambda *s, std=1.0: (torch.randn(*s, generator=g, device=dev) * std)
        self.layers = []
        per = (ctx + 127) // 128
        for i in range(layers):
            L = dict(attn=(i % 4 == 3))
            if L["attn"]:
                L["qkv_w"], L["qkv_s"] = _fp8((9216, H), g, dev)
                L["q_norm"], L["k_norm"] = rn(256, std=0.1).to(bf), rn(256, std=0.1).to(bf)
                L["o_w"], L["o_s"] = _fp8((H, 4096), g, dev)
                P = B * per + 1
                L["kcache"] = torch.randn(P, 2, 128, 256, generator=g, device=dev).to(torch.float8_e4m3fn).view(torch.uint8)
                L["vcache"] = torch.randn(P, 2, 256, 128, generator=g, device=dev).to(torch.float8_e4m3fn).view(torch.uint8)
                L["page_table"] = torch.randperm(P, generator=g, device=dev)[:B * per].to(torch.int32).reshape(B, per).contiguous()
            else:
                L["in_w"], L["in_s"] = _fp8((GDN_PROJ, H), g, dev)
                L["out_w"], L["out_s"] = _fp8((H, 4096), g, dev)
                L["conv_state"] = rn(B, 8192, 3).to(bf)
                L["conv_w"] = rn(8192, 4, std=0.5).to(bf)
                L["a_log"] = torch.rand(32, generator=g, device=dev) * math.log(16.0)
                L["dt_bias"] = rn(32)
                L["state"] = rn(B, 32, 128, 128, std=0.1)
                L["gdn_norm"] = rn(128, std=0.1).to(bf)
                if gdn_layout == "ring":   # pools of B slots, request b in slot b; `ring_fill` committed entries
                    L["window"] = torch.zeros(B, 8192, 6, dtype=bf, device=dev)
                    L["d_ring"] = (torch.randn(B, 32, 16, 128, generator=g_ring, device=dev) * 0.3).to(bf)
                    L["dlo_ring"] = torch.zeros(B, 32, 16, 128, dtype=bf, device=dev)
                    L["k_ring"] = torch.nn.functional.normalize(torch.randn(B, 16, 16, 128, generator=g_ring, device=dev),
                                                                dim=-1).to(bf)
                    L["klo_ring"] = torch.zeros(B, 16, 16, 128, dtype=bf, device=dev)
                    L["g_ring"] = -torch.rand(B, 32, 16, generator=g_ring, device=dev) * 0.5
            L["post_norm"] = rn(H, std=0.1).to(bf)     # norm between the mixer and the MoE
            L["next_norm"] = rn(H, std=0.1).to(bf)     # input norm of the next layer (final norm after the last)
            L["wr"] = rn(experts, H, std=0.02)
            L["gate_w"] = rn(H, std=0.02).to(bf)
            w13, s13 = _fp8((experts, 2 * I, H), g, dev)
            w2, s2 = _fp8((experts, H, I), g, dev)
            sh13, shs13 = _fp8((2 * I, H), g, dev)
            sh2, shs2 = _fp8((H, I), g, dev)
            L["w"] = ops.MoeW8A8Weights(w13, s13, w2, s2, sh13, shs13, sh2, shs2)
            self.layers.append(L)
        vb = (vocab + 127) // 128 * 128
        lm = torch.zeros(vb, H, device=dev)
        lm[:vocab] = torch.randn(vocab, H, generator=g, device=dev) * 0.02
        wq, self.lm_s = quant_fp8_blocks(lm)
        self.lm_w = wq[:vocab].contiguous()
        del lm, wq
        self.first_norm = rn(H, std=0.1).to(bf)
        half = 32
        inv = torch.pow(torch.tensor(1e7, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / 64)
        ang = torch.arange(ctx + 8, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos_sin = torch.cat([ang.cos(), ang.sin()], 1).float().to(dev)
        self.seqlens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        self.positions = (torch.arange(B, device=dev)[:, None] * 0 + torch.arange(ctx - 4, ctx, device=dev)[None, :]).reshape(-1).to(torch.int64).contiguous()
        self.accepted = torch.randint(0, 5, (B,), generator=g, device=dev, dtype=torch.int32)
        self.slots = torch.arange(B, dtype=torch.int32, device=dev)
        self.write_pos = torch.full((B,), int(ring_fill), dtype=torch.int32, device=dev)
        self.cache_base = torch.zeros(B, dtype=torch.int32, device=dev)
        # buffers reused by every layer
        T = self.T
        self.lists = ops.RoutingLists(T, K, experts, 64, dev)
        self.moe_ws = ops.moe_fp8_workspace(T, H, I, K, dev)
        self.cache = torch.zeros(T * (K + 1), H, dtype=bf, device=dev)
        self.scratch = ops.router_scratch(T, H, experts, dev)
        self.ids = torch.empty(T, K, dtype=torch.int32, device=dev)
        self.wts = torch.empty(T, K, dtype=torch.float32, device=dev)
        self.gdn_ws = ops.gdn_workspace(B, dev)
        self.launches = 0

    def step(self, x: torch.Tensor) -> torch.Tensor:
        """x bf16 [T, 2048] (embedded draft tokens) -> greedy next-token ids int32 [T]."""
        st = self.status
        residual = torch.zeros_like(x)
        h = ops.add_rmsnorm(x, residual, self.first_norm)          # residual <- x, h = norm(x)
        n = 1
        for L in self.layers:
            if L["attn"]:
                q, gate, k, v = ops.attn_front(h, L["qkv_w"], L["qkv_s"], L["q_norm"], L["k_norm"], self.positions,
                                               self.cos_sin, 1e-6, True, status=st)
                core = ops.attn_verify(q, gate, k, v, L["kcache"], L["vcache"], L["page_table"], self.seqlens, status=st)
                proj = ops.dense_fp8(core, L["o_w"], L["o_s"], status=st)
                n += 2 + 3 + 2
            else:
                p = ops.dense_fp8(h, L["in_w"], L["in_s"], status=st)
                mixed, z = p[:, :8192].contiguous(), p[:, 8192:12288].contiguous()
                b, a = p[:, 12288:12320].contiguous(), p[:, 12320:12352].contiguous()
                if self.gdn_layout == "ring":
                    core = ops.gdn_verify_replay(mixed, z, a, b, L["conv_state"], L["conv_w"], L["window"], L["a_log"],
                                                 L["dt_bias"], L["state"], L["d_ring"], L["dlo_ring"], L["k_ring"],
                                                 L["klo_ring"], L["g_ring"], self.slots, self.slots, self.slots,
                                                 self.write_pos, self.cache_base, L["gdn_norm"], 1e-6, status=st,
                                                 ws=self.gdn_ws)
                else:
                    core = ops.gdn_verify(mixed, z, a, b, L["conv_state"], L["conv_w"], L["a_log"], L["dt_bias"], L["state"],
                                          self.accepted, L["gdn_norm"], 1e-6, status=st, ws=self.gdn_ws)
                proj = ops.dense_fp8(core, L["out_w"], L["out_s"], status=st)
                n += 2 + 2 + 2
            h2 = ops.add_rmsnorm(proj, residual, L["post_norm"])
            ops.router(h2, L["wr"], K, None, scratch=self.scratch, want_logits=False, ids=self.ids, wts=self.wts)
            ops.build_lists(self.ids, self.wts, self.lists)
            ops.moe_fp8(h2, L["w"], self.lists, cache=self.cache, ws=self.moe_ws, status=st)
            _, h = ops.moe_combine_norm(self.cache, h2, L["gate_w"], K, residual, L["next_norm"])
            n += 1 + 2 + 1 + 4 + 1
        _, idx, _ = ops.lmhead_argmax(h, self.lm_w, self.lm_s, 0, status=st)
        self.launches = n + 3
        return idx
