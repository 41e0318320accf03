"""Seeded synthetic inputs and random-init weights of the benchmark configurations.

No dataset or checkpoint is involved: weights are N(0, 0.02) quantised to the named formats,
activations are bf16 N(0, 1).  Everything is generated with a CPU `torch.Generator` so that the
parity tests can hand identical bytes to the CUDA path and to the checker.  Quantisation here is
the one-time `prepare` step of the layer node (the reference quantises its private expert copy at
prepare time as well: i8x_reloc.py:193-241, i8x_kernels.py:112-148).
"""
from __future__ import annotations

import math

import torch

from .prepare import quant_fp8_blocks, quant_int8_rows  # noqa: F401  (the prepare-time quantisers)

SEEDS = {"moe_fp8": 1001, "moe_w8a8": 1002, "gdn": 1003, "attn": 1004, "step": 1005}


def _gen(seed, device="cpu"):
    return torch.Generator(device=device).manual_seed(int(seed))


def _randn(*shape, g):
    return torch.randn(*shape, generator=g, device=g.device)


def zipf_bias(E: int, s: float, gen) -> torch.Tensor:
    """bias_e = log(rank_e^-s / Z) over a seeded permutation of the experts (skewed expert load)."""
    perm = torch.randperm(E, generator=gen)
    p = torch.arange(1, E + 1, dtype=torch.float64).pow(-s)
    p = p / p.sum()
    bias = torch.empty(E, dtype=torch.float64)
    bias[perm] = p.log()
    return bias.float()


def moe_common(seed, T, H, E, device="cpu"):
    g = _gen(seed, device)
    x = _randn(T, H, g=g).to(torch.bfloat16)
    wr = _randn(E, H, g=g) * 0.02
    gate_w = (_randn(H, g=g) * 0.02).to(torch.bfloat16)
    return g, x, wr, gate_w


def moe_w8a8(seed=SEEDS["moe_w8a8"], T=256, H=2048, I=512, E=512, zipf_s=1.1, device="cpu"):
    """Config: int8 W8A8 routed MoE at decode (per-output-channel weights, per-token activations),
    Zipf-skewed router bias.  `device` selects where the random stream is drawn (the CPU stream is
    the one the parity tests use; a CUDA stream gives different, equally distributed values)."""
    g, x, wr, gate_w = moe_common(seed, T, H, E, device)
    bias = zipf_bias(E, zipf_s, _gen(seed + 1)).to(device) if zipf_s else None
    w13q = torch.empty(E, 2 * I, H, dtype=torch.int8, device=device)
    s13 = torch.empty(E, 2 * I, device=device)
    w2q = torch.empty(E, H, I, dtype=torch.int8, device=device)
    s2 = torch.empty(E, H, device=device)
    for e0 in range(0, E, 32):
        n = min(32, E - e0)
        w13q[e0:e0 + n], s13[e0:e0 + n] = quant_int8_rows(_randn(n, 2 * I, H, g=g) * 0.02)
        w2q[e0:e0 + n], s2[e0:e0 + n] = quant_int8_rows(_randn(n, H, I, g=g) * 0.02)
    sh13q, shs13 = quant_int8_rows(_randn(2 * I, H, g=g) * 0.02)
    sh2q, shs2 = quant_int8_rows(_randn(H, I, g=g) * 0.02)
    return dict(x=x, wr=wr, bias=bias, gate_w=gate_w, w13=w13q, s13=s13, w2=w2q, s2=s2, sh13=sh13q, shs13=shs13,
                sh2=sh2q, shs2=shs2)


def moe_fp8(seed=SEEDS["moe_fp8"], T=16, H=2048, I=512, E=512):
    """Config: single fp8 MoE block, 128 x 128 block scales."""
    g, x, wr, gate_w = moe_common(seed, T, H, E)
    w13q = torch.empty(E, 2 * I, H, dtype=torch.uint8)
    s13 = torch.empty(E, 2 * I // 128, H // 128)
    w2q = torch.empty(E, H, I, dtype=torch.uint8)
    s2 = torch.empty(E, H // 128, I // 128)
    for e0 in range(0, E, 32):
        n = min(32, E - e0)
        w13q[e0:e0 + n], s13[e0:e0 + n] = quant_fp8_blocks(torch.randn(n, 2 * I, H, generator=g) * 0.02)
        w2q[e0:e0 + n], s2[e0:e0 + n] = quant_fp8_blocks(torch.randn(n, H, I, generator=g) * 0.02)
    sh13q, shs13 = quant_fp8_blocks(torch.randn(2 * I, H, generator=g) * 0.02)
    sh2q, shs2 = quant_fp8_blocks(torch.randn(H, I, generator=g) * 0.02)
    return dict(x=x, wr=wr, bias=None, gate_w=gate_w, w13=w13q, s13=s13, w2=w2q, s2=s2, sh13=sh13q, shs13=shs13,
                sh2=sh2q, shs2=shs2)


def gdn(seed=SEEDS["gdn"], B=32):
    """Config: Gated DeltaNet speculative verify, 4 draft tokens, 16 q/k heads, 32 v heads, d = 128."""
    g = _gen(seed)
    bf = torch.bfloat16
    return dict(
        mixed=torch.randn(B * 4, 8192, generator=g).to(bf),
        z=torch.randn(B * 4, 4096, generator=g).to(bf),
        a=torch.randn(B * 4, 32, generator=g).to(bf),
        b=torch.randn(B * 4, 32, generator=g).to(bf),
        conv_state=torch.randn(B, 8192, 3, generator=g).to(bf),
        conv_w=(torch.randn(8192, 4, generator=g) * 0.5).to(bf),
        a_log=torch.rand(32, generator=g) * math.log(16.0),
        dt_bias=torch.randn(32, generator=g),
        state=torch.randn(B, 32, 128, 128, generator=g) * 0.1,
        accepted=torch.randint(0, 5, (B,), generator=g, dtype=torch.int32),
        norm_w=(1.0 + torch.randn(128, generator=g) * 0.1).to(bf),
    )


def gdn_replay(seed=SEEDS["gdn"] + 1, B=32, extra_slots=3):
    """Config: the same verify step on the checkpoint + 16-entry (d, k, g) ring layout: `B + extra_slots`
    pool slots in shuffled order, write positions 0..16 (16: the ring is full, nothing is appended), random
    ring bases, gates of the committed entries drawn like the step's own (negative)."""
    g = _gen(seed)
    bf = torch.bfloat16
    c = gdn(seed, B)
    n = B + extra_slots
    out = {k: c[k] for k in ("mixed", "z", "a", "b", "conv_w", "a_log", "dt_bias", "norm_w")}
    out.update(
        conv_state=torch.randn(n, 8192, 3, generator=g).to(bf),
        window=torch.zeros(n, 8192, 6, dtype=bf),
        checkpoint=torch.randn(n, 32, 128, 128, generator=g) * 0.1,
        d_ring=(torch.randn(n, 32, 16, 128, generator=g) * 0.3).to(bf),
        dlo_ring=torch.zeros(n, 32, 16, 128, dtype=bf),
        k_ring=torch.nn.functional.normalize(torch.randn(n, 16, 16, 128, generator=g), dim=-1).to(bf),
        klo_ring=torch.zeros(n, 16, 16, 128, dtype=bf),
        g_ring=-torch.rand(n, 32, 16, generator=g) * 0.5,
        state_idx=torch.randperm(n, generator=g)[:B].to(torch.int32),
        ring_idx=torch.randperm(n, generator=g)[:B].to(torch.int32),
        win_idx=torch.randperm(n, generator=g)[:B].to(torch.int32),
        write_pos=torch.randint(0, 17, (n,), generator=g, dtype=torch.int32),
        cache_base=torch.randint(0, 16, (n,), generator=g, dtype=torch.int32),
    )
    return out


def attn(seed=SEEDS["attn"], T=4096, H=2048):
    """Config: fused gated-attention projections; W [9216, 2048] fp8 block-scaled."""
    g = _gen(seed)
    bf = torch.bfloat16
    wq, ws = quant_fp8_blocks(torch.randn(9216, H, generator=g) * 0.02)
    return dict(x=torch.randn(T, H, generator=g).to(bf), w=wq, w_s=ws,
                q_norm_w=(torch.randn(256, generator=g) * 0.1).to(bf),
                k_norm_w=(torch.randn(256, generator=g) * 0.1).to(bf),
                positions=torch.arange(T, dtype=torch.int64))


def lmhead(seed=SEEDS["step"], T=64, V=151936, H=2048):
    """Config: fp8 LM head [V, 2048] with 128 x 128 block scales (V padded up to a block multiple
    inside the scale tensor only)."""
    g = _gen(seed + 7)
    vb = (V + 127) // 128 * 128
    w = torch.zeros(vb, H)
    w[:V] = torch.randn(V, H, generator=g) * 0.02
    wq, ws = quant_fp8_blocks(w)
    return dict(x=torch.randn(T, H, generator=g).to(torch.bfloat16), w=wq[:V].contiguous(), w_s=ws)


def attn_verify(seed=SEEDS["step"], B=64, ctx=8192, ragged=False, device="cpu"):
    """Config: attention verify over a paged e4m3 KV cache (128-token pages; K [P,2,128,256], V [P,2,256,128]).
    Every request holds `ctx` tokens including its 4 drafts (`ragged`: lengths drawn from [ctx/2, ctx]); cache,
    q, k_new, v_new are e4m3 of N(0,1), gate bf16 N(0,1); pages are handed out in a seeded random order, with a
    few spare pages that no request owns."""
    g = torch.Generator(device=device).manual_seed(seed)
    if ragged:
        seqlens = torch.randint(max(4, ctx // 2), ctx + 1, (B,), generator=g, device=device, dtype=torch.int32)
    else:
        seqlens = torch.full((B,), ctx, dtype=torch.int32, device=device)
    per = (ctx + 127) // 128
    P = B * per + 3
    perm = torch.randperm(P, generator=g, device=device).to(torch.int32)
    page_table = perm[:B * per].reshape(B, per).contiguous()

    def e4(*shape):
        return torch.randn(*shape, generator=g, device=device).to(torch.float8_e4m3fn).view(torch.uint8)

    return dict(q=e4(4 * B, 16, 256), gate=torch.randn(4 * B, 16, 256, generator=g, device=device).to(torch.bfloat16),
                k_new=e4(4 * B, 2, 256), v_new=e4(4 * B, 2, 256), kcache=e4(P, 2, 128, 256), vcache=e4(P, 2, 256, 128),
                page_table=page_table, seqlens=seqlens)
