"""The C twin of the oracle (CPU baseline) agrees with the numpy oracle."""
import numpy as np
import torch

from bundles_b200 import synth
from oracle import clib
from oracle import moe as omoe
from oracle import numerics as num
from oracle import router as orouter


def test_c_router_is_bit_exact_with_numpy():
    g = torch.Generator().manual_seed(21)
    x = torch.randn(24, 2048, generator=g).to(torch.bfloat16)
    wr = (torch.randn(512, 2048, generator=g) * 0.02).numpy()
    bias = synth.zipf_bias(512, 1.1, g).numpy()
    xb = x.view(torch.int16).numpy().view(np.uint16)
    lc = clib.gate_logits(xb, wr, bias)
    ln = orouter.gate_logits(x.float().numpy(), wr, bias)
    assert np.array_equal(lc.view(np.uint32), ln.view(np.uint32))
    ic, wc = clib.topk(lc, 10)
    i_n, wn = orouter.topk_softmax(ln, 10)
    assert np.array_equal(ic, i_n)
    np.testing.assert_allclose(wc, wn, rtol=2e-6)


def test_c_moe_block_matches_numpy():
    cfg = synth.moe_w8a8(seed=31, T=12, E=16, zipf_s=1.1)
    K = 4
    x = cfg["x"].float().numpy()
    _, ids, wts = orouter.route(x, cfg["wr"].numpy(), K, cfg["bias"].numpy())
    n = {k: v.numpy() for k, v in cfg.items() if isinstance(v, torch.Tensor) and v.dtype != torch.bfloat16}
    ref = omoe.moe_int8(x, ids, wts, n["w13"], n["s13"], n["w2"], n["s2"], n["sh13"], n["shs13"], n["sh2"], n["shs2"],
                        cfg["gate_w"].float().numpy())
    xb = cfg["x"].view(torch.int16).numpy().view(np.uint16)
    gb = cfg["gate_w"].view(torch.int16).numpy().view(np.uint16)
    out, _ = clib.moe_w8a8(xb, ids, wts, n["w13"], n["s13"], n["w2"], n["s2"], n["sh13"], n["shs13"], n["sh2"],
                           n["shs2"], gb)
    d = np.abs(out.astype(np.int32) - num.bf16_bits(ref).astype(np.int32))
    assert d.max() <= 1 and np.mean(d != 0) < 5e-3      # exp() of libm vs numpy: rare one-ulp flips


def test_c_e4m3_codec_and_group_quantiser_equal_numpy():
    g = np.random.default_rng(5)
    x = np.concatenate([g.standard_normal(4096).astype(np.float32) * s for s in (1e-4, 0.02, 1.0, 100.0, 600.0)])
    x = np.concatenate([x, np.array([0.0, -0.0, 448.0, -448.0, 1e9, 2 ** -9, 2 ** -10, 3 * 2 ** -10, np.nan], np.float32)])
    tab = num.e4m3_decode(np.arange(256, dtype=np.uint8))
    mid = (tab[:126] + tab[1:127]) / 2                       # exact ties between neighbouring codes
    x = np.concatenate([x, mid, -mid]).astype(np.float32)
    assert np.array_equal(clib.e4m3_encode(x), num.e4m3_encode(x))
    a = (g.standard_normal((7, 512)) * 3).astype(np.float32)
    a[2] = 0.0
    qc, sc = clib.quant_fp8_groups(a)
    qn, sn = num.quant_fp8_groups(a)
    assert np.array_equal(qc, qn) and np.array_equal(sc.view(np.uint32), sn.view(np.uint32))


def test_c_block_gemm_matches_numpy():
    g = np.random.default_rng(6)
    a = g.standard_normal((5, 512)).astype(np.float32)
    w = (g.standard_normal((200, 512)) * 0.02).astype(np.float32)
    aq, a_s = num.quant_fp8_groups(a)
    wp = np.zeros((256, 512), np.float32)
    wp[:200] = w
    wq, w_s = num.quant_fp8_blocks(wp)
    ref = omoe.gemm_fp8_blocks(aq, a_s, wq[:200], w_s)
    got = clib.gemm_fp8_blocks(aq, a_s, wq[:200], w_s)
    np.testing.assert_allclose(got, ref, rtol=1e-6, atol=1e-7)


def test_c_fp8_moe_block_matches_numpy():
    cfg = synth.moe_fp8(seed=33, T=12, E=16)
    K = 4
    x = cfg["x"].float().numpy()
    _, ids, wts = orouter.route(x, cfg["wr"].numpy(), K)
    n = {k: v.numpy() for k, v in cfg.items() if isinstance(v, torch.Tensor) and v.dtype != torch.bfloat16}
    ref = omoe.moe_fp8(x, ids, wts, n["w13"], n["s13"], n["w2"], n["s2"], n["sh13"], n["shs13"], n["sh2"], n["shs2"],
                       cfg["gate_w"].float().numpy())
    xb = cfg["x"].view(torch.int16).numpy().view(np.uint16)
    gb = cfg["gate_w"].view(torch.int16).numpy().view(np.uint16)
    out, _ = clib.moe_fp8(xb, ids, wts, n["w13"], n["s13"], n["w2"], n["s2"], n["sh13"], n["shs13"], n["sh2"], n["shs2"],
                          gb)
    d = np.abs(out.astype(np.int32) - num.bf16_bits(ref).astype(np.int32))
    assert d.max() <= 1 and np.mean(d != 0) < 5e-3      # exp() of libm vs numpy: rare one-ulp flips
