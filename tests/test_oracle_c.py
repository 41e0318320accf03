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
