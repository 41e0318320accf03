"""Attention-verify core against the oracle (paged e4m3 KV, 4 drafts, causal tail, split-KV merge, gate)."""
import numpy as np
import pytest
import torch

from oracle import attn_verify as oav

pytestmark = pytest.mark.gpu


def _run(B, ctx, ragged, splits, seed):
    from bundles_b200 import ops, synth
    dev = torch.device("cuda", 0)
    cfg = synth.attn_verify(seed=seed, B=B, ctx=ctx, ragged=ragged)
    if ragged:  # include the shortest legal request and a length that ends exactly on a page
        cfg["seqlens"][0] = 4
        if B > 1:
            cfg["seqlens"][1] = min(ctx, 128) if ctx >= 128 else ctx
    want, kc, vc = oav.attn_verify(cfg["q"].numpy(), cfg["gate"].float().numpy(), cfg["k_new"].numpy(),
                                   cfg["v_new"].numpy(), cfg["kcache"].numpy(), cfg["vcache"].numpy(),
                                   cfg["page_table"].numpy(), cfg["seqlens"].numpy())
    d = {k: v.to(dev) for k, v in cfg.items()}
    status = ops.new_status(dev)
    out = ops.attn_verify(d["q"], d["gate"], d["k_new"], d["v_new"], d["kcache"], d["vcache"], d["page_table"],
                          d["seqlens"], splits=splits, status=status)
    torch.cuda.synchronize()
    assert ops.read_status(status) == 0
    # the drafts' rows are in the cache, bit for bit, and nothing else moved
    assert np.array_equal(d["kcache"].cpu().numpy(), kc)
    assert np.array_equal(d["vcache"].cpu().numpy(), vc)
    got = out.float().cpu().numpy()
    # bf16 output of a convex combination of e4m3 values: 2 bf16 ulps of the largest magnitude in play
    err = np.abs(got - want)
    tol = 2.0 ** -7 * np.maximum(np.abs(want), 0.25)
    assert np.all(err <= tol), f"max err {err.max()} at {np.unravel_index(err.argmax(), err.shape)}"


@pytest.mark.parametrize("B,ctx,ragged,splits", [(1, 4, False, 1), (2, 100, True, 1), (3, 700, True, 1),
                                                 (3, 700, True, 3), (2, 1500, True, 16), (5, 384, False, None)])
def test_attn_verify_matches_oracle(B, ctx, ragged, splits):
    _run(B, ctx, ragged, splits, seed=900 + B + ctx)


def test_attn_verify_second_step_reuses_cache():
    """Two steps in a row on the same cache: the second sees the first step's 4 tokens as prefix."""
    from bundles_b200 import ops, synth
    dev = torch.device("cuda", 0)
    cfg = synth.attn_verify(seed=931, B=2, ctx=300, ragged=True)
    d = {k: v.to(dev) for k, v in cfg.items()}
    ops.attn_verify(d["q"], d["gate"], d["k_new"], d["v_new"], d["kcache"], d["vcache"], d["page_table"], d["seqlens"])
    cfg2 = synth.attn_verify(seed=932, B=2, ctx=300, ragged=True)
    sl2 = (cfg["seqlens"] + 4).to(torch.int32)
    out2 = ops.attn_verify(cfg2["q"].to(dev), cfg2["gate"].to(dev), cfg2["k_new"].to(dev), cfg2["v_new"].to(dev),
                           d["kcache"], d["vcache"], d["page_table"], sl2.to(dev))
    torch.cuda.synchronize()
    _, kc, vc = oav.attn_verify(cfg["q"].numpy(), cfg["gate"].float().numpy(), cfg["k_new"].numpy(), cfg["v_new"].numpy(),
                                cfg["kcache"].numpy(), cfg["vcache"].numpy(), cfg["page_table"].numpy(),
                                cfg["seqlens"].numpy())
    want, _, _ = oav.attn_verify(cfg2["q"].numpy(), cfg2["gate"].float().numpy(), cfg2["k_new"].numpy(),
                                 cfg2["v_new"].numpy(), kc, vc, cfg["page_table"].numpy(), sl2.numpy())
    err = np.abs(out2.float().cpu().numpy() - want)
    assert np.all(err <= 2.0 ** -7 * np.maximum(np.abs(want), 0.25))
