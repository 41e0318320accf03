"""The layer-stack step driver against the composed oracle, and its expert-parallel form against the single-GPU form.

Parity with the oracle is checked layer by layer and stage by stage, every stage on the GPU's own input of that
stage (a difference of one bf16 ulp in a GEMM's input can move an e4m3 code of its quantised operand by a whole
step, or flip a router pick between two nearly equal logits; a free-running comparison would then compare different
arithmetic): per layer the mixer's projection, the rows fed to the router, the expert ids (exactly), the routed
rows, the block's output, the next layer's rows within the bf16 tolerance (2e-2 relative / 1e-2 absolute), the
running residual exactly, the GDN state within 1e-3, the conv state (carried in_proj outputs) within the bf16
tolerance; then the tokens.
"""
import numpy as np
import pytest
import torch

from oracle import attn_lmhead as al
from tests.util import bf16_to_np, close_bf16

pytestmark = pytest.mark.gpu

SMALL = dict(layers=4, ctx=300, vocab=128 * 40 + 17, experts=64)


def _np(t):
    if t.dtype == torch.bfloat16:
        return bf16_to_np(t)
    return t.detach().cpu().numpy()


def to_model(step):
    """A DecodeStep's weights and state as the oracle's dict of numpy arrays (taken BEFORE the step runs)."""
    layers = []
    for L in step.layers:
        d = {k: _np(v) for k, v in L.items() if isinstance(v, torch.Tensor)}
        d["attn"] = L["attn"]
        w = L["w"]
        for k in ("w13", "s13", "w2", "s2", "sh13", "shs13", "sh2", "shs2"):
            d[k] = _np(getattr(w, k))
        layers.append(d)
    return dict(layers=layers, first_norm=_np(step.first_norm), lm_w=_np(step.lm_w), lm_s=_np(step.lm_s),
                cos_sin=_np(step.cos_sin), positions=_np(step.positions), seqlens=_np(step.seqlens),
                accepted=_np(step.accepted))


def _x(T, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    return torch.randn(T, 2048, generator=g, device=dev).to(torch.bfloat16)


def test_small_stack_matches_the_composed_oracle():
    from bundles_b200 import decode_step, ops
    from oracle import decode_step as ostep
    dev = torch.device("cuda", 0)
    step = decode_step.DecodeStep(B=3, seed=7, device=dev, **SMALL)
    assert [L["attn"] for L in step.layers] == [False, False, False, True]
    model = to_model(step)
    x = _x(step.T, 1, dev)
    step.trace = []
    tokens = step.step(x)
    torch.cuda.synchronize()
    assert ops.read_status(step.status) == 0
    assert tokens.shape == (step.T,) and tokens.dtype == torch.int32
    for li, (L, rec) in enumerate(zip(model["layers"], step.trace)):
        # every stage of the layer on the GPU's own input of that stage
        h_in, r_in = _np(rec["h_in"]), _np(rec["residual_in"])
        if L["attn"]:
            proj, kc, vc = ostep.mixer_attn(L, h_in, model["positions"], model["cos_sin"], model["seqlens"])
        else:
            proj, state, conv = ostep.mixer_gdn(L, h_in, model["accepted"])
        ok, err, nbad = close_bf16(_np(rec["proj"]), proj)
        assert ok, (li, "proj", err, nbad)
        h2, r_mid = al.add_rmsnorm(_np(rec["proj"]), r_in, L["post_norm"])
        assert np.array_equal(_np(rec["residual_mid"]), r_mid), li
        ok, err, nbad = close_bf16(_np(rec["h2"]), h2)
        assert ok, (li, "h2", err, nbad)
        _, ids, wts = ostep.route(L, _np(rec["h2"]))
        assert np.array_equal(_np(rec["ids"]), ids), (li, "expert ids")          # the router is bit-exact
        np.testing.assert_allclose(_np(rec["wts"]), wts, rtol=1e-5, atol=1e-7)
        moe_out, dbg = ostep.moe(L, _np(rec["h2"]), ids, _np(rec["wts"]))
        ok, err, nbad = close_bf16(_np(rec["cache"]), dbg["cache"])
        assert ok, (li, "cache", err, nbad)
        ok, err, nbad = close_bf16(_np(rec["moe_out"]), moe_out)
        assert ok, (li, "moe_out", err, nbad)
        h_out, r_out = al.add_rmsnorm(_np(rec["moe_out"]), r_mid, L["next_norm"])
        assert np.array_equal(_np(rec["residual_out"]), r_out), li
        ok, err, nbad = close_bf16(_np(rec["h_out"]), h_out)
        assert ok, (li, "h_out", err, nbad)
        gl = step.layers[li]
        if L["attn"]:
            assert (_np(gl["kcache"]) != kc).mean() < 1e-3 and (_np(gl["vcache"]) != vc).mean() < 1e-3, li
        else:
            assert np.abs(_np(gl["state"]) - state).max() < 1e-3, li
            ok, err, nbad = close_bf16(_np(gl["conv_state"]), conv)   # the carried inputs are the in_proj's bf16 outputs
            assert ok, (li, "conv_state", err, nbad)
    # tokens from the GPU's own final hidden rows
    ref_tokens, logits = ostep.lm_tokens(model, _np(step.final_hidden))
    got = tokens.cpu().numpy()
    for t in np.nonzero(got != ref_tokens)[0]:
        a, b = logits[t, got[t]], logits[t, ref_tokens[t]]
        assert abs(a - b) <= 2e-4 * max(1.0, abs(b)), (t, got[t], ref_tokens[t])


def test_free_running_oracle_agrees_on_a_two_layer_stack():
    # without teacher forcing: two GDN layers, final hidden rows within the bf16 tolerance and the same tokens
    from bundles_b200 import decode_step, ops
    from oracle import decode_step as ostep
    dev = torch.device("cuda", 0)
    step = decode_step.DecodeStep(B=2, seed=11, device=dev, **dict(SMALL, layers=2))
    model = to_model(step)
    x = _x(step.T, 3, dev)
    tokens = step.step(x)
    torch.cuda.synchronize()
    assert ops.read_status(step.status) == 0
    ref_tokens, ref_h, outs = ostep.decode_step(model, bf16_to_np(x))
    step2 = decode_step.DecodeStep(B=2, seed=11, device=dev, **dict(SMALL, layers=2))
    step2.trace = []
    step2.step(x)
    same_routing = all(np.array_equal(_np(r["ids"]), o["ids"]) for r, o in zip(step2.trace, outs))
    if same_routing:   # otherwise a near tie flipped a pick and the rows legitimately differ
        ok, err, nbad = close_bf16(_np(step.final_hidden), ref_h, rtol=4e-2, atol=2e-2)
        assert ok, (err, nbad)
        assert (tokens.cpu().numpy() == ref_tokens).mean() >= 0.75


def test_step_is_deterministic_and_rolls_back():
    from bundles_b200 import decode_step, ops
    dev = torch.device("cuda", 0)
    step = decode_step.DecodeStep(B=3, seed=7, device=dev, **SMALL)
    other = decode_step.DecodeStep(B=3, seed=7, device=dev, **SMALL)
    x = _x(step.T, 1, dev)
    a, b = step.step(x), other.step(x)
    torch.cuda.synchronize()
    assert ops.read_status(step.status) == 0 and ops.read_status(other.status) == 0
    assert torch.equal(a, b)
    assert int(a.min()) >= 0 and int(a.max()) < SMALL["vocab"]
    # the GDN state of a sequence with accepted > 0 moved, one with accepted == 0 did not
    fresh = decode_step.DecodeStep(B=3, seed=7, device=dev, **SMALL)
    for bi in range(3):
        moved = not torch.equal(step.layers[0]["state"][bi], fresh.layers[0]["state"][bi])
        assert moved == (int(step.accepted[bi]) > 0)


def test_ring_layout_with_empty_rings_gives_the_same_tokens():
    # the GDN layers on the checkpoint + ring layout with no committed entries see the same state as the explicit form
    from bundles_b200 import decode_step, ops
    dev = torch.device("cuda", 0)
    kw = dict(B=3, seed=9, device=dev, **SMALL)
    explicit = decode_step.DecodeStep(**kw)
    ring = decode_step.DecodeStep(gdn_layout="ring", **kw)
    x = _x(explicit.T, 2, dev)
    a, b = explicit.step(x), ring.step(x)
    torch.cuda.synchronize()
    assert ops.read_status(ring.status) == 0
    assert torch.equal(a, b)
    assert torch.equal(ring.layers[0]["state"], decode_step.DecodeStep(**kw).layers[0]["state"]), "checkpoint is read-only"
    hist = decode_step.DecodeStep(gdn_layout="ring", ring_fill=7, **kw)
    c = hist.step(x)
    torch.cuda.synchronize()
    assert ops.read_status(hist.status) == 0 and c.shape == a.shape


@pytest.mark.parametrize("world,B", [(2, 4), (4, 4), (2, 20), (8, 8)])
def test_expert_parallel_form_equals_the_single_gpu_form(world, B):
    """Virtual ranks on one GPU (every rank's buffers in the same memory, steps in lockstep): sequences, experts and
    vocabulary split `world` ways give the same tokens, hidden rows, GDN states and KV bytes as the one-GPU step.
    B = 20 makes 80 rows: the dense projections and the LM head run as two 64-row launches."""
    from bundles_b200 import decode_step, ops, parallel
    dev = torch.device("cuda", 0)
    kw = dict(B=B, seed=21, device=dev, attn_splits=2, **SMALL)     # same split count in both forms: same merge order
    single = decode_step.DecodeStep(**kw)
    x = _x(single.T, 5, dev)
    want = single.step(x)
    torch.cuda.synchronize()
    assert ops.read_status(single.status) == 0
    vg = parallel.VirtualEpGroup(world, dev)
    ranks = [decode_step.DecodeStep(ep=vg.view(r), **kw) for r in range(world)]
    Tl = ranks[0].T
    got = decode_step.step_virtual(ranks, [x[r * Tl:(r + 1) * Tl].contiguous() for r in range(world)])
    torch.cuda.synchronize()
    for r, s in enumerate(ranks):
        assert ops.read_status(s.status) == 0
        assert torch.equal(got[r], want), f"rank {r}: tokens differ"
        assert torch.equal(s.final_hidden, single.final_hidden[r * Tl:(r + 1) * Tl]), f"rank {r}: hidden rows differ"
        Bl = s.B
        for li, (Ls, L1) in enumerate(zip(s.layers, single.layers)):
            if Ls["attn"]:
                continue
            assert torch.equal(Ls["state"], L1["state"][r * Bl:(r + 1) * Bl]), (r, li)
            assert torch.equal(Ls["conv_state"], L1["conv_state"][r * Bl:(r + 1) * Bl]), (r, li)
