"""The layer-stack step driver: runs end to end on small shapes, is deterministic, leaves no device status."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_decode_step_small_stack():
    from bundles_b200 import decode_step, ops
    dev = torch.device("cuda", 0)
    step = decode_step.DecodeStep(layers=4, B=3, ctx=300, vocab=128 * 40 + 17, experts=64, seed=7, device=dev)
    assert [L["attn"] for L in step.layers] == [False, False, False, True]
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(step.T, 2048, generator=g, device=dev).to(torch.bfloat16)
    # state and caches advance in place: run two identically prepared stacks instead of one stack twice
    other = decode_step.DecodeStep(layers=4, B=3, ctx=300, vocab=128 * 40 + 17, experts=64, seed=7, device=dev)
    a = step.step(x)
    b = other.step(x)
    torch.cuda.synchronize()
    assert ops.read_status(step.status) == 0 and ops.read_status(other.status) == 0
    assert a.shape == (step.T,) and a.dtype == torch.int32
    assert torch.equal(a, b)
    assert int(a.min()) >= 0 and int(a.max()) < 128 * 40 + 17
    # the GDN state of a sequence with accepted > 0 moved, one with accepted == 0 did not
    fresh = decode_step.DecodeStep(layers=4, B=3, ctx=300, vocab=128 * 40 + 17, experts=64, seed=7, device=dev)
    for bi in range(3):
        moved = not torch.equal(step.layers[0]["state"][bi], fresh.layers[0]["state"][bi])
        assert moved == (int(step.accepted[bi]) > 0)


def test_decode_step_ring_layout_with_empty_rings_gives_the_same_tokens():
    # the GDN layers on the checkpoint + ring layout with no committed entries see the same state as the explicit form
    from bundles_b200 import decode_step, ops
    dev = torch.device("cuda", 0)
    kw = dict(layers=4, B=3, ctx=300, vocab=128 * 40 + 17, experts=64, seed=9, device=dev)
    explicit = decode_step.DecodeStep(**kw)
    ring = decode_step.DecodeStep(gdn_layout="ring", **kw)
    g = torch.Generator(device=dev).manual_seed(2)
    x = torch.randn(explicit.T, 2048, generator=g, device=dev).to(torch.bfloat16)
    a, b = explicit.step(x), ring.step(x)
    torch.cuda.synchronize()
    assert ops.read_status(ring.status) == 0
    assert torch.equal(a, b)
    assert torch.equal(ring.layers[0]["state"], decode_step.DecodeStep(**kw).layers[0]["state"]), "checkpoint is read-only"
    # a committed history changes the state the window sees
    hist = decode_step.DecodeStep(gdn_layout="ring", ring_fill=7, **kw)
    c = hist.step(x)
    torch.cuda.synchronize()
    assert ops.read_status(hist.status) == 0 and c.shape == a.shape
