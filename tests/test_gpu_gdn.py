"""Gated DeltaNet verify parity on the GPU through the C ABI: bf16 outputs within 2e-2 / 1e-2,
fp32 state within 1e-3, conv state exact."""
import numpy as np
import pytest
import torch

from bundles_b200 import ops, synth
from oracle import gdn as ogdn
from tests.util import bf16_to_np, close_bf16, dev

pytestmark = pytest.mark.gpu


def _run(cfg):
    d = {k: v.to(dev()) for k, v in cfg.items()}
    state = d["state"].clone()
    conv = d["conv_state"].clone()
    status = ops.new_status(dev())
    out = ops.gdn_verify(d["mixed"], d["z"], d["a"], d["b"], conv, d["conv_w"], d["a_log"], d["dt_bias"], state,
                         d["accepted"], d["norm_w"], 1e-6, status=status)
    torch.cuda.synchronize()
    assert ops.read_status(status) == 0
    return bf16_to_np(out), state.cpu().numpy(), bf16_to_np(conv)


def _oracle(cfg):
    f = bf16_to_np
    return ogdn.gdn_verify(f(cfg["mixed"]), f(cfg["z"]), f(cfg["a"]), f(cfg["b"]), f(cfg["conv_state"]),
                           f(cfg["conv_w"]), cfg["a_log"].numpy(), cfg["dt_bias"].numpy(), cfg["state"].numpy(),
                           cfg["accepted"].numpy(), f(cfg["norm_w"]), 1e-6)


def _check(cfg):
    out, state, conv = _run(cfg)
    r_out, r_state, r_conv = _oracle(cfg)
    ok, err, nbad = close_bf16(out, r_out)
    assert ok, f"out: max err {err}, {nbad} outside tolerance"
    serr = np.abs(state - r_state).max()
    assert serr < 1e-3, f"state max abs err {serr}"
    assert np.array_equal(conv, r_conv), "conv state differs"
    return out, state, conv


def test_config_b32():
    _check(synth.gdn())                       # B=32, accepted ~ U{0..4}


@pytest.mark.parametrize("n", [0, 1, 2, 3, 4])
def test_every_accepted_length(n):
    cfg = synth.gdn(seed=50 + n, B=3)
    cfg["accepted"] = torch.full((3,), n, dtype=torch.int32)
    out, state, conv = _check(cfg)
    if n == 0:                                # full rollback: state and conv state untouched
        assert np.array_equal(state, cfg["state"].numpy())
        assert np.array_equal(conv, bf16_to_np(cfg["conv_state"]))


def test_single_sequence_and_out_of_range_accept_is_clamped():
    cfg = synth.gdn(seed=60, B=1)
    cfg["accepted"] = torch.tensor([9], dtype=torch.int32)
    out, state, conv = _run(cfg)
    cfg["accepted"] = torch.tensor([4], dtype=torch.int32)
    r_out, r_state, r_conv = _oracle(cfg)
    assert np.abs(state - r_state).max() < 1e-3
    assert np.array_equal(conv, r_conv)


def test_two_steps_chain_like_sequential_decode():
    # property: verifying [x0..x3] with accepted = 2 and then the next window equals the oracle run twice
    cfg = synth.gdn(seed=61, B=2)
    cfg["accepted"] = torch.tensor([2, 4], dtype=torch.int32)
    out1, state1, conv1 = _run(cfg)
    cfg2 = synth.gdn(seed=62, B=2)
    cfg2["state"] = torch.from_numpy(state1)
    cfg2["conv_state"] = torch.from_numpy(conv1).to(torch.bfloat16)
    cfg2["accepted"] = torch.tensor([1, 3], dtype=torch.int32)
    _check(cfg2)


def test_large_batch_property_zero_accept_is_identity():
    cfg = synth.gdn(seed=63, B=128)
    cfg["accepted"] = torch.zeros(128, dtype=torch.int32)
    out, state, conv = _run(cfg)
    assert np.array_equal(state, cfg["state"].numpy())
    assert np.array_equal(conv, bf16_to_np(cfg["conv_state"]))
    assert np.isfinite(out).all()
