"""Gated DeltaNet verify on the checkpoint + (d, k, g) ring layout, on the GPU through the C ABI, against the
oracle: bf16 outputs within 2e-2 / 1e-2; appended ring entries (high + low parts) within 1e-3 of the fp64
values; everything the kernel must not touch bit-identical."""
import numpy as np
import pytest
import torch

from bundles_b200 import ops, synth
from oracle import gdn as ogdn
from tests.util import bf16_to_np, close_bf16, dev

pytestmark = pytest.mark.gpu

MUTABLE = ("conv_state", "window", "d_ring", "dlo_ring", "k_ring", "klo_ring", "g_ring")


def _np(cfg):
    return {k: (bf16_to_np(v) if v.dtype == torch.bfloat16 else v.numpy().copy()) for k, v in cfg.items()}


def _run(cfg):
    d = {k: v.to(dev()).clone() for k, v in cfg.items()}
    status = ops.new_status(dev())
    out = ops.gdn_verify_replay(d["mixed"], d["z"], d["a"], d["b"], d["conv_state"], d["conv_w"], d["window"], d["a_log"],
                                d["dt_bias"], d["checkpoint"], d["d_ring"], d["dlo_ring"], d["k_ring"], d["klo_ring"],
                                d["g_ring"], d["state_idx"], d["ring_idx"], d["win_idx"], d["write_pos"],
                                d["cache_base"], d["norm_w"], 1e-6, status=status)
    torch.cuda.synchronize()
    assert ops.read_status(status) == 0
    assert torch.equal(d["checkpoint"].cpu(), cfg["checkpoint"]), "the checkpoint is read-only"
    return bf16_to_np(out), _np({k: d[k].cpu() for k in MUTABLE})


def _check(cfg):
    out, after = _run(cfg)
    c = _np(cfg)
    r = ogdn.gdn_verify_replay(c["mixed"], c["z"], c["a"], c["b"], c["conv_state"], c["conv_w"], c["a_log"], c["dt_bias"],
                               c["checkpoint"], c["d_ring"], c["k_ring"], c["g_ring"], c["state_idx"], c["ring_idx"],
                               c["write_pos"], c["cache_base"], c["norm_w"], 1e-6)
    ok, err, nbad = close_bf16(out, r["out"])
    assert ok, f"out: max err {err}, {nbad} outside tolerance"
    want = {k: c[k].copy() for k in MUTABLE}
    B = len(c["state_idx"])
    for i in range(B):
        if not r["live"][i]:
            continue
        rs, ws, ss = c["ring_idx"][i], c["win_idx"][i], c["state_idx"][i]
        for s in range(4):
            ph = r["slots"][i, s]
            if ph < 0:
                continue
            dsum = after["d_ring"][rs, :, ph] + after["dlo_ring"][rs, :, ph]
            dref = r["d_hi"][i, s] + r["d_lo"][i, s]
            # 1e-3 of the largest entry; a rare bf16 rounding flip of a conv output (fast exp in the SiLU) moves
            # single entries by up to one bf16 step of v
            derr, scale = np.abs(dsum - dref), max(1.0, np.abs(dref).max())
            assert derr.max() < 2.0 ** -6 * scale and (derr > 1e-3 * scale).mean() < 1e-3, "appended d"
            ksum = after["k_ring"][rs, :, ph] + after["klo_ring"][rs, :, ph]
            kref = r["k_hi"][i, s] + r["k_lo"][i, s]
            kerr = np.abs(ksum - kref)
            # the conv output is a bf16 value: a rare rounding flip of it (fast exp in the SiLU) moves one key
            # element by one bf16 step; everything else agrees to the precision of the two parts
            assert (kerr < 2.0 ** -7 * np.abs(kref) + 1e-4).all() and (kerr > 1e-4).mean() < 1e-3, "appended k"
            assert np.abs(after["g_ring"][rs, :, ph] - r["g"][i, s]).max() < 1e-4 * max(1.0, np.abs(r["g"][i, s]).max())
            # low part = bf16(value - high): the two parts carry 16 mantissa bits of the fp32 value
            assert np.abs(after["dlo_ring"][rs, :, ph]).max() <= np.abs(after["d_ring"][rs, :, ph]).max() * 2.0 ** -7
            for name in ("d_ring", "dlo_ring", "k_ring", "klo_ring", "g_ring"):   # compared above, not bit for bit
                want[name][rs, :, ph] = after[name][rs, :, ph]
        want["window"][ws] = r["window"][i]
        want["conv_state"][ss] = r["new_conv"][i]
    for name in MUTABLE:
        assert np.array_equal(after[name], want[name]), f"{name}: touched outside this window's entries, or wrong"
    return out


def test_config_b32_mixed_write_positions():
    _check(synth.gdn_replay())                 # B=32, write positions 0..16, shuffled slots


@pytest.mark.parametrize("wp", [0, 1, 12, 13, 15, 16])
def test_write_positions_around_the_ring_end(wp):
    cfg = synth.gdn_replay(seed=80 + wp, B=3)
    cfg["write_pos"][:] = wp
    _check(cfg)


def test_padded_request_is_zero_and_touches_nothing():
    cfg = synth.gdn_replay(seed=90, B=4)
    cfg["state_idx"][2] = -1
    out = _check(cfg)
    assert not out[8:12].any()


def test_empty_ring_equals_the_explicit_state_kernel_bit_for_bit():
    # with no committed entries the state is the checkpoint itself: the same tensor-core products, the same window
    # algebra, so the two entry points agree exactly
    cfg = synth.gdn_replay(seed=91, B=5, extra_slots=0)
    cfg["write_pos"][:] = 0
    ident = torch.arange(5, dtype=torch.int32)
    cfg["state_idx"], cfg["ring_idx"], cfg["win_idx"] = ident, ident.clone(), ident.clone()
    out, _ = _run(cfg)
    d = {k: v.to(dev()).clone() for k, v in cfg.items()}
    ref = ops.gdn_verify(d["mixed"], d["z"], d["a"], d["b"], d["conv_state"], d["conv_w"], d["a_log"], d["dt_bias"],
                         d["checkpoint"], torch.zeros(5, dtype=torch.int32, device=dev()), d["norm_w"], 1e-6)
    torch.cuda.synchronize()
    assert np.array_equal(out, bf16_to_np(ref))


def test_two_windows_chain_through_the_ring():
    # property: verify a window, accept 2 of its drafts by advancing the cursor, verify the next window: equals the
    # explicit-state kernel stepping its state by the same accepted counts (the ring's bf16 high parts carry the
    # history, so the agreement is to the output tolerance)
    cfg = synth.gdn_replay(seed=92, B=2, extra_slots=0)
    cfg["write_pos"][:] = torch.tensor([3, 9], dtype=torch.int32)
    ident = torch.arange(2, dtype=torch.int32)
    cfg["state_idx"], cfg["ring_idx"], cfg["win_idx"] = ident, ident.clone(), ident.clone()
    c = _np(cfg)
    state = np.stack([ogdn.ring_state(c["checkpoint"][i], c["d_ring"][i], c["k_ring"][i], c["g_ring"][i],
                                      c["write_pos"][i], c["cache_base"][i]) for i in range(2)]).astype(np.float32)
    d = {k: v.to(dev()).clone() for k, v in cfg.items()}
    st = ops.new_status(dev())
    args = lambda: (d["mixed"], d["z"], d["a"], d["b"], d["conv_state"], d["conv_w"], d["window"], d["a_log"], d["dt_bias"],
                    d["checkpoint"], d["d_ring"], d["dlo_ring"], d["k_ring"], d["klo_ring"], d["g_ring"], d["state_idx"],
                    d["ring_idx"], d["win_idx"], d["write_pos"], d["cache_base"], d["norm_w"], 1e-6)
    ops.gdn_verify_replay(*args(), status=st)
    # the engine's part: accept 2 drafts -> cursor + 2, conv state = the last three inputs of [.. s2 x0 x1] = elements
    # [1, 4) of the window record [s1 s2 x0 x1 x2 x3]
    d["write_pos"] += 2
    d["conv_state"] = d["window"][:, :, 1:4].contiguous()
    restored = d["conv_state"].clone()
    nxt = synth.gdn(seed=93, B=2)
    for k in ("mixed", "z", "a", "b"):
        d[k] = nxt[k].to(dev())
    out2 = ops.gdn_verify_replay(*args(), status=st)
    # explicit-state twin
    e_state = torch.from_numpy(state).to(dev())
    e_conv = cfg["conv_state"].to(dev()).clone()
    acc2 = torch.full((2,), 2, dtype=torch.int32, device=dev())
    ops.gdn_verify(cfg["mixed"].to(dev()), cfg["z"].to(dev()), cfg["a"].to(dev()), cfg["b"].to(dev()), e_conv,
                   d["conv_w"], d["a_log"], d["dt_bias"], e_state, acc2, d["norm_w"], 1e-6, status=st)
    assert torch.equal(e_conv, restored), "conv state restored from the window record"
    ref2 = ops.gdn_verify(d["mixed"], d["z"], d["a"], d["b"], e_conv, d["conv_w"], d["a_log"], d["dt_bias"], e_state,
                          acc2, d["norm_w"], 1e-6, status=st)
    torch.cuda.synchronize()
    assert ops.read_status(st) == 0
    ok, err, nbad = close_bf16(bf16_to_np(out2), bf16_to_np(ref2))
    assert ok, f"second window: max err {err}, {nbad} outside tolerance"


def test_ring_fold_matches_the_state_the_ring_stands_for():
    # fold the committed entries (high + low parts) into the checkpoint: equals the state the oracle says the ring
    # stands for; requests with an empty ring and padded requests leave their slots alone
    cfg = synth.gdn_replay(seed=95, B=4)
    cfg["write_pos"][cfg["ring_idx"].long()] = torch.tensor([0, 5, 16, 9], dtype=torch.int32)
    cfg["dlo_ring"] = (torch.randn(cfg["d_ring"].shape) * 1e-3).to(torch.bfloat16)
    cfg["klo_ring"] = (torch.randn(cfg["k_ring"].shape) * 1e-3).to(torch.bfloat16)
    cfg["state_idx"][3] = -1
    c = _np(cfg)
    d = {k: v.to(dev()).clone() for k, v in cfg.items()}
    ops.gdn_ring_fold(d["checkpoint"], d["d_ring"], d["dlo_ring"], d["k_ring"], d["klo_ring"], d["g_ring"], d["state_idx"],
                      d["ring_idx"], d["write_pos"], d["cache_base"])
    torch.cuda.synchronize()
    got = d["checkpoint"].cpu().numpy()
    want = c["checkpoint"].copy()
    for i in range(3):
        rs, ss = c["ring_idx"][i], c["state_idx"][i]
        want[ss] = ogdn.ring_state(c["checkpoint"][ss], c["d_ring"][rs] + c["dlo_ring"][rs], c["k_ring"][rs] + c["klo_ring"][rs],
                                   c["g_ring"][rs], c["write_pos"][rs], c["cache_base"][rs])
    assert np.abs(got - want).max() < 1e-4
    untouched = np.ones(len(want), dtype=bool)
    untouched[c["state_idx"][1:3]] = False          # wp = 0 and the padded request leave their slots alone
    assert np.array_equal(got[untouched], c["checkpoint"][untouched])
