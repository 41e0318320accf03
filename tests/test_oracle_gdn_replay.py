"""The checkpoint + (d, k, g) ring form of the Gated DeltaNet verify oracle against the explicit-state form:
the two are one recurrence on the state the ring stands for (qk_gdn_verify.cu:633-752)."""
import numpy as np
import torch

from bundles_b200 import synth
from oracle import gdn as ogdn
from tests.util import bf16_to_np, close_bf16


def _np(cfg):
    out = {}
    for k, v in cfg.items():
        out[k] = bf16_to_np(v) if v.dtype == torch.bfloat16 else v.numpy()
    return out


def _replay(c):
    return ogdn.gdn_verify_replay(c["mixed"], c["z"], c["a"], c["b"], c["conv_state"], c["conv_w"], c["a_log"],
                                  c["dt_bias"], c["checkpoint"], c["d_ring"], c["k_ring"], c["g_ring"], c["state_idx"],
                                  c["ring_idx"], c["write_pos"], c["cache_base"], c["norm_w"], 1e-6)


def test_empty_ring_is_the_explicit_state_step():
    c = _np(synth.gdn_replay(seed=71, B=2))
    c["write_pos"][:] = 0
    r = _replay(c)
    sidx = c["state_idx"]
    out, _, conv = ogdn.gdn_verify(c["mixed"], c["z"], c["a"], c["b"], c["conv_state"][sidx], c["conv_w"], c["a_log"],
                                   c["dt_bias"], c["checkpoint"][sidx], np.full(2, 4), c["norm_w"], 1e-6)
    assert np.array_equal(r["out"], out)
    assert np.array_equal(r["new_conv"], conv)
    assert (r["slots"] == (c["cache_base"][c["ring_idx"]][:, None] + np.arange(4)) % 16).all()


def test_ring_equals_explicit_state_and_appended_entries_fold_into_it():
    c = _np(synth.gdn_replay(seed=72, B=3))
    c["write_pos"][c["ring_idx"]] = [5, 16, 14]     # mid ring, full ring, the last two entries free
    r = _replay(c)
    sidx, ridx = c["state_idx"], c["ring_idx"]
    state = np.stack([ogdn.ring_state(c["checkpoint"][sidx[i]], c["d_ring"][ridx[i]], c["k_ring"][ridx[i]],
                                      c["g_ring"][ridx[i]], c["write_pos"][ridx[i]], c["cache_base"][ridx[i]])
                      for i in range(3)])
    out, new_state, _ = ogdn.gdn_verify(c["mixed"], c["z"], c["a"], c["b"], c["conv_state"][sidx], c["conv_w"],
                                        c["a_log"], c["dt_bias"], state.astype(np.float32), np.full(3, 4), c["norm_w"])
    ok, err, nbad = close_bf16(r["out"], out)
    assert ok, (err, nbad)
    assert (r["slots"][1] == -1).all() and (r["slots"][2, 2:] == -1).all() and (r["slots"][2, :2] >= 0).all()
    # request 0: write the four entries (high + low parts) into the ring, advance the cursor by n = 1..4: the ring
    # then stands for the explicit state after n tokens
    i, rs = 0, ridx[0]
    d, k, g = c["d_ring"][rs].copy(), c["k_ring"][rs].copy(), c["g_ring"][rs].copy()
    for s in range(4):
        ph = r["slots"][i, s]
        d[:, ph] = r["d_hi"][i, s] + r["d_lo"][i, s]
        k[:, ph] = r["k_hi"][i, s] + r["k_lo"][i, s]
        g[:, ph] = r["g"][i, s]
    for n in (1, 2, 4):
        acc = np.array([n, 0, 0])
        _, st_n, _ = ogdn.gdn_verify(c["mixed"], c["z"], c["a"], c["b"], c["conv_state"][sidx], c["conv_w"], c["a_log"],
                                     c["dt_bias"], state.astype(np.float32), acc, c["norm_w"])
        folded = ogdn.ring_state(c["checkpoint"][sidx[0]], d, k, g, c["write_pos"][rs] + n, c["cache_base"][rs])
        assert np.abs(folded - st_n[0]).max() < 2e-4


def test_padded_request_and_window_record():
    c = _np(synth.gdn_replay(seed=73, B=2))
    c["state_idx"][1] = -1
    r = _replay(c)
    assert not r["out"][4:].any() and r["out"][:4].any()
    x = c["mixed"].reshape(2, 4, 8192)
    cs = c["conv_state"][c["state_idx"][0]]
    assert np.array_equal(r["window"][0][:, :2], cs[:, 1:]) and np.array_equal(r["window"][0][:, 2:], x[0].T)
    assert np.array_equal(r["new_conv"][0], x[0, 1:].T)
