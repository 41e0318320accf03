"""CPU checks of the attention-verify oracle: cache append, causal limit, and two closed-form cases."""
import numpy as np
import torch

from bundles_b200 import synth
from oracle import attn_verify as oav
from oracle.numerics import e4m3_decode, e4m3_encode


def _cfg(**kw):
    cfg = synth.attn_verify(**kw)
    return {k: (v.float().numpy() if v.dtype == torch.bfloat16 else v.numpy()) for k, v in cfg.items()}


def test_append_places_rows_and_columns():
    c = _cfg(seed=11, B=2, ctx=200, ragged=True)
    kc, vc = oav.append_kv(c["kcache"], c["vcache"], c["k_new"], c["v_new"], c["page_table"], c["seqlens"])
    for r, n in enumerate(c["seqlens"]):
        for t in range(4):
            pos = int(n) - 4 + t
            pg = int(c["page_table"][r, pos // 128])
            assert np.array_equal(kc[pg, 1, pos % 128], c["k_new"][4 * r + t, 1])
            assert np.array_equal(vc[pg, 0, :, pos % 128], c["v_new"][4 * r + t, 0])
    changed = (kc != c["kcache"]).sum() + (vc != c["vcache"]).sum()
    assert changed <= 2 * 4 * 2 * 2 * 256


def test_constant_values_pass_through_and_gate():
    """All V equal to a constant c: o = c whatever the scores; out = bf16(bf16(c) * sigmoid(gate))."""
    c = _cfg(seed=12, B=1, ctx=140)
    cval = e4m3_encode(np.array([0.75], dtype=np.float32))[0]
    c["vcache"][:] = cval
    c["v_new"][:] = cval
    out, _, _ = oav.attn_verify(c["q"], c["gate"], c["k_new"], c["v_new"], c["kcache"], c["vcache"], c["page_table"],
                                c["seqlens"])
    sig = 1.0 / (1.0 + np.exp(-c["gate"].reshape(4, -1).astype(np.float64)))
    assert np.allclose(out, 0.75 * sig, rtol=2.0 ** -8, atol=0)


def test_causal_limit_among_drafts():
    """Changing draft token 3's K and V must not change the outputs of draft tokens 0..2."""
    c = _cfg(seed=13, B=1, ctx=50)
    a, _, _ = oav.attn_verify(c["q"], c["gate"], c["k_new"], c["v_new"], c["kcache"], c["vcache"], c["page_table"],
                              c["seqlens"])
    k2, v2 = c["k_new"].copy(), c["v_new"].copy()
    k2[3] = e4m3_encode(-e4m3_decode(k2[3]))
    v2[3] = e4m3_encode(-e4m3_decode(v2[3]))
    b, _, _ = oav.attn_verify(c["q"], c["gate"], k2, v2, c["kcache"], c["vcache"], c["page_table"], c["seqlens"])
    assert np.array_equal(a[:3], b[:3]) and not np.array_equal(a[3], b[3])
