"""LM head shard + fused argmax on the GPU through the C ABI: argmax ids equal to the oracle's,
logits within the bf16 tolerance."""
import numpy as np
import pytest
import torch

from bundles_b200 import ops, synth
from oracle import attn_lmhead as olm
from tests.util import bf16_to_np, close_bf16, dev

pytestmark = pytest.mark.gpu


def _check_ids(idx, mx, ref_logits, lo=0):
    """ids must equal the oracle's argmax; a differing id is accepted only where the oracle's two
    logits are closer than the tensor core's accumulation noise (near tie)."""
    r_mx, r_idx = olm.shard_argmax(ref_logits, lo)
    for t in np.nonzero(idx != r_idx)[0]:
        a, b = ref_logits[t, idx[t] - lo], ref_logits[t, r_idx[t] - lo]
        assert abs(a - b) <= 2e-4 * max(1.0, abs(b)), f"row {t}: {idx[t]} vs {r_idx[t]} ({a} vs {b})"
    np.testing.assert_allclose(mx, r_mx, rtol=2e-3, atol=2e-3)
    return int((idx != r_idx).sum())


@pytest.mark.parametrize("T,V", [(64, 4096), (5, 1280), (16, 128 * 37), (150, 128 * 9 + 5), (100, 128 * 3), (256, 128 * 5 + 40)])
def test_single_shard(T, V):
    cfg = synth.lmhead(seed=70 + T, T=T, V=V)
    mx, idx, logits = ops.lmhead_argmax(cfg["x"].to(dev()), cfg["w"].to(dev()), cfg["w_s"].to(dev()), 0, True,
                                        status=(st := ops.new_status(dev())))
    torch.cuda.synchronize()
    assert ops.read_status(st) == 0
    ref = olm.lmhead_logits(bf16_to_np(cfg["x"]), cfg["w"].numpy(), cfg["w_s"].numpy())
    ok, err, nbad = close_bf16(logits.cpu().numpy(), ref)
    assert ok, (err, nbad)
    assert _check_ids(idx.cpu().numpy(), mx.cpu().numpy(), ref) == 0


def test_exact_ties_go_to_the_lower_id():
    cfg = synth.lmhead(seed=80, T=8, V=1024)
    w = cfg["w"].clone()
    w[900] = w[17]          # identical rows in different tiles -> identical logits
    w[300] = w[17]
    ws = cfg["w_s"].clone()
    ws[900 // 128] = ws[17 // 128]
    ws[300 // 128] = ws[17 // 128]
    x = cfg["x"]
    mx, idx, logits = ops.lmhead_argmax(x.to(dev()), w.to(dev()), ws.to(dev()), 0, True)
    torch.cuda.synchronize()
    lg = logits.cpu().numpy()
    assert np.array_equal(lg[:, 17], lg[:, 300]) and np.array_equal(lg[:, 17], lg[:, 900])
    ref_idx = np.argmax(lg, axis=1)          # first occurrence = lowest id, on the kernel's own logits
    assert np.array_equal(idx.cpu().numpy(), ref_idx)


def test_eight_shards_merge_equals_whole_vocab():
    V, T = 128 * 75, 64                                        # 75 scale blocks -> 3 x 10 + 5 x 9 blocks
    cfg = synth.lmhead(seed=81, T=T, V=V)
    ref = olm.lmhead_logits(bf16_to_np(cfg["x"]), cfg["w"].numpy(), cfg["w_s"].numpy())
    shards = olm.vocab_shards(V, 8)
    assert [hi - lo for lo, hi in shards] == [1280] * 3 + [1152] * 5
    x = cfg["x"].to(dev())
    maxes, idxs = [], []
    for lo, hi in shards:
        mx, idx, _ = ops.lmhead_argmax(x, cfg["w"][lo:hi].contiguous().to(dev()),
                                       cfg["w_s"][lo // 128:hi // 128].contiguous().to(dev()), lo)
        maxes.append(mx)
        idxs.append(idx)
    tokens = ops.argmax_merge(torch.stack(maxes), torch.stack(idxs))
    torch.cuda.synchronize()
    r_m = [olm.shard_argmax(ref[:, lo:hi], lo) for lo, hi in shards]
    r_tok = olm.merge_argmax(np.stack([m for m, _ in r_m]), np.stack([i for _, i in r_m]))
    assert np.array_equal(r_tok, np.argmax(ref, axis=1))
    _check_ids(tokens.cpu().numpy(), torch.stack(maxes).max(0).values.cpu().numpy(), ref)
    assert np.array_equal(tokens.cpu().numpy(), r_tok)


def test_full_vocab_shard_of_the_8way_split():
    lo, hi = olm.vocab_shards(151936, 8)[0]
    assert (lo, hi) == (0, 19072)
    cfg = synth.lmhead(T=64, V=hi - lo)
    mx, idx, _ = ops.lmhead_argmax(cfg["x"].to(dev()), cfg["w"].to(dev()), cfg["w_s"].to(dev()), lo)
    torch.cuda.synchronize()
    ref = olm.lmhead_logits(bf16_to_np(cfg["x"]), cfg["w"].numpy(), cfg["w_s"].numpy())
    _check_ids(idx.cpu().numpy(), mx.cpu().numpy(), ref, lo)
