"""Router parity on the GPU, through the C ABI: logits and expert ids bit-exact against the oracle."""
import numpy as np
import pytest
import torch

from bundles_b200 import ops, synth
from oracle import router as orouter
from tests.util import bf16_to_np, dev

pytestmark = pytest.mark.gpu


def _run(T, E, K, seed, bias=False, round_bf16=False, H=2048):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    wr = torch.randn(E, H, generator=g) * 0.02
    b = synth.zipf_bias(E, 1.1, g) if bias else None
    logits, ids, wts = ops.router(x.to(dev()), wr.to(dev()), K, None if b is None else b.to(dev()), round_bf16)
    torch.cuda.synchronize()
    ref_l, ref_ids, ref_w = orouter.route(bf16_to_np(x), wr.numpy(), K, None if b is None else b.numpy(), round_bf16)
    assert np.array_equal(logits.cpu().numpy().view(np.uint32), ref_l.view(np.uint32)), "logits not bit-exact"
    assert np.array_equal(ids.cpu().numpy(), ref_ids), "expert ids differ"
    np.testing.assert_allclose(wts.cpu().numpy(), ref_w, rtol=1e-5, atol=1e-8)
    assert np.allclose(wts.cpu().numpy().sum(1), 1.0, atol=1e-5)


@pytest.mark.parametrize("T", [1, 16, 64, 256])
def test_router_512_top10(T):
    _run(T, 512, 10, 1000 + T)


def test_router_zipf_bias():
    _run(256, 512, 10, 1002, bias=True)


def test_router_reference_shape_bf16_logits():
    _run(48, 256, 8, 77, round_bf16=True)      # the reference's own 256 / top-8 with bf16-rounded logits


def test_router_ragged_and_small_h():
    _run(19, 64, 4, 5, H=256)


def test_router_ties_and_nan():
    E, K, T, H = 512, 10, 4, 128
    x = torch.zeros(T, H, dtype=torch.bfloat16)
    wr = torch.zeros(E, H)
    x[1, 0] = 1.0
    wr[7, 0] = 2.0
    wr[300, 0] = 2.0     # tie between experts 7 and 300 on token 1
    wr[9, 0] = -0.0
    logits, ids, wts = ops.router(x.to(dev()), wr.to(dev()), K)
    torch.cuda.synchronize()
    ids = ids.cpu().numpy()
    assert list(ids[0]) == list(range(K))                 # all-equal row -> lowest ids
    assert list(ids[1][:2]) == [7, 300]
    assert list(ids[1][2:]) == [i for i in range(12) if i != 7][:K - 2]
    # NaN logits (through a NaN bias) rank below everything and never win
    bias = torch.zeros(E)
    bias[5] = float("nan")
    bias[6] = 100.0
    logits, ids, wts = ops.router(x.to(dev()), wr.to(dev()), K, bias.to(dev()))
    torch.cuda.synchronize()
    ref_ids, ref_w = orouter.topk_softmax(logits.cpu().numpy(), K)
    assert np.array_equal(ids.cpu().numpy(), ref_ids)
    assert 5 not in ids.cpu().numpy() and np.all(ids.cpu().numpy()[:, 0] == 6)
    assert np.isfinite(wts.cpu().numpy()).all()


def test_lists_match_oracle():
    T, E, K = 96, 512, 10
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(T, E, generator=g) * 2
    ids_np, w_np = orouter.topk_softmax(logits.numpy(), K)
    pos = torch.ones(T, dtype=torch.int64)
    pos[5] = 0
    pos[40] = 0
    for block in (128, 64, 16):
        lists = ops.RoutingLists(T, K, E, block, dev())
        ops.build_lists(torch.from_numpy(ids_np).to(dev()), torch.from_numpy(w_np).to(dev()), lists, pos.to(dev()))
        torch.cuda.synchronize()
        ref = orouter.routing_lists(ids_np, E, pos.numpy() != 0, block)
        assert np.array_equal(lists.counts.cpu().numpy()[:E], ref["counts"])
        assert int(lists.counts[E]) == T
        assert np.array_equal(lists.row_of_pair.cpu().numpy(), ref["row_of_pair"])
        n = int(ref["offsets"][-1])
        assert np.array_equal(lists.slot_of_row.cpu().numpy()[:n], ref["pair_of_row"])
        assert np.all(lists.slot_of_row.cpu().numpy()[n:T * K] == -1)
        sh = lists.slot_of_row.cpu().numpy()[T * K:]
        assert sh[5] == -1 and sh[40] == -1 and sh[0] == T * K and sh[95] == T * K + 95
        nb = int(lists.nblocks[0])
        nref = len(ref["blk_expert"])
        assert nb == nref + (T + block - 1) // block
        # the shared expert (index E, rows T*K .. T*K + T) is the last expert of each size class
        want = [[], [], [], [], []]
        for e, r0, n_ in zip(ref["blk_expert"], ref["blk_row0"], ref["blk_rows"]):
            want[0 if (n_ == block or block != 128) else 4 - min(3, (4 * n_) // block)].append((int(e), int(r0), int(n_)))
        for r0 in range(0, T, block):
            n_ = min(block, T - r0)
            want[0 if (n_ == block or block != 128) else 4 - min(3, (4 * n_) // block)].append((E, T * K + r0, n_))
        want = [t for cl in want for t in cl]
        got = list(zip(lists.blk_expert.cpu().numpy()[:nb].tolist(), lists.blk_row0.cpu().numpy()[:nb].tolist(),
                       lists.blk_rows.cpu().numpy()[:nb].tolist()))
        assert got == want
        w_rows = lists.wt_of_row.cpu().numpy()[:n]
        assert np.array_equal(w_rows, w_np.reshape(-1)[ref["pair_of_row"]])


def test_lists_expert_parallel_shard():
    T, E, K = 64, 512, 10
    g = torch.Generator().manual_seed(4)
    ids_np, w_np = orouter.topk_softmax((torch.randn(T, E, generator=g) * 2).numpy(), K)
    tot = 0
    for r in range(8):
        lists = ops.RoutingLists(T, K, 64, 128, dev())
        ops.build_lists(torch.from_numpy(ids_np).to(dev()), torch.from_numpy(w_np).to(dev()), lists, None,
                        e_lo=64 * r, with_shared=False)
        torch.cuda.synchronize()
        c = lists.counts.cpu().numpy()
        assert np.array_equal(c[:64], np.bincount(ids_np.reshape(-1), minlength=E)[64 * r:64 * r + 64])
        assert c[64] == 0
        tot += int(c[:64].sum())
    assert tot == T * K


def test_lists_shared_rows_for_a_token_range():
    """An expert-parallel rank builds lists over the gathered tokens but shared-expert rows for its own only."""
    T, E, K = 320, 512, 10
    g = torch.Generator().manual_seed(5)
    ids_np, w_np = orouter.topk_softmax((torch.randn(T, E, generator=g) * 2).numpy(), K)
    lo, n = 160, 160
    lists = ops.RoutingLists(T, K, 64, 128, dev())
    ops.build_lists(torch.from_numpy(ids_np).to(dev()), torch.from_numpy(w_np).to(dev()), lists, None, e_lo=128,
                    shared_range=(lo, n))
    torch.cuda.synchronize()
    c, off = lists.counts.cpu().numpy(), lists.offsets.cpu().numpy()
    assert c[64] == n and off[64] == T * K + lo and off[65] == T * K + lo + n
    slot = lists.slot_of_row.cpu().numpy()
    assert np.array_equal(slot[T * K + lo:T * K + lo + n], np.arange(T * K + lo, T * K + lo + n))
    nb = int(lists.nblocks.item())
    be, b0, br = (t.cpu().numpy()[:nb] for t in (lists.blk_expert, lists.blk_row0, lists.blk_rows))
    sh = be == 64
    assert list(b0[sh]) == [T * K + lo, T * K + lo + 128] and list(br[sh]) == [128, 32]
