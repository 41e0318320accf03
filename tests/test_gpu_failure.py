"""The failure paths of the device code, exercised without faulting or hanging anything: a wait whose budget runs
out records a status code and the kernel returns with the GPU still usable.  (The reference's waits spin without
a limit: qk_gdn_verify.cu:140-144, qk_moe_up16.cu:656.)"""
import pytest
import torch

from bundles_b200 import ops, synth
from tests.util import dev

pytestmark = pytest.mark.gpu

WAIT_CODES = (101, 102, 103, 104)


@pytest.fixture()
def short_budget():
    ops.set_wait_budget_ns(300_000)        # 0.3 ms instead of one second
    yield
    torch.cuda.synchronize()
    ops.set_wait_budget_ns(0)


def test_a_wait_that_nothing_satisfies_returns_with_a_status(short_budget):
    st = ops.new_status(dev())
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    ops.selftest_wait_expiry(st)
    t1.record()
    torch.cuda.synchronize()
    assert ops.read_status(st) == 101
    assert 0.2 < t0.elapsed_time(t1) < 50.0


def _int8_case():
    cfg = synth.moe_w8a8(seed=31, T=8, E=64, zipf_s=0.0)
    d = {k: (v.to(dev()) if isinstance(v, torch.Tensor) else v) for k, v in cfg.items()}
    _, ids, wts = ops.router(d["x"], d["wr"], 10, d["bias"])
    lists = ops.RoutingLists(8, 10, 64, 128, dev())
    ops.build_lists(ids, wts, lists)
    w = ops.MoeW8A8Weights(d["w13"], d["s13"], d["w2"], d["s2"], d["sh13"], d["shs13"], d["sh2"], d["shs2"])
    return d, lists, w


def test_int8_gemm_winds_down_when_its_stages_never_fill(short_budget):
    """Every role of the GEMM CTA gives up (producer, MMA issuer, epilogue warps), TMEM is freed, and the next
    ordinary call on the same GPU gives the same bits as before."""
    d, lists, w = _int8_case()
    st = ops.new_status(dev())
    want = ops.moe_w8a8(d["x"], w, lists, status=st).clone()
    torch.cuda.synchronize()
    assert ops.read_status(st) == 0
    bad = ops.new_status(dev())
    ops.moe_w8a8(d["x"], w, lists, status=bad, stages=ops.STAGE_UP | ops.TEST_STARVE)
    torch.cuda.synchronize()
    assert ops.read_status(bad) in WAIT_CODES
    again = ops.moe_w8a8(d["x"], w, lists, status=st)
    torch.cuda.synchronize()
    assert ops.read_status(st) == 0 and torch.equal(again, want)


def test_fp8_gemm_winds_down_when_its_stages_never_fill(short_budget):
    cfg = synth.moe_fp8(seed=32, T=8, E=64)
    d = {k: (v.to(dev()) if isinstance(v, torch.Tensor) else v) for k, v in cfg.items()}
    _, ids, wts = ops.router(d["x"], d["wr"], 10)
    lists = ops.RoutingLists(8, 10, 64, 32, dev())
    ops.build_lists(ids, wts, lists)
    w = ops.MoeW8A8Weights(d["w13"], d["s13"], d["w2"], d["s2"], d["sh13"], d["shs13"], d["sh2"], d["shs2"])
    st = ops.new_status(dev())
    want = ops.moe_fp8(d["x"], w, lists, status=st).clone()
    torch.cuda.synchronize()
    assert ops.read_status(st) == 0
    bad = ops.new_status(dev())
    ops.moe_fp8(d["x"], w, lists, status=bad, stages=ops.STAGE_UP | ops.TEST_STARVE)
    torch.cuda.synchronize()
    assert ops.read_status(bad) in WAIT_CODES
    again = ops.moe_fp8(d["x"], w, lists, status=st)
    torch.cuda.synchronize()
    assert ops.read_status(st) == 0 and torch.equal(again, want)


def test_barrier_of_one_rank_passes_and_counts():
    flags = torch.zeros(4 * 8, dtype=torch.int64, device=dev())
    epochs = torch.zeros(4, dtype=torch.int64, device=dev())
    st = ops.new_status(dev())
    for _ in range(3):
        ops.ep_barrier([flags.data_ptr()], epochs, 0, 1, 1_000_000, st)
    torch.cuda.synchronize()
    assert ops.read_status(st) == 0
    assert int(epochs[1]) == 3 and int(flags[8]) == 3 and int(epochs[0]) == 0


def test_barrier_gives_up_on_a_rank_that_never_arrives():
    """Two ranks' flag arrays in this GPU's memory; rank 1 never runs.  Rank 0's barrier ends after its time limit
    with B200_ST_WAIT_PEER, the next one returns at once, and the GPU carries on."""
    f0 = torch.zeros(4 * 8, dtype=torch.int64, device=dev())
    f1 = torch.zeros(4 * 8, dtype=torch.int64, device=dev())
    epochs = torch.zeros(4, dtype=torch.int64, device=dev())
    st = ops.new_status(dev())
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    e[0].record()
    ops.ep_barrier([f0.data_ptr(), f1.data_ptr()], epochs, 0, 0, 500_000, st)
    e[1].record()
    ops.ep_barrier([f0.data_ptr(), f1.data_ptr()], epochs, 0, 0, 500_000, st)
    e[2].record()
    torch.cuda.synchronize()
    assert ops.read_status(st) == 107
    assert 0.4 < e[0].elapsed_time(e[1]) < 50.0
    assert e[1].elapsed_time(e[2]) < 0.3            # no second wait
    assert int(f1[0]) == 2 and int(f0[0]) == 2      # its own epochs were still published
    x = torch.arange(8, device=dev()).sum()
    assert int(x) == 28
