"""Host-side logic of the multi-GPU path on CPU ranks (gloo, world_size 2): the expert-parallel
exchange and the vocab-shard merge give exactly what one rank computes over everything."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bundles_b200 import parallel, synth
from oracle import attn_lmhead as olm
from oracle import moe as omoe
from oracle import numerics as num
from oracle import router as orouter

K = 4


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class OracleBackend:
    """This rank's experts computed by the CPU oracle (stands in for the GPU operators)."""

    def __init__(self, cfg, e_lo, e_n):
        self.c = {k: (v.numpy() if isinstance(v, torch.Tensor) and v.dtype != torch.bfloat16 else v)
                  for k, v in cfg.items()}
        self.gate_w = cfg["gate_w"].float().numpy()
        self.e_lo, self.e_n = e_lo, e_n

    def route(self, x):
        _, ids, wts = orouter.route(x.numpy(), self.c["wr"], K, self.c["bias"])
        return torch.from_numpy(ids), torch.from_numpy(wts)

    def experts(self, x_all, ids_all, wts_all, cache_all):
        x = x_all.numpy()
        xq, xs = num.quant_int8_rows(x)
        ids, wts = ids_all.numpy(), wts_all.numpy()
        for t in range(x.shape[0]):
            for j in range(K):
                e = int(ids[t, j])
                if self.e_lo <= e < self.e_lo + self.e_n:
                    y, _ = omoe.mlp_int8(xq[t:t + 1], xs[t:t + 1], self.c["w13"][e], self.c["s13"][e],
                                         self.c["w2"][e], self.c["s2"][e])
                    cache_all[t * K + j] = torch.from_numpy(num.bf16_round((y * wts[t, j]).astype(np.float32)))[0]

    def shared_and_combine(self, x, routed_rows):
        xn = x.numpy()
        T = xn.shape[0]
        xq, xs = num.quant_int8_rows(xn)
        y, _ = omoe.mlp_int8(xq, xs, self.c["sh13"], self.c["shs13"], self.c["sh2"], self.c["shs2"])
        cache = np.concatenate([routed_rows.numpy(), num.bf16_round(y)], axis=0)
        return torch.from_numpy(omoe.combine(cache, xn, self.gate_w, K))


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T_local, E = 6, 8
        cfg = synth.moe_w8a8(seed=300, T=T_local * world, H=256, I=128, E=E, zipf_s=1.1)
        e_lo, e_n = parallel.expert_range(E, rank, world)
        ep = parallel.ExpertParallelMoe(OracleBackend(cfg, e_lo, e_n), K, 256)
        x = cfg["x"].float()[rank * T_local:(rank + 1) * T_local].contiguous()
        y = ep(x)
        # vocab-shard merge on the same ranks
        V = 128 * 5
        lm = synth.lmhead(seed=301, T=4, V=V, H=256)
        logits = olm.lmhead_logits(lm["x"].float().numpy(), lm["w"].numpy(), lm["w_s"].numpy())
        lo, hi = parallel.vocab_shards(V, world)[rank]
        mx, idx = olm.shard_argmax(logits[:, lo:hi], lo)
        maxes = [torch.empty(4) for _ in range(world)]
        idxs = [torch.empty(4, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(maxes, torch.from_numpy(mx))
        dist.all_gather(idxs, torch.from_numpy(idx))
        tok = olm.merge_argmax(torch.stack(maxes).numpy(), torch.stack(idxs).numpy())
        torch.save({"y": y, "tok": torch.from_numpy(tok), "ref_tok": torch.from_numpy(np.argmax(logits, 1))},
                   os.path.join(out, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_and_vocab_merge_on_two_cpu_ranks(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    T_local, E = 6, 8
    cfg = synth.moe_w8a8(seed=300, T=T_local * world, H=256, I=128, E=E, zipf_s=1.1)
    x = cfg["x"].float().numpy()
    _, ids, wts = orouter.route(x, cfg["wr"].numpy(), K, cfg["bias"].numpy())
    n = {k: v.numpy() for k, v in cfg.items() if isinstance(v, torch.Tensor) and v.dtype != torch.bfloat16}
    ref = omoe.moe_int8(x, ids, wts, n["w13"], n["s13"], n["w2"], n["s2"], n["sh13"], n["shs13"], n["sh2"], n["shs2"],
                        cfg["gate_w"].float().numpy())
    for r in range(world):
        got = torch.load(os.path.join(tmp_path, f"r{r}.pt"))
        assert np.array_equal(got["y"].numpy(), ref[r * T_local:(r + 1) * T_local]), f"rank {r} differs"
        assert torch.equal(got["tok"], got["ref_tok"].to(torch.int32))


def _gate_worker(rank, world, path, out):
    store = dist.FileStore(path, world)
    gate = parallel.StepGate(store, rank, world, timeout_s=1.0)
    log = []
    try:
        for step in range(1, 4):
            if rank == 1 and step == 3:
                break                      # this rank leaves between steps and never reports for step 3
            log.append(gate.sync())
        log.append("left" if rank == 1 else "done")
    except parallel.RankLost as exc:
        log.append(f"lost: {exc}")
    torch.save(log, os.path.join(out, f"gate{rank}.pt"))


def test_a_rank_that_never_reports_is_noticed_on_the_host(tmp_path):
    """Rank 1 takes part in two steps and leaves; rank 0's roll call for step 3 ends with RankLost after its time limit
    instead of launching a step that would wait for rank 1 on the device."""
    world = 2
    mp.spawn(_gate_worker, args=(world, str(tmp_path / "store"), str(tmp_path)), nprocs=world, join=True)
    log0 = torch.load(os.path.join(tmp_path, "gate0.pt"))
    log1 = torch.load(os.path.join(tmp_path, "gate1.pt"))
    assert log1 == [1, 2, "left"]
    assert log0[:2] == [1, 2] and log0[2].startswith("lost: rank 1 did not report for step 3")


def test_virtual_ranks_share_buffers_and_run_in_lockstep():
    vg = parallel.VirtualEpGroup(3, "cpu")
    views = [vg.view(r) for r in range(3)]
    bufs = [v.shared((4, 2), torch.float32) for v in views]
    ptrs = bufs[0][1]
    assert all(b[1] == ptrs for b in bufs) and len(set(ptrs)) == 3
    assert [b[0].data_ptr() for b in bufs] == ptrs
    with pytest.raises(ValueError):
        views[0].shared((4, 2), torch.float32)
        views[1].shared((4, 2), torch.float32)
        views[2].shared((5, 2), torch.float32)        # a rank asking for another shape
    order = []

    def rank_step(r):
        for phase in range(3):
            order.append((phase, r))
            yield phase
        return r * 10

    assert parallel.run_lockstep([rank_step(r) for r in range(3)]) == [0, 10, 20]
    assert order == [(p, r) for p in range(3) for r in range(3)]


def test_partition_math():
    assert parallel.expert_range(512, 3, 8) == (192, 64)
    with pytest.raises(ValueError):
        parallel.expert_range(10, 0, 4)
    sh = parallel.vocab_shards(151936, 8)
    assert [hi - lo for lo, hi in sh] == [19072] * 3 + [18944] * 5
    assert sh[0][0] == 0 and sh[-1][1] == 151936 and all(lo % 128 == 0 for lo, _ in sh)
    assert parallel.vocab_shards(300, 2) == [(0, 256), (256, 300)]


def test_evidence_prints_one_line_per_path(capsys):
    from bundles_b200 import evidence
    evidence.note("unit_test_path", 12)
    evidence.note("unit_test_path", 40)          # same (process, rank, path, capture state): no second line
    err = capsys.readouterr().err
    assert err.count("B200NODES: unit_test_path") == 1 and "rows=12" in err and "captured=0" in err
