"""Multi-GPU path on real GPUs (needs >= 2): expert-parallel MoE over NCCL equals the single-GPU
block bit for bit, and the vocab-sharded argmax equals the single-shard argmax."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    import torch.distributed as dist
    from bundles_b200 import moe_block, ops, parallel, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import faulthandler
    faulthandler.dump_traceback_later(240, exit=True)   # a rank stuck in a collective ends itself with a traceback
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        K, T_local, E = 10, 24, 64
        cfg = synth.moe_w8a8(seed=400, T=T_local * world, E=E, zipf_s=1.1)
        d = {k: v.to(dev) for k, v in cfg.items()}
        e_lo, e_n = parallel.expert_range(E, rank, world)
        w_local = ops.MoeW8A8Weights(d["w13"][e_lo:e_lo + e_n].contiguous(), d["s13"][e_lo:e_lo + e_n].contiguous(),
                                     d["w2"][e_lo:e_lo + e_n].contiguous(), d["s2"][e_lo:e_lo + e_n].contiguous(),
                                     d["sh13"], d["shs13"], d["sh2"], d["shs2"])
        backend = parallel.GpuMoeBackend(d["wr"], w_local, d["gate_w"], K, e_lo, bias=d["bias"])
        ep = parallel.ExpertParallelMoe(backend, K, 2048)
        y = ep(d["x"][rank * T_local:(rank + 1) * T_local].contiguous())
        # single-GPU block over all tokens on this rank
        w_all = ops.MoeW8A8Weights(d["w13"], d["s13"], d["w2"], d["s2"], d["sh13"], d["shs13"], d["sh2"], d["shs2"])
        ref = moe_block.MoeBlockW8A8(d["wr"], w_all, d["gate_w"], K, bias=d["bias"], use_graph=False)(d["x"])
        fused = parallel.FusedExpertParallelMoe(backend, K, 2048, T_local)
        xl = d["x"][rank * T_local:(rank + 1) * T_local].contiguous()
        y2 = fused(xl).clone()
        y3 = fused(xl).clone()                      # a second step reuses the peer-written caches
        torch.cuda.synchronize()
        # the pipelined host-to-host form: three calls in a row, every result equal to the plain call's
        xh = xl.cpu().pin_memory()
        ohs = [torch.empty_like(xh).pin_memory() for _ in range(3)]
        for oh in ohs:
            fused.forward_host(xh, oh)
        fused.join_host()
        torch.cuda.synchronize()
        ok_host = all(torch.equal(oh.to(dev), y) for oh in ohs)
        fused.close()
        ok_moe = torch.equal(y, ref[rank * T_local:(rank + 1) * T_local]) and ops.read_status(backend.status) == 0
        ok_moe = ok_moe and torch.equal(y2, y) and torch.equal(y3, y) and ok_host
        # vocab-sharded greedy token
        V = 128 * 21
        lm = synth.lmhead(seed=401, T=16, V=V)
        lo, hi = parallel.vocab_shards(V, world)[rank]
        x = lm["x"].to(dev)
        tok = parallel.sharded_argmax(x, lm["w"][lo:hi].contiguous().to(dev),
                                      lm["w_s"][lo // 128:(hi + 127) // 128].contiguous().to(dev), lo)
        _, idx, _ = ops.lmhead_argmax(x, lm["w"].to(dev), lm["w_s"].to(dev), 0)
        torch.cuda.synchronize()
        # the whole decode + verify step on the ranks (sequences, experts and vocabulary split, the library's own
        # barrier between the phases) against the one-GPU step; twice, the second step on the advanced state
        from bundles_b200 import decode_step
        kw = dict(layers=4, B=4, ctx=300, vocab=128 * 40 + 17, experts=64, seed=21, device=dev, attn_splits=2)
        part = decode_step.DecodeStep(ep=parallel.EpGroup(device=dev), **kw)
        single = decode_step.DecodeStep(**kw)
        gx = torch.Generator(device=dev).manual_seed(5)
        xs = torch.randn(single.T, 2048, generator=gx, device=dev).to(torch.bfloat16)
        Tl = part.T
        ok_step = True
        for _ in range(2):
            got = part.step(xs[rank * Tl:(rank + 1) * Tl].contiguous())
            want = single.step(xs)
            torch.cuda.synchronize()
            ok_step = ok_step and torch.equal(got, want) and \
                torch.equal(part.final_hidden, single.final_hidden[rank * Tl:(rank + 1) * Tl])
        ok_step = ok_step and ops.read_status(part.status) == 0 and ops.read_status(single.status) == 0
        # the logits node with a process group: full logits for the stock processor + the merged greedy tokens
        import sys
        bundle = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bundles_b200", "bundle")
        if bundle not in sys.path:
            sys.path.insert(0, bundle)
        from qwen36_lmhead8 import node as qnode
        from tests.fake_engine import FakeLogitsProcessor
        gw = torch.Generator().manual_seed(402)
        wfull = (torch.randn(V, 2048, generator=gw) * 0.02).to(torch.bfloat16).to(dev)
        head = type("Head", (), {"weight": wfull})()
        xs16 = lm["x"].to(dev)
        sharded = qnode.forward(qnode.prepare(FakeLogitsProcessor(V), dist.group.WORLD), None, xs16, head, None)
        whole = qnode.forward(qnode.prepare(FakeLogitsProcessor(V)), None, xs16, head, None)
        torch.cuda.synchronize()
        ok_node = (sharded.next_token_logits.shape == whole.next_token_logits.shape
                   and torch.equal(sharded.next_token_logits, whole.next_token_logits)
                   and torch.equal(sharded.next_token_ids, whole.next_token_ids))
        dist.barrier()
        torch.save({"moe": ok_moe, "lm": torch.equal(tok, idx), "step": ok_step, "node": ok_node},
                   os.path.join(out, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_matches_single_gpu(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        got = torch.load(os.path.join(tmp_path, f"r{r}.pt"))
        assert got["moe"], f"rank {r}: expert-parallel output differs from the single-GPU block"
        assert got["lm"], f"rank {r}: sharded argmax differs"
        assert got["step"], f"rank {r}: the expert-parallel decode step differs from the one-GPU step"
        assert got["node"], f"rank {r}: the logits node with a process group differs from the one-rank node"
