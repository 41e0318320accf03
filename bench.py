"""Benchmark of the decode / speculative-verify hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload step|moe_int8]

Default workload (`config.workload`): one whole decode + verify step of the 48-layer stack (36 Gated DeltaNet + 12
gated-attention layers, every layer with a 512-expert top-10 fp8 MoE + shared expert; LM head 151936 x 2048 fp8 with
greedy argmax) for a batch of 64 sequences x 4 draft tokens at 8192 tokens of context, random-init weights and
synthetic state / KV pages drawn from a seed.  One step = one CUDA-graph replay of every launch of the stack.
On N GPUs the same batch is split N ways (sequences, experts and vocabulary; "strong" scaling: the batch is the
configuration's, 64): the expert exchange is peer stores over NVLink plus the library's bounded barrier, no NCCL
call in the step.  A step streams every expert that is hit (about 1.6 GB per layer on one GPU), far more than the
126 MB L2, so no flush is needed.

One JSON line on stdout (rank 0): rows (draft tokens) verified per second with inputs resident in HBM (`value`),
the same from pinned host memory to pinned host memory (`e2e`), the roofline of the dominant kernel (the fp8 gate/up
expert GEMM) from CUDA events, the CPU baseline (the C restatement of the same arithmetic on the host cores, on a
stated sample) and, under `kernels`, every other kernel of the path at its named configuration (1 GPU only).
`--workload moe_int8` measures the int8 W8A8 MoE block at 256 tokens instead (BASELINE configuration 2).
`--impl reference` times only the CPU restatement.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

T, H, I, E, K = 256, 2048, 512, 512, 10
LAYERS, BATCH, CTX, VOCAB = 48, 64, 8192, 151936
STEP_WORKLOAD = ("48-layer decode+verify step: batch 64 x 4 draft tokens, ctx 8192, 36 GDN + 12 gated-attention layers, "
                 "512 fp8 experts top-10 + shared per layer, LM head 151936 fp8 + greedy argmax")
STEP_METRIC = "decode-step tokens/s @bs64 (draft-token rows verified per second; us/layer = ms_per_step*1000/48)"
WORKLOAD = "int8 W8A8 routed MoE block at decode: T=256 H=2048 E=512 top-10 I=512 + shared expert, Zipf(1.1) router bias"
METRIC = "decode tokens/s through one MoE layer (us/layer = ms_per_step*1000)"


_OUT = None


def quiet_stdout():
    """From here on file descriptor 1 is stderr, so that whatever a library writes to stdout (NCCL's version line at
    communicator set-up) cannot land beside the result; `emit` writes the JSON line to the real stdout."""
    global _OUT
    if _OUT is None:
        sys.stdout.flush()
        _OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line):
    out = _OUT if _OUT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline(cfg_host, repeats=2):
    """The C restatement (router + int8 MoE block + combine) on the host cores, whole workload."""
    import numpy as np
    from oracle import clib
    clib.use_all_cores()
    xb = cfg_host["x"].view(__import__("torch").int16).numpy().view(np.uint16)
    gb = cfg_host["gate_w"].view(__import__("torch").int16).numpy().view(np.uint16)
    n = {k: v.numpy() for k, v in cfg_host.items() if k not in ("x", "gate_w") and v is not None}
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        logits = clib.gate_logits(xb, n["wr"], n["bias"])
        ids, wts = clib.topk(logits, K)
        clib.moe_w8a8(xb, ids, wts, n["w13"], n["s13"], n["w2"], n["s2"], n["sh13"], n["shs13"], n["sh2"], n["shs2"], gb)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best, clib.threads()


def run_reference(args, rank, world):
    """`--impl reference`: the reference path's CPU arithmetic (the oracle's C twin) on the host cores."""
    if rank != 0:
        return
    import torch
    from bundles_b200 import synth
    cfg = synth.moe_w8a8(T=T, H=H, I=I, E=E)
    times = []
    for i in range(args.warmup + args.steps):
        dt, cores = cpu_baseline(cfg, repeats=1)
        if i >= args.warmup:
            times.append(dt)
    ms = 1000.0 * sum(times) / len(times)
    val = T / (ms / 1000.0)
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": WORKLOAD, "l2": "not applicable (CPU)"},
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port",
                             "sample": "whole workload (256 tokens), every step"},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


def other_kernels(dev, steps, warmup, only=None):
    """The other kernels of the hot path at their named configurations, each timed alone with CUDA events
    (inputs larger than L2 or rotated over several copies so that every launch reads HBM).  `only`: run a single
    entry with plain launches instead of graph replays (the target of an ncu capture; `attn_verify` then runs a
    16-request case, 134 MB of KV)."""
    import math
    import torch
    from bundles_b200 import ops, synth
    from bundles_b200.synth import quant_fp8_blocks
    hbm, which = peaks()
    out = {}

    def want(name):
        return only is None or only == name

    def timed(fn, n=steps, calls=1, graph=only is None):
        """ms per call of fn.  The calls are captured into a CUDA graph (`calls` of them, e.g. one per
        rotating buffer) so that host-side launch cost does not hide the device time."""
        for _ in range(max(warmup, calls)):
            fn()
        torch.cuda.synchronize()
        run = fn
        per = 1
        if graph:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for _ in range(calls):
                    fn()
            run, per = gr.replay, calls
            run()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            run()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (n * per)

    # dense fp8 GEMM peak of this GPU (cuBLASLt through torch._scaled_mm, 8192^3), the tensor-pipe denominator
    fp8_peak = None
    try:
        if only is not None:
            raise RuntimeError("skipped in single-kernel mode")
        a = torch.randn(8192, 8192, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(8192, 8192, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        ms = min(timed(lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16), 5,
                       graph=False) for _ in range(3))
        fp8_peak = 2 * 8192 ** 3 / (ms * 1e-3) / 1e12
        del a, b
    except Exception as exc:  # noqa: BLE001
        out["fp8_peak_error"] = repr(exc)[:120]
    out["fp8_dense_tflops_measured"] = fp8_peak
    # dense int8 GEMM peak (torch._int_mm, 8192^3), the denominator of the int8 tensor-pipe fractions
    int8_peak = None
    try:
        if only is not None:
            raise RuntimeError("skipped in single-kernel mode")
        a8 = torch.randint(-127, 128, (8192, 8192), device=dev, dtype=torch.int8)
        b8 = torch.randint(-127, 128, (8192, 8192), device=dev, dtype=torch.int8).t()
        ms = min(timed(lambda: torch._int_mm(a8, b8), 5, graph=False) for _ in range(3))
        int8_peak = 2 * 8192 ** 3 / (ms * 1e-3) / 1e12
        del a8, b8
    except Exception as exc:  # noqa: BLE001
        out["int8_peak_error"] = repr(exc)[:120]
    out["int8_dense_tops_measured"] = int8_peak
    out["_int8_peak"] = int8_peak

    # Gated DeltaNet verify: B = 32 x 4 drafts; 4 rotating copies of the state (268 MB > L2)
    st = ops.new_status(dev)
    it = [0]
    if want("gdn_verify"):
        _gdn_entry(dev, ops, synth, timed, st, it, out, hbm, which)
    for name, Bv in (("attn_verify_b64", 64), ("attn_verify_b8", 8), ("attn_verify", 16)):
        if not (want(name) and (only is not None or name != "attn_verify")):
            continue
        _attn_verify_entry(dev, ops, synth, timed, st, out, hbm, which, name, Bv)
    torch.cuda.empty_cache()
    if want("attn_front"):
        _attn_front_entry(dev, ops, synth, timed, st, out, fp8_peak)
    if want("lmhead_shard_argmax"):
        _lmhead_entry(dev, ops, synth, timed, st, it, out, hbm)
    if want("moe_fp8_t16") or want("router"):
        _moe_fp8_router_entry(dev, ops, synth, timed, st, out, hbm, want)
    if want("moe_w8a8_prefill"):
        _moe_w8a8_prefill_entry(dev, ops, synth, timed, st, out)
    out.pop("_int8_peak", None)
    if want("moe_w8a8_t256"):
        _moe_w8a8_block_entry(dev, ops, synth, timed, st, out, hbm, which)
    if want("moe_fp8_t256"):
        _moe_fp8_block_entry(dev, ops, timed, st, out, hbm, which, sets=1 if only is not None else 3)
    return out


def _moe_w8a8_prefill_entry(dev, ops, synth, timed, st, out):
    # the int8 block at prefill-sized chunks (1024 and 2048 tokens): the same kernels over longer block lists,
    # many experts with several 128-row blocks; int8 operations per second over the routed + shared rows
    import torch
    torch.cuda.empty_cache()
    try:
        Hh, Ii, Kk = 2048, 512, 10
        c = synth.moe_w8a8(T=2048, device=dev)
        w = ops.MoeW8A8Weights(c["w13"], c["s13"], c["w2"], c["s2"], c["sh13"], c["shs13"], c["sh2"], c["shs2"])
        for Tn in (1024, 2048):
            x = c["x"][:Tn].contiguous()
            lists = ops.RoutingLists(Tn, Kk, 512, 128, dev)
            scr = ops.router_scratch(Tn, Hh, 512, dev)
            ids = torch.empty(Tn, Kk, dtype=torch.int32, device=dev)
            wts = torch.empty(Tn, Kk, dtype=torch.float32, device=dev)
            ws = ops.moe_w8a8_workspace(Tn, Hh, Ii, Kk, dev)
            cache = torch.zeros(Tn * (Kk + 1), Hh, dtype=torch.bfloat16, device=dev)
            res = torch.empty(Tn, Hh, dtype=torch.bfloat16, device=dev)

            def block():
                ops.router(x, c["wr"], Kk, c["bias"], scratch=scr, want_logits=False, ids=ids, wts=wts)
                ops.build_lists(ids, wts, lists)
                ops.moe_w8a8(x, w, lists, cache=cache, ws=ws, status=st)
                ops.moe_combine(cache, x, c["gate_w"], Kk, out=res)

            ms = timed(block)
            ms_gemm = timed(lambda: ops.moe_w8a8(x, w, lists, cache=cache, ws=ws, status=st))
            rows = Tn * (Kk + 1)
            iops = 2 * rows * 3 * Hh * Ii
            act = int((lists.counts > 0).sum().item())
            out[f"moe_w8a8_prefill_t{Tn}"] = {
                "config": f"T={Tn}, E=512, top-10 + shared, int8 W8A8, Zipf(1.1) (router, lists, 4 GEMM-chain launches, combine)",
                "ms": ms, "tokens_per_s": Tn / ms * 1e3, "ms_quant_up_hquant_down": ms_gemm,
                "int8_tops_gemm_chain": iops / ms_gemm / 1e9,
                "frac_of_measured_int8_dense": (iops / ms_gemm / 1e9 / out["_int8_peak"]) if out.get("_int8_peak") else None,
                "active_experts": act,
                "blocks": int(lists.nblocks.item()), "weight_bytes_once": act * 3 * Hh * Ii,
                "status": ops.read_status(st)}
            del lists, scr, ws, cache, res
        del c, w
    except Exception as exc:  # noqa: BLE001
        out["moe_w8a8_prefill"] = {"error": repr(exc)[:300]}
    torch.cuda.empty_cache()


def _moe_fp8_block_entry(dev, ops, timed, st, out, hbm, which, sets=3):
    # the fp8 expert block of ONE layer at the one-GPU batch-64 shape (256 rows, 512 experts, top-10 + shared) and
    # at the shape one rank of 8 sees (256 gathered rows, its 64 experts): gate/up and down GEMMs alone, over
    # `sets` weight sets taken in turn so that every launch streams from HBM
    import torch
    from bundles_b200.prepare import quant_fp8_blocks
    for name, En in (("moe_fp8_t256", 512), ("moe_fp8_t256_rank_of_8", 64)):
        try:
            torch.cuda.empty_cache()
            g = torch.Generator(device=dev).manual_seed(1011)

            def fp8(n, rows, cols):
                q = torch.empty(n, rows, cols, dtype=torch.uint8, device=dev)
                sc = torch.empty(n, rows // 128, cols // 128, device=dev)
                for e0 in range(0, n, 64):
                    m = min(64, n - e0)
                    q[e0:e0 + m], sc[e0:e0 + m] = quant_fp8_blocks(torch.randn(m, rows, cols, generator=g, device=dev) * 0.02)
                return q, sc

            ws_ = []
            for _ in range(sets):
                w13, s13 = fp8(En, 2 * I, H)
                w2, s2 = fp8(En, H, I)
                sh13, shs13 = quant_fp8_blocks(torch.randn(2 * I, H, generator=g, device=dev) * 0.02)
                sh2, shs2 = quant_fp8_blocks(torch.randn(H, I, generator=g, device=dev) * 0.02)
                ws_.append(ops.MoeW8A8Weights(w13, s13, w2, s2, sh13, shs13, sh2, shs2))
            x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
            wr = torch.randn(512, H, generator=g, device=dev) * 0.02
            _, ids, wts = ops.router(x, wr, K)
            lists = ops.RoutingLists(T, K, En, 32, dev)
            ops.build_lists(ids, wts, lists, None, e_lo=0)          # the rank's experts are ids 0..En-1
            wsb = ops.moe_fp8_workspace(T, H, I, K, dev)
            cache = torch.zeros(T * (K + 1), H, dtype=torch.bfloat16, device=dev)
            for w in ws_:
                ops.moe_fp8(x, w, lists, cache=cache, ws=wsb, status=st)
            counts = lists.counts.cpu()
            act, rows = int((counts > 0).sum().item()), int(counts.sum().item())
            upb = act * (2 * I * H + 2 * (I // 128) * (H // 128) * 4) + rows * (H + (H // 128) * 4) + rows * I * 2
            dnb = act * (H * I + (H // 128) * (I // 128) * 4) + rows * (I + (I // 128) * 4) + rows * H * 2
            it = [0]

            def stage(mask):
                def run():
                    w = ws_[it[0] % sets]
                    it[0] += 1
                    ops.moe_fp8(x, w, lists, cache=cache, ws=wsb, status=st, stages=mask)
                return run

            ms_up = timed(stage(ops.STAGE_UP), calls=sets)
            ms_dn = timed(stage(ops.STAGE_DOWN), calls=sets)
            ms_all = timed(stage(15), calls=sets)
            out[name] = {"config": f"fp8 expert block, 256 rows, {En} local experts of 512, top-10 + shared (4 launches)",
                         "active_experts": act, "rows": rows, "blocks": int(lists.nblocks.item()), "ms": ms_all,
                         "up": {"ms": ms_up, "algorithmic_bytes": upb, "achieved_gbs": upb / ms_up / 1e6, "frac": upb / ms_up / 1e6 / hbm},
                         "down": {"ms": ms_dn, "algorithmic_bytes": dnb, "achieved_gbs": dnb / ms_dn / 1e6, "frac": dnb / ms_dn / 1e6 / hbm},
                         "bound": "hbm", "peak_source": which, "status": ops.read_status(st)}
            del ws_, wsb, cache, lists
        except Exception as exc:  # noqa: BLE001
            out[name] = {"error": repr(exc)[:300]}
    torch.cuda.empty_cache()


def _moe_w8a8_block_entry(dev, ops, synth, timed, st, out, hbm, which):
    # the int8 W8A8 MoE block at 256 tokens with a Zipf(1.1) router bias (BASELINE configuration 2): the whole block as
    # one CUDA graph, and its two GEMMs alone
    import torch
    from bundles_b200 import moe_block
    try:
        torch.cuda.empty_cache()
        c = synth.moe_w8a8(T=T, H=H, I=I, E=E, device=dev)
        w = ops.MoeW8A8Weights(c["w13"], c["s13"], c["w2"], c["s2"], c["sh13"], c["shs13"], c["sh2"], c["shs2"])
        block = moe_block.MoeBlockW8A8(c["wr"], w, c["gate_w"], K, bias=c["bias"], use_graph=False)
        ms = timed(lambda: block(c["x"]))
        b = block._buffers(T, dev)
        plain = dict(graph=False)
        ms_up = timed(lambda: ops.moe_w8a8(c["x"], w, b["lists"], cache=b["cache"], ws=b["ws"], status=st, stages=ops.STAGE_UP),
                      **plain)
        ms_dn = timed(lambda: ops.moe_w8a8(c["x"], w, b["lists"], cache=b["cache"], ws=b["ws"], status=st, stages=ops.STAGE_DOWN),
                      **plain)
        counts = b["lists"].counts.cpu()
        active, rows = int((counts > 0).sum().item()), int(counts.sum().item())
        up_bytes = active * (2 * I * H + 2 * I * 4) + rows * (H + 4) + rows * I * 2
        dn_bytes = active * (H * I + H * 4) + rows * (I + 12) + rows * H * 2
        out["moe_w8a8_t256"] = {"config": "int8 W8A8 MoE block at decode: T=256, E=512, top-10 + shared, Zipf(1.1) router bias "
                                          "(router, lists, quantise, up, re-quantise, down, combine)",
                                "ms": ms, "tokens_per_s": T / ms * 1e3, "active_experts": active, "rows": rows,
                                "up": {"ms": ms_up, "algorithmic_bytes": up_bytes, "achieved_gbs": up_bytes / ms_up / 1e6,
                                       "frac": up_bytes / ms_up / 1e6 / hbm},
                                "down": {"ms": ms_dn, "algorithmic_bytes": dn_bytes, "achieved_gbs": dn_bytes / ms_dn / 1e6,
                                         "frac": dn_bytes / ms_dn / 1e6 / hbm},
                                "bound": "hbm", "peak_source": which,
                                "status": max(ops.read_status(st), ops.read_status(block.status))}
        del block, c, w
    except Exception as exc:  # noqa: BLE001
        out["moe_w8a8_t256"] = {"error": repr(exc)[:300]}
    torch.cuda.empty_cache()


def _gdn_entry(dev, ops, synth, timed, st, it, out, hbm, which):
    g = {k: v.to(dev) for k, v in synth.gdn().items()}
    states = [g["state"].clone() for _ in range(4)]
    convs = [g["conv_state"].clone() for _ in range(4)]

    gws = ops.gdn_workspace(32, dev)

    def gdn_step():
        i = it[0] % 4
        it[0] += 1
        ops.gdn_verify(g["mixed"], g["z"], g["a"], g["b"], convs[i], g["conv_w"], g["a_log"], g["dt_bias"], states[i],
                       g["accepted"], g["norm_w"], 1e-6, status=st, ws=gws)

    ms = timed(gdn_step, calls=4)
    B = 32
    wrote = int((g["accepted"] > 0).sum().item())
    gbytes = B * 32 * 65536 + wrote * 32 * 65536 + B * 4 * (8192 + 4096 + 64) * 2 + B * 8192 * 3 * 2 * 2 + B * 4 * 4096 * 2
    out["gdn_verify"] = {"config": "B=32 x 4 drafts, 16/32 heads, d=128, accepted~U{0..4}", "ms": ms,
                         "algorithmic_bytes": gbytes, "achieved_gbs": gbytes / ms / 1e6, "bound": "hbm",
                         "frac": gbytes / ms / 1e6 / hbm, "peak_source": which, "status": ops.read_status(st)}
    del states, convs, g
    # the same step on the checkpoint + ring layout: a 128-slot pool (268 MB of checkpoints), four disjoint sets of
    # 32 slots taken in turn so that every launch reads its checkpoints from HBM; nothing is written back but the
    # ring entries, the conv state and the window record
    import torch
    r = {k: v.to(dev) for k, v in synth.gdn_replay(B=32, extra_slots=96).items()}
    perm = torch.randperm(128, device=dev).to(torch.int32)
    sets = [perm[32 * i:32 * i + 32].contiguous() for i in range(4)]

    def replay_step():
        i = it[0] % 4
        it[0] += 1
        ops.gdn_verify_replay(r["mixed"], r["z"], r["a"], r["b"], r["conv_state"], r["conv_w"], r["window"], r["a_log"],
                              r["dt_bias"], r["checkpoint"], r["d_ring"], r["dlo_ring"], r["k_ring"], r["klo_ring"],
                              r["g_ring"], sets[i], sets[i], sets[i], r["write_pos"], r["cache_base"], r["norm_w"], 1e-6,
                              status=st, ws=gws)

    ms = timed(replay_step, calls=4)
    wp = r["write_pos"].clamp(0, 16).float().mean().item()
    rbytes = int(B * 32 * 65536 + B * wp * (32 + 16) * 256 + B * 4 * (8192 + 4096 + 64) * 2 + B * 8192 * (3 + 3 + 6) * 2 +
                 B * 4 * 4096 * 2 + B * 4 * (32 + 16) * 256 * 2)
    out["gdn_verify_replay"] = {"config": "B=32 x 4 drafts on a read-only fp32 checkpoint + 16-entry (d, k, g) ring, "
                                          "write positions ~U{0..16}", "ms": ms, "algorithmic_bytes": rbytes,
                                "achieved_gbs": rbytes / ms / 1e6, "bound": "hbm", "frac": rbytes / ms / 1e6 / hbm,
                                "peak_source": which, "status": ops.read_status(st)}
    del r


def _attn_verify_entry(dev, ops, synth, timed, st, out, hbm, which, name, Bv):
    # attention verify core: 64 requests x 8192 tokens of context (537 MB of e4m3 KV, read once per step), and
    # the 8-request share of one GPU when the batch is sharded over 8 (9 splits per (request, kv head))
    import torch
    if True:
        try:
            av = synth.attn_verify(B=Bv, ctx=8192, device=dev)
            spl = ops._lib.lib().b200_attn_verify_splits(Bv)
            ws_av = torch.empty(ops._lib.lib().b200_attn_verify_workspace_bytes(Bv, spl), dtype=torch.uint8, device=dev)
            out_av = torch.empty(4 * Bv, 4096, dtype=torch.bfloat16, device=dev)

            def av_step():
                ops.attn_verify(av["q"], av["gate"], av["k_new"], av["v_new"], av["kcache"], av["vcache"], av["page_table"],
                                av["seqlens"], splits=spl, out=out_av, ws=ws_av, status=st)

            ms = timed(av_step)
            kvb = Bv * 8192 * 2 * 256 * 2
            out[name] = {"config": f"B={Bv} x 4 drafts, ctx 8192, e4m3 KV in 128-token pages, {spl} split(s); 3 launches "
                                   "(append, core, merge + gate)", "ms": ms, "algorithmic_bytes": kvb,
                         "achieved_gbs": kvb / ms / 1e6, "bound": "hbm", "frac": kvb / ms / 1e6 / hbm,
                         "peak_source": which, "status": ops.read_status(st),
                         "note": "B=8: 67 MB of KV, L2-resident across timed steps" if Bv == 8 else None}
            del av, ws_av, out_av
        except Exception as exc:  # noqa: BLE001
            out[name] = {"error": repr(exc)[:160]}


def _attn_front_entry(dev, ops, synth, timed, st, out, fp8_peak):
    # fused attention projection front: T = 4096
    import torch
    a = {k: v.to(dev) for k, v in synth.attn().items()}
    half = 32
    inv = torch.pow(torch.tensor(1e7, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / 64)
    ang = torch.arange(4096, dtype=torch.float64)[:, None] * inv[None, :]
    cs = torch.cat([ang.cos(), ang.sin()], 1).float().to(dev)
    ms = timed(lambda: ops.attn_front(a["x"], a["w"], a["w_s"], a["q_norm_w"], a["k_norm_w"], a["positions"], cs, 1e-6,
                                      True, status=st))
    fl = 2 * 4096 * 2048 * 9216
    out["attn_front"] = {"config": "T=4096, W [9216,2048] fp8 block-scaled, norm + RoPE fused, e4m3 q/k/v", "ms": ms,
                         "flops": fl, "achieved_tflops": fl / ms / 1e9, "bound": "tensor",
                         "frac_of_measured_fp8_dense": (fl / ms / 1e9 / fp8_peak) if fp8_peak else None,
                         "includes": "activation quantiser launch", "status": ops.read_status(st)}
    del a


def _lmhead_entry(dev, ops, synth, timed, st, it, out, hbm):
    # LM head shard (1/8 of the vocabulary), T = 64, 4 rotating weight copies (156 MB > L2)
    lm = synth.lmhead(T=64, V=19072)
    x = lm["x"].to(dev)
    ws_ = lm["w_s"].to(dev)
    wcopies = [lm["w"].to(dev).clone() for _ in range(4)]
    it[0] = 0

    def lm_step():
        i = it[0] % 4
        it[0] += 1
        ops.lmhead_argmax(x, wcopies[i], ws_, 0, status=st)

    ms = timed(lm_step, calls=4)
    lb = 19072 * 2048 + 149 * 16 * 4 + 64 * 2048 * 2
    out["lmhead_shard_argmax"] = {"config": "T=64, shard 19072 x 2048 fp8 (1/8 of 151936)", "ms": ms,
                                  "algorithmic_bytes": lb, "achieved_gbs": lb / ms / 1e6, "bound": "hbm",
                                  "frac": lb / ms / 1e6 / hbm, "status": ops.read_status(st)}
    del wcopies


def _moe_fp8_router_entry(dev, ops, synth, timed, st, out, hbm, want):
    # fp8 MoE block, T = 16 (single block configuration)
    import torch
    c = {k: (v.to(dev) if v is not None else None) for k, v in synth.moe_fp8(E=512).items()}
    w = ops.MoeW8A8Weights(c["w13"], c["s13"], c["w2"], c["s2"], c["sh13"], c["shs13"], c["sh2"], c["shs2"])
    _, ids, wts = ops.router(c["x"], c["wr"], 10)
    lists = ops.RoutingLists(16, 10, 512, 32, dev)
    ops.build_lists(ids, wts, lists)
    wsb = ops.moe_fp8_workspace(16, 2048, 512, 10, dev)
    cache = torch.zeros(16 * 11, 2048, dtype=torch.bfloat16, device=dev)
    if want("moe_fp8_t16"):
        ms = timed(lambda: ops.moe_fp8(c["x"], w, lists, cache=cache, ws=wsb, status=st))
        act = int((lists.counts > 0).sum().item())
        fb = act * (3 * 2048 * 512 + 768 * 4) + 16 * 2048 * 4
        out["moe_fp8_t16"] = {"config": "T=16, E=512, top-10, fp8 128x128 block scales (4 launches)", "ms": ms,
                          "active_experts": act, "algorithmic_bytes": fb, "achieved_gbs": fb / ms / 1e6,
                          "bound": "hbm", "frac": fb / ms / 1e6 / hbm,
                          "note": "the same weights every step: partly L2-resident when < 126 MB",
                          "status": ops.read_status(st)}
    # router alone at T = 256 and T = 64
    for Tn in (256, 64):
        if not want("router"):
            break
        xr = torch.randn(Tn, 2048, device=dev).to(torch.bfloat16)
        scr = ops.router_scratch(Tn, 2048, 512, dev)
        ms = timed(lambda: ops.router(xr, c["wr"], 10, scratch=scr, want_logits=False))
        out[f"router_t{Tn}"] = {"ms": ms, "flops": 2 * Tn * 512 * 2048, "bytes": 4 * 512 * 2048 + 2 * Tn * 2048}


# ---------------------------------------------------------------------------------------------------------
# the decode + verify step (default workload)
# ---------------------------------------------------------------------------------------------------------
def _cpu_layer_sample(rows=256, seed=1005):
    """Host-side inputs of the CPU baseline: the fp8 weights of ONE Gated-DeltaNet-type layer at full width (router,
    512 experts + shared, in_proj, out_proj) and `rows` activation rows.  Thirty-two distinct experts are drawn and
    repeated sixteen times (CPU time does not depend on the values; the footprint, 1.6 GB, is the real one)."""
    import numpy as np
    import torch
    from bundles_b200.prepare import quant_fp8_blocks
    g = torch.Generator().manual_seed(seed)
    rn = lambda *sh, std=0.02: torch.randn(*sh, generator=g) * std  # noqa: E731
    base = 32
    w13, s13 = quant_fp8_blocks(rn(base, 2 * I, H))
    w2, s2 = quant_fp8_blocks(rn(base, H, I))
    rep = E // base
    d = dict(w13=np.tile(w13.numpy(), (rep, 1, 1)), s13=np.tile(s13.numpy(), (rep, 1, 1)),
             w2=np.tile(w2.numpy(), (rep, 1, 1)), s2=np.tile(s2.numpy(), (rep, 1, 1)))
    for name, shape in (("sh13", (2 * I, H)), ("sh2", (H, I)), ("in", (12416, H)), ("out", (H, 4096))):
        q, sc = quant_fp8_blocks(rn(*shape))
        d[name], d[name + "_s"] = q.numpy(), sc.numpy()
    d["wr"] = rn(E, H).numpy()
    bits = lambda t: t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    d["x"] = bits(torch.randn(rows, H, generator=g))
    d["core"] = torch.randn(rows, 4096, generator=g).to(torch.bfloat16).float().numpy()
    d["gate_w"] = bits(rn(H))
    return d


def _cpu_layer_seconds(d):
    """One pass of the sample: in_proj GEMM, out_proj GEMM, router, fp8 expert block + combine (C, OpenMP)."""
    import numpy as np
    from oracle import clib
    t0 = time.perf_counter()
    xf = (d["x"].astype(np.uint32) << 16).view(np.float32)
    xq, xs = clib.quant_fp8_groups(xf)
    clib.gemm_fp8_blocks(xq, xs, d["in"][:12352], d["in_s"])
    cq, cs = clib.quant_fp8_groups(d["core"])
    clib.gemm_fp8_blocks(cq, cs, d["out"], d["out_s"])
    logits = clib.gate_logits(d["x"], d["wr"], None)
    ids, wts = clib.topk(logits, K)
    clib.moe_fp8(d["x"], ids, wts, d["w13"], d["s13"], d["w2"], d["s2"], d["sh13"], d["sh13_s"], d["sh2"], d["sh2_s"],
                 d["gate_w"])
    return time.perf_counter() - t0


CPU_SAMPLE = ("one layer of the 48 at all 256 rows: in_proj + out_proj fp8 GEMMs, router, fp8 expert block + combine "
              "(C + OpenMP restatement); the step is taken as 48 x this, the GDN recurrence, attention core and LM head "
              "are left out, so the CPU figure is an upper bound on its rate")


def cpu_step_baseline(repeats=2):
    from oracle import clib
    cores = clib.use_all_cores()
    d = _cpu_layer_sample(4 * BATCH)
    best = min(_cpu_layer_seconds(d) for _ in range(repeats))
    return {"value": 4 * BATCH / (LAYERS * best), "unit": "tokens/s", "cores": cores, "kind": "port", "sample": CPU_SAMPLE,
            "seconds_per_layer": best}


def run_step_reference(args, rank, world):
    """`--impl reference` for the step workload: the CPU restatement on the host cores, one sample per step."""
    if rank != 0:
        return
    from oracle import clib
    cores = clib.use_all_cores()
    d = _cpu_layer_sample(4 * BATCH)
    times = []
    for i in range(args.warmup + args.steps):
        dt = _cpu_layer_seconds(d)
        if i >= args.warmup:
            times.append(dt)
    per_layer = sum(times) / len(times)
    ms = 1000.0 * per_layer * LAYERS
    val = 4 * BATCH / (ms / 1000.0)
    line = {"impl": "reference", "metric": STEP_METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8 e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": STEP_WORKLOAD, "l2": "not applicable (CPU)"},
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": CPU_SAMPLE,
                             "seconds_per_layer": per_layer},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


def _ep_check(dev, ep, world, rank):
    """Before anything is timed: a 4-layer stack (3 GDN + 1 attention layer) at full width (batch 64, 512 experts,
    full vocabulary, 512 tokens of context) run in the expert-parallel form, against the one-GPU form of the same
    stack on rank 0.  Tokens and final hidden rows must be equal bit for bit.  On one GPU the expert-parallel form
    runs as two virtual ranks."""
    import torch
    import torch.distributed as dist
    from bundles_b200 import decode_step, ops, parallel
    kw = dict(layers=4, B=BATCH, ctx=512, vocab=VOCAB, experts=E, seed=77, device=dev, attn_splits=2)   # same split count in both forms
    g = torch.Generator(device=dev).manual_seed(78)
    x = torch.randn(4 * BATCH, H, generator=g, device=dev).to(torch.bfloat16)
    res = {"form": None, "tokens_equal": None, "hidden_equal": None, "status": None}
    if world == 1:
        single = decode_step.DecodeStep(**kw)
        want = single.step(x)
        vg = parallel.VirtualEpGroup(2, dev)
        ranks = [decode_step.DecodeStep(ep=vg.view(r), **kw) for r in range(2)]
        Tl = ranks[0].T
        got = decode_step.step_virtual(ranks, [x[r * Tl:(r + 1) * Tl].contiguous() for r in range(2)])
        torch.cuda.synchronize()
        hid = torch.cat([r.final_hidden for r in ranks])
        res.update(form="2 virtual ranks on one GPU", tokens_equal=bool(torch.equal(got[0], want) and torch.equal(got[1], want)),
                   hidden_equal=bool(torch.equal(hid, single.final_hidden)),
                   status=max(ops.read_status(single.status), *[ops.read_status(r.status) for r in ranks]))
        del single, ranks, vg
    else:
        part = decode_step.DecodeStep(ep=ep, **kw)
        Tl = part.T
        got = part.step(x[rank * Tl:(rank + 1) * Tl].contiguous())
        torch.cuda.synchronize()
        hid = [torch.empty_like(part.final_hidden) for _ in range(world)]
        dist.all_gather(hid, part.final_hidden.contiguous())
        flag = torch.ones(1, device=dev)
        st = ops.read_status(part.status)
        if rank == 0:
            single = decode_step.DecodeStep(**kw)
            want = single.step(x)
            torch.cuda.synchronize()
            res.update(form=f"{world} ranks against the one-GPU step on rank 0", tokens_equal=bool(torch.equal(got, want)),
                       hidden_equal=bool(torch.equal(torch.cat(hid), single.final_hidden)))
            st = max(st, ops.read_status(single.status))
            del single
        sts = torch.tensor([st], device=dev)
        dist.all_reduce(sts, op=dist.ReduceOp.MAX)
        res["status"] = int(sts.item())
        del part, flag
    torch.cuda.empty_cache()
    res["ok"] = bool(res["tokens_equal"] and res["hidden_equal"] and res["status"] == 0) if (world == 1 or rank == 0) else None
    return res


def run_step_virtual(args, dev):
    """Diagnostic (one GPU): the N ranks of the expert-parallel step as virtual ranks in one process, their launches
    in lockstep on one stream inside one CUDA graph.  The time of one replay divided by N is what one rank of N spends
    in its own kernels per step (no NVLink latency, no barrier wait); `ncu` on this command lists the rank-shaped
    kernels.  Prints one JSON line that is NOT the benchmark's headline."""
    import torch
    from bundles_b200 import decode_step, ops, parallel
    n = args.virtual_ranks
    vg = parallel.VirtualEpGroup(n, dev)
    steps = [decode_step.DecodeStep(layers=args.layers, B=BATCH, ctx=CTX, vocab=VOCAB, experts=E, seed=1005, device=dev,
                                    ep=vg.view(r)) for r in range(n)]
    Tl = steps[0].T
    g = torch.Generator(device=dev).manual_seed(9000)
    x_all = torch.randn(steps[0].T_all, H, generator=g, device=dev).to(torch.bfloat16)
    xs = [x_all[r * Tl:(r + 1) * Tl].contiguous() for r in range(n)]
    decode_step.step_virtual(steps, xs)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        decode_step.step_virtual(steps, xs)
    for _ in range(args.warmup):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    emit({"diagnostic": "virtual ranks on one GPU", "virtual_ranks": n, "layers": args.layers,
          "ms_all_ranks": ms, "ms_per_rank_step": ms / n, "us_per_rank_layer": ms / n * 1000.0 / args.layers,
          "launches_per_rank_step": steps[0].launches, "status": max(ops.read_status(s.status) for s in steps)})


def run_step(args, rank, world, local, dev):
    """The default workload on `world` GPUs (one process each)."""
    import torch
    import torch.distributed as dist
    from bundles_b200 import decode_step, ops, parallel
    if world == 1 and args.virtual_ranks > 1:
        run_step_virtual(args, dev)
        return
    ep = parallel.EpGroup(device=dev) if world > 1 else None
    check = None if args.no_ep_check else _ep_check(dev, ep, world, rank)
    t_build = time.perf_counter()
    step = decode_step.DecodeStep(layers=args.layers, B=BATCH, ctx=CTX, vocab=VOCAB, experts=E, seed=1005, device=dev, ep=ep)
    torch.cuda.synchronize()
    t_build = time.perf_counter() - t_build
    Tl, Ta = step.T, step.T_all
    g = torch.Generator(device=dev).manual_seed(9000)
    x_all = torch.randn(Ta, H, generator=g, device=dev).to(torch.bfloat16)
    x_dev = x_all[rank * Tl:(rank + 1) * Tl].contiguous()
    x_host = x_dev.cpu().pin_memory()
    n_tok = Ta if world > 1 else Tl
    tok_host = torch.empty(n_tok, dtype=torch.int32).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # one eager step (one-time set-up inside the operators), then the whole step as one CUDA graph
    step.step(x_dev)
    barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        tokens = step.step(x_dev)
    barrier()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step = timed(graph.replay, args.steps, args.warmup)

    def e2e_step():
        # the user's call: this rank's embedded rows from pinned host memory in, the step, the tokens out to pinned
        # host memory, all on the current stream
        x_dev.copy_(x_host, non_blocking=True)
        graph.replay()
        tok_host.copy_(tokens, non_blocking=True)

    ms_e2e = timed(e2e_step, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None

    # the dominant kernel alone: the fp8 gate/up expert GEMM (+ SwiGLU) of every layer in turn, each over its own
    # weights (so that every launch streams from HBM), with the routing lists the last layer left behind
    lists = step.lists
    src = step.x_all if world > 1 else step.final_hidden

    def up_all_layers():
        for L in step.layers:   # this stage writes h into the workspace only; `cache` is not touched
            ops.moe_fp8(src, L["w"], lists, cache=step.cache, ws=step.moe_ws, status=step.status, stages=ops.STAGE_UP)

    ms_up = timed(up_all_layers, max(2, args.steps // 4), 1) / len(step.layers)
    counts = lists.counts.cpu()
    active = int((counts > 0).sum().item())
    rows = int(counts.sum().item())
    up_bytes = active * (2 * I * H + 2 * (I // 128) * (H // 128) * 4) + rows * (H + (H // 128) * 4) + rows * I * 2
    status = torch.tensor([ops.read_status(step.status)], device=dev)
    if world > 1:
        dist.all_reduce(status, op=dist.ReduceOp.MAX)
    peak, which = peaks()
    mem_gb = round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 1)
    launches = step.launches
    if rank != 0:
        del graph
        if world > 1:
            dist.destroy_process_group()
        return
    achieved = up_bytes / (ms_up * 1e-3) / 1e9
    exchange = ("1 GPU" if world == 1 else
                f"{world} GPUs: {BATCH // world} sequences, {E // world} experts and 1/{world} of the vocabulary per rank; rows "
                "and routing dispatched by peer stores into every rank's symmetric-memory buffers, weighted rows stored by "
                "the down-GEMM epilogue into the home rank's cache, (max, argmax) pairs gathered by peer stores; the library's "
                "bounded barrier kernel between the phases (no NCCL call in the step)")
    line = {
        "metric": STEP_METRIC, "value": Ta / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "us_per_layer": ms_step * 1000.0 / len(step.layers),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8 e4m3 (fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": STEP_WORKLOAD, "layers": len(step.layers), "batch": BATCH, "rows_per_step": Ta,
                   "parallelism": exchange,
                   "l2": f"every layer streams its own expert weights ({active} experts hit on this rank in the last layer, "
                         f"{up_bytes / 1e6:.0f} MB for the gate/up GEMM alone), {len(step.layers)} layers per step: far more than "
                         "the 126 MB L2; no flush"},
        "e2e": {"value": Ta / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": Tl * H * 2,
                "d2h_bytes_per_step": n_tok * 4, "ms_per_step": ms_e2e},
        "gpu_launches": launches * args.steps,
        "roofline": {"kernel": "moe_gemm_f8_kernel<UP> (fp8 gate/up expert GEMM + SwiGLU)", "bound": "hbm", "achieved": achieved,
                     "peak": peak, "peak_source": which, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": F8_UP_TRAFFIC_RATIO * up_bytes if F8_UP_TRAFFIC_RATIO else None,
                     "traffic_source": "DRAM read + write of one launch of this kernel under ncu on the same case (one layer, 256 "
                                       "rows x 512 experts; profiles/moe_fp8_up_down_t256.md), scaled by this launch's "
                                       "algorithmic bytes",
                     "algorithmic_bytes": up_bytes, "ms": ms_up, "active_experts": active, "rows": rows},
        "clocks": clocks, "device_status": int(status.item()), "ep_check": check,
        "launches_per_step": launches, "device_memory_gb": mem_gb, "build_seconds": round(t_build, 1),
    }
    del graph, step
    torch.cuda.empty_cache()
    if world == 1 and not args.no_kernels:
        try:
            line["kernels"] = other_kernels(dev, args.steps, args.warmup)
        except Exception as exc:  # noqa: BLE001  (the headline line must still be printed)
            line["kernels"] = {"error": repr(exc)[:300]}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_step_baseline()
    emit(line)
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (read + write) of one launch of moe_gemm_f8_kernel<UP> divided by its algorithmic bytes, from the ncu
# capture summarised in profiles/moe_fp8_up_down_t256.md (1.1077 GB read + 12.5 MB written for 1.0786 GB)
F8_UP_TRAFFIC_RATIO = 1.032



def run_expert_parallel(args, rank, world, dev, cfg):
    """N > 1: experts split over the ranks (512 / N each), every rank brings its own 256 tokens (weak
    scaling: rows per rank stay ~2560 routed + 256 shared).  All ranks draw the SAME layer (seed) and keep
    their slice of it."""
    import torch
    import torch.distributed as dist
    from bundles_b200 import ops, parallel, synth
    full = synth.moe_w8a8(seed=synth.SEEDS["moe_w8a8"], T=T, H=H, I=I, E=E, device=dev)
    e_lo, e_n = parallel.expert_range(E, rank, world)
    w_local = ops.MoeW8A8Weights(full["w13"][e_lo:e_lo + e_n].clone(), full["s13"][e_lo:e_lo + e_n].clone(),
                                 full["w2"][e_lo:e_lo + e_n].clone(), full["s2"][e_lo:e_lo + e_n].clone(),
                                 full["sh13"], full["shs13"], full["sh2"], full["shs2"])
    wr, gate_w, bias = full["wr"], full["gate_w"], full["bias"]
    del full
    torch.cuda.empty_cache()
    backend = parallel.GpuMoeBackend(wr, w_local, gate_w, K, e_lo, bias=bias)
    exchange = ("tokens and routing dispatched by peer stores into every rank's symmetric-memory buffers + barrier; "
                "peer stores from the down-GEMM epilogue into the home rank's cache + barrier (no NCCL call in the step)")
    try:
        ep = parallel.FusedExpertParallelMoe(backend, K, H, T)
    except Exception as exc:  # noqa: BLE001  (symmetric memory unavailable: NCCL reduce-scatter baseline)
        ep = parallel.ExpertParallelMoe(backend, K, H)
        exchange = ("all-gather of tokens and routing, reduce-scatter of the weighted expert rows (NCCL); "
                    f"symmetric memory unavailable: {repr(exc)[:80]}")
    g = torch.Generator(device=dev).manual_seed(7000 + rank)
    x_dev = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    x_host = x_dev.cpu().pin_memory()
    out_host = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()

    def timed(fn, tail=None):
        for _ in range(args.warmup):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        if tail is not None:
            tail()  # copies the steps left on other streams join the timed stream before the closing event
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    ms_step = timed(lambda: ep(x_dev))

    if hasattr(ep, "forward_host"):
        ms_e2e = timed(lambda: ep.forward_host(x_host, out_host), tail=ep.join_host)
    else:
        def e2e_step():
            out_host.copy_(ep(x_host.to(dev, non_blocking=True)), non_blocking=True)

        ms_e2e = timed(e2e_step)
    clocks = sampler.stop() if rank == 0 else None
    status = torch.tensor([ops.read_status(backend.status)], device=dev)
    dist.all_reduce(status, op=dist.ReduceOp.MAX)
    if rank == 0:
        line = {"metric": METRIC, "value": world * T / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": {"workload": WORKLOAD, "tokens_per_gpu": T,
                           "parallelism": f"ep{world}: {E // world} experts per rank; " + exchange,
                           "l2": "weights streamed per step exceed the 126 MB L2; no flush"},
                "e2e": {"value": world * T / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2,
                        "d2h_bytes_per_step": T * H * 2, "ms_per_step": ms_e2e},
                "gpu_launches": getattr(ep, "launches_per_call", backend.launches_per_call) * args.steps, "clocks": clocks,
                "device_status": int(status.item())}
        emit(line)
    if hasattr(ep, "close"):
        ep.close()      # the captured graph holds NCCL kernels: release it before the communicator
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="step", choices=["step", "moe_int8"],
                    help="step: the 48-layer decode+verify step at batch 64 (default); moe_int8: the int8 W8A8 MoE block at 256 tokens")
    ap.add_argument("--layers", type=int, default=LAYERS, help="layers of the step workload (48; fewer only for quick checks)")
    ap.add_argument("--virtual-ranks", type=int, default=0,
                    help="one GPU only, diagnostic: run the N-rank expert-parallel step as N virtual ranks and print its time")
    ap.add_argument("--no-ep-check", action="store_true", help="skip the expert-parallel == one-GPU check before the timed runs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel measurements of the other rows")
    ap.add_argument("--parallel", default="ep", choices=["ep", "replicas"],
                    help="N > 1: expert-parallel (experts split over ranks) or independent replicas")
    ap.add_argument("--only-kernel", default=None,
                    choices=["gdn_verify", "attn_verify", "attn_front", "lmhead_shard_argmax", "moe_fp8_t16", "router",
                             "moe_w8a8_prefill", "moe_w8a8_t256", "moe_fp8_t256"],
                    help="run one entry of `kernels` alone with plain launches (a small target for an ncu capture) and exit")
    args = ap.parse_args()
    quiet_stdout()
    if args.only_kernel:
        import torch
        torch.cuda.set_device(0)
        emit({"kernels": other_kernels(torch.device("cuda", 0), min(args.steps, 3), 1, only=args.only_kernel)})
        return
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        (run_step_reference if args.workload == "step" else run_reference)(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from bundles_b200 import moe_block, ops, synth

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.workload == "step":
        run_step(args, rank, world, local, dev)
        return

    # weights: the CPU random stream at rank 0 of a 1-GPU run (so the CPU baseline sees the same bytes),
    # a CUDA stream elsewhere (every rank holds a full replica of the layer and its own 256 tokens)
    need_host = (world == 1 and not args.no_cpu_baseline)
    if need_host:
        cfg_host = synth.moe_w8a8(T=T, H=H, I=I, E=E)
        cfg = {k: (v.to(dev) if v is not None else None) for k, v in cfg_host.items()}
    else:
        cfg_host = None
        cfg = synth.moe_w8a8(seed=synth.SEEDS["moe_w8a8"] + rank, T=T, H=H, I=I, E=E, device=dev)
    w = ops.MoeW8A8Weights(cfg["w13"], cfg["s13"], cfg["w2"], cfg["s2"], cfg["sh13"], cfg["shs13"], cfg["sh2"],
                           cfg["shs2"])
    if world > 1 and args.parallel == "ep":
        run_expert_parallel(args, rank, world, dev, cfg)
        return
    block = moe_block.MoeBlockW8A8(cfg["wr"], w, cfg["gate_w"], K, bias=cfg["bias"])
    x_dev = cfg["x"]
    x_host = x_dev.cpu().pin_memory()
    out_host = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    x_stage = torch.empty_like(x_dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, tail=None):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if tail is not None:
            tail()  # work the steps left on other streams joins the timed stream before the closing event
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step = timed(lambda: block(x_dev), args.steps, args.warmup)

    def e2e_step():
        # the user's call: host activations in, host result out; consecutive calls overlap their copies with the
        # kernels of their neighbours (two device buffer sets), every call moves its own input and output
        block.forward_host(x_host, out_host)

    ms_e2e = timed(e2e_step, args.steps, args.warmup, tail=block.join_host)
    block.synchronize_host()

    # the dominant kernel alone: gate/up GEMM (+ SwiGLU) over the same routing
    block._forward_eager(x_dev)
    b = block._buffers(T, dev)
    ms_up = timed(lambda: ops.moe_w8a8(x_dev, w, b["lists"], cache=b["cache"], ws=b["ws"], status=block.status,
                                       stages=ops.STAGE_UP), args.steps, args.warmup)
    ms_down = timed(lambda: ops.moe_w8a8(x_dev, w, b["lists"], cache=b["cache"], ws=b["ws"], status=block.status,
                                         stages=ops.STAGE_DOWN), args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    status = ops.read_status(block.status)

    counts = b["lists"].counts.cpu()
    active = int((counts > 0).sum().item())            # experts whose weights are streamed (shared included)
    rows = int(counts.sum().item())
    up_bytes = active * (2 * I * H + 2 * I * 4) + rows * (H + 4) + rows * I * 2
    down_bytes = active * (H * I + H * 4) + rows * (I + 4 + 8) + rows * H * 2
    peak, which = peaks()
    achieved = up_bytes / (ms_up * 1e-3) / 1e9
    # DRAM bytes of one launch of this kernel from an ncu capture of the same workload
    # (summary kept under profiles/): read + write = 1.005 x the algorithmic bytes of that launch;
    # traffic grows with the experts hit, so it is scaled by this launch's algorithmic bytes.
    traffic = 1.005 * up_bytes

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    line = {
        "metric": METRIC, "value": world * T / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_gpu": T,
                   "parallelism": "1 GPU" if world == 1 else f"{world} replicas, no data-path collective",
                   "l2": f"{active} experts hit: {(up_bytes + down_bytes) / 1e6:.0f} MB of weights and rows streamed per "
                         "step, more than the 126 MB L2; no flush"},
        "e2e": {"value": world * T / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2,
                "d2h_bytes_per_step": T * H * 2, "ms_per_step": ms_e2e},
        "gpu_launches": block.launches_per_call * args.steps,
        "roofline": {"kernel": "moe_gemm_i8_kernel<up> (gate/up GEMM + SwiGLU)", "bound": "hbm",
                     "achieved": achieved, "peak": peak, "peak_source": which, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": traffic, "algorithmic_bytes": up_bytes, "ms": ms_up,
                     "active_experts": active, "rows": rows,
                     "down_kernel": {"ms": ms_down, "algorithmic_bytes": down_bytes,
                                     "achieved": down_bytes / (ms_down * 1e-3) / 1e9}},
        "clocks": clocks, "device_status": status,
    }
    if world == 1 and not args.no_kernels:
        del block, w, cfg
        torch.cuda.empty_cache()
        try:
            line["kernels"] = other_kernels(dev, args.steps, args.warmup)
        except Exception as exc:  # noqa: BLE001  (the headline line must still be printed)
            line["kernels"] = {"error": repr(exc)[:300]}
    if cfg_host is not None:
        dt, cores = cpu_baseline(cfg_host)
        line["cpu_baseline"] = {"value": T / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
                                "sample": "whole workload (256 tokens, 2816 expert rows), best of 2", "seconds": dt}
    emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
