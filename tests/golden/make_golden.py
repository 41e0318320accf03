"""Generates tests/golden/reference_vectors.npz by RUNNING the reference bundle's CPU-runnable code.

Run once, in a container that has the reference checked out (it does not travel to the GPU box):

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference/qwen36_nodes_kb34

What runs is the reference's own code, unmodified, imported from its directory: its torch
quantisers and its Triton kernels under the Triton CPU interpreter, at the reference's own
shapes (256 experts, top-8).  The compiled CUDA units those modules import at load time are
replaced by empty stub modules (none of the functions called here touches them); the one
third-party import of gdn.py (an SGLang decorator) is stubbed by an identity decorator.
Only inputs and outputs are stored; no reference source is copied.
"""
from __future__ import annotations

import os
import sys
import types

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch


class _Stub(types.ModuleType):
    def __getattr__(self, item):  # any compiled entry point the modules look up at import time
        if item.startswith("__"):
            raise AttributeError(item)
        return None


def _stub(name, **attrs):
    m = _Stub(name)
    for k, v in attrs.items():
        setattr(m, k, v)
    sys.modules[name] = m
    return m


def main(ref_dir: str, out_path: str) -> None:
    sys.path.insert(0, ref_dir)
    for n in ("qk_route", "qk_moe_up16", "qk_proj_decode", "qk_lt", "qk_conv_gate", "qk_inproj",
              "qk_moe_prefill_i8", "qk_moe_prefill", "qk_moe_decode", "qk_gated_norm"):
        _stub(n)
    _stub("qk_moe_dn16", MAX_ROWS=128)
    for n in ("sglang", "sglang.srt", "sglang.srt.model_executor",
              "sglang.srt.model_executor.runner_backend_utils"):
        _stub(n)
    _stub("sglang.srt.model_executor.runner_backend_utils.breakable_cuda_graph",
          eager_on_graph=lambda *a, **k: (lambda f: f))

    g = torch.Generator().manual_seed(7001)
    out = {}

    # -- per-token int8 activation quantiser + W8A8 GEMM epilogue (qwen36_lmhead8/w8a8.py) -------
    from qwen36_lmhead8 import w8a8, lmhead8
    x = torch.randn(12, 512, generator=g).to(torch.bfloat16)
    x[3] = 0  # all-zero row: scale 0, divide by 1
    xq, xs = w8a8.quantize_act(x)
    out["act_x_bf16bits"] = x.view(torch.int16).numpy().copy()
    out["act_q"] = xq.numpy().copy()
    out["act_s"] = xs.numpy().copy()
    w = (torch.randn(96, 512, generator=g) * 0.02)
    wq, ws = lmhead8.quantize_rows_torch(w)
    out["w_f32"] = w.numpy().copy()
    out["w_q"] = wq.numpy().copy()
    out["w_s"] = ws.numpy().copy()
    y = torch.empty(12, 96, dtype=torch.bfloat16)
    w8a8.w8a8_gemm(xq, xs, wq, ws, y, config=(32, 16, 64, 4, 2))
    out["w8a8_y_bf16bits"] = y.view(torch.int16).numpy().copy()

    # -- softmax / top-8 / renormalise (qwen36_layer/i8x_decode.py `_top8` via i8x_dec_topk) ------
    from qwen36_layer import i8x_decode as dec
    T, E, SK = 24, 256, dec.GATE_SPLIT_K
    part = torch.randn(SK, dec.MAX_T, E, generator=g) * 0.6
    # force exact ties after the bf16 rounding, and a -0 / +0 pair
    part[:, 1, 17] = part[:, 1, 5]
    part[:, 1, 200] = part[:, 1, 5]
    part[:, 2, :] = 0.0
    part[0, 2, 9] = -0.0
    ids = torch.zeros(dec.MAX_T * dec.TOPK, dtype=torch.int32)
    wts = torch.zeros(dec.MAX_T * dec.TOPK, dtype=torch.float32)
    dec.i8x_dec_topk[(T,)](part, ids, wts, E=E, SPLIT_K=SK, TOPK=dec.TOPK, MAX_T=dec.MAX_T, PDL=False)
    logits = torch.zeros(T, E)
    for s in range(SK):  # the kernel's own order: ((0 + p0) + p1) + ...
        logits = logits + part[s, :T]
    out["topk_logits"] = logits.numpy().copy()
    out["topk_ids"] = ids[:T * dec.TOPK].view(T, dec.TOPK).numpy().copy()
    out["topk_wts"] = wts[:T * dec.TOPK].view(T, dec.TOPK).numpy().copy()

    # -- routing lists (i8x_dec_lists) ------------------------------------------------------------
    M = T
    pos = torch.ones(M, dtype=torch.int64)
    pos[4] = 0  # a graph-padding row
    counts = torch.zeros(E, dtype=torch.int32)
    tokens = torch.zeros(E * dec.MAX_T, dtype=torch.int32)
    slots = torch.zeros(E * dec.MAX_T, dtype=torch.int32)
    nblocks = torch.zeros(1, dtype=torch.int32)
    nb_max = E + dec.MAX_T * dec.TOPK // dec.BLOCK_T + dec.MAX_T // dec.BLOCK_T
    bexp = torch.zeros(nb_max, dtype=torch.int32)
    bt0 = torch.zeros(nb_max, dtype=torch.int32)
    dec.i8x_dec_lists[(E + 1,)](ids, pos, counts, tokens, slots, nblocks, bexp, bt0, M, E=E, TOPK=dec.TOPK,
                                MAX_T=dec.MAX_T, BLOCK=4096, BLOCK_T=dec.BLOCK_T, PDL=False)
    out["lists_pos"] = pos.numpy().copy()
    out["lists_counts"] = counts.numpy().copy()
    out["lists_tokens"] = tokens.view(E, dec.MAX_T).numpy().copy()
    out["lists_slots"] = slots.view(E, dec.MAX_T).numpy().copy()

    # -- combine with the sigmoid shared-expert gate (i8x_dec_combine) ----------------------------
    H = 2048
    Mc = 6
    cache = (torch.randn(Mc * (dec.TOPK + 1), H, generator=g) * 0.3).to(torch.bfloat16)
    xc = torch.randn(Mc, H, generator=g).to(torch.bfloat16)
    gw = (torch.randn(H, generator=g) * 0.02).to(torch.bfloat16)
    posc = torch.ones(Mc, dtype=torch.int64)
    posc[2] = 0
    outc = torch.empty(Mc, H, dtype=torch.bfloat16)
    cnt2 = torch.ones(E, dtype=torch.int32)
    nb2 = torch.ones(1, dtype=torch.int32)
    dec.i8x_dec_combine[(Mc, H // 256)](cache, xc, gw, posc, outc, cnt2, nb2, Mc, E=E, TOPK=dec.TOPK, H=H,
                                        BLOCK_H=256, PDL=False)
    out["comb_cache_bf16bits"] = cache.view(torch.int16).numpy().copy()
    out["comb_x_bf16bits"] = xc.view(torch.int16).numpy().copy()
    out["comb_gw_bf16bits"] = gw.view(torch.int16).numpy().copy()
    out["comb_pos"] = posc.numpy().copy()
    out["comb_out_bf16bits"] = outc.view(torch.int16).numpy().copy()

    # -- SwiGLU rounding points (`_swiglu_store`) through the shared-expert branch of i8x_dec_up ---
    # (bf16 weights, fp32 MMA under the interpreter: INTERPRETER / F32 switch of the reference)
    I, Hs = 64, 256
    Ms = 5
    xs_ = torch.randn(Ms, Hs, generator=g).to(torch.bfloat16)
    s13 = (torch.randn(2 * I, Hs, generator=g) * 0.06).to(torch.bfloat16)
    hbuf = torch.zeros(Ms * (dec.TOPK + 1), I, dtype=torch.bfloat16)
    cnt3 = torch.zeros(E, dtype=torch.int32)
    nb3 = torch.tensor([1], dtype=torch.int32)
    bexp3 = torch.tensor([E], dtype=torch.int32)
    bt03 = torch.tensor([0], dtype=torch.int32)
    dummy8 = torch.zeros(16, dtype=torch.int8)
    dummy16 = torch.zeros(16, dtype=torch.float16)
    BN = 32
    dec.i8x_dec_up[(I // BN,)](xs_, dummy8, dummy16, s13, hbuf, cnt3, tokens, slots, nb3, bexp3, bt03, Ms, H=Hs, I=I,
                               E=E, EB=0, C13=0, MAX_T=dec.MAX_T, TOPK=dec.TOPK, GROUP=128, BLOCK_T=16, BLOCK_N=BN,
                               BLOCK_K=128, GROUP_M=1, G128=True, SHARED_DONE=False, EARLY_SH=False, EVICT="",
                               PDL=False, F32=True, PRMT=False)
    out["sw_x_bf16bits"] = xs_.view(torch.int16).numpy().copy()
    out["sw_w13_bf16bits"] = s13.view(torch.int16).numpy().copy()
    out["sw_h_bf16bits"] = hbuf[Ms * dec.TOPK:Ms * dec.TOPK + Ms].view(torch.int16).numpy().copy()

    # -- the reference's expert-weight quantiser (i8x_kernels._quant_row_kernel) -------------------
    try:
        _stub("qwen36_layer.lt", linear=None)
        from qwen36_layer import i8x_kernels as ik
        wch = torch.randn(40, 256, generator=g) * 0.02
        qch = torch.empty(40, 256, dtype=torch.int8)
        cch = torch.empty(40, 2, dtype=torch.float16)
        ik.quantize_channel(wch, qch, cch)
        out["ch_w"] = wch.numpy().copy()
        out["ch_q"] = qch.numpy().copy()
        out["ch_c"] = cch.numpy().copy()
    except Exception as exc:  # recorded, not fatal: the target format does not use this quantiser
        print("quantize_channel not generated:", repr(exc))

    # -- row-wise fp8 quantiser (fp8._rowwise_fp8) --------------------------------------------------
    try:
        _stub("qwen36_layer.i8x_tail")
        from qwen36_layer import fp8 as rfp8
        xf = torch.randn(9, 256, generator=g).to(torch.bfloat16)
        yf = torch.empty(9, 256, dtype=torch.float8_e4m3fn)
        sf = torch.empty(9, 1, dtype=torch.float32)
        rfp8._rowwise_fp8[(9,)](xf, yf, sf, 9, K=256, BLOCK=128)
        out["fp8_x_bf16bits"] = xf.view(torch.int16).numpy().copy()
        out["fp8_codes"] = yf.view(torch.uint8).numpy().copy()
        out["fp8_scale"] = sf.view(-1).numpy().copy()
    except Exception as exc:
        print("rowwise fp8 not generated:", repr(exc))

    # -- GDN conv + gates (gdn._conv_split_gate_kernel), one 4-token sequence per request ----------
    try:
        from qwen36_layer import gdn as rgdn
        B, NT, D = 3, 4, 8192
        xm = torch.randn(B * NT, D, generator=g).to(torch.bfloat16)
        cw = (torch.randn(D, 4, generator=g) * 0.5).to(torch.bfloat16)
        cs = torch.randn(B, D, 3, generator=g).to(torch.bfloat16)
        cs_in = cs.clone()
        qsl = torch.arange(0, B * NT + 1, NT, dtype=torch.int32)
        idx = torch.arange(B, dtype=torch.int32)
        hinit = torch.ones(B, dtype=torch.int32)
        av = torch.randn(B * NT, 32, generator=g).to(torch.bfloat16)
        bv = torch.randn(B * NT, 32, generator=g).to(torch.bfloat16)
        alog = torch.rand(32, generator=g) * float(np.log(16.0))
        dtb = torch.randn(32, generator=g)
        qo = torch.empty(B * NT, 16, 128, dtype=torch.bfloat16)
        ko = torch.empty(B * NT, 16, 128, dtype=torch.bfloat16)
        vo = torch.empty(B * NT, 32, 128, dtype=torch.bfloat16)
        go = torch.empty(B * NT, 32, dtype=torch.float32)
        bo = torch.empty(B * NT, 32, dtype=torch.float32)
        grid = (D // rgdn.BLOCK_C, 1, B)
        rgdn._conv_split_gate_kernel[grid](xm, cw, cs, qsl, idx, hinit, av, bv, alog, dtb, qo, ko, vo, go, bo,
                                           D=D, HEAD=128, NQ=16, NK=16, NV=32, BLOCK_T=rgdn.BLOCK_T,
                                           BLOCK_C=rgdn.BLOCK_C, L2NORM=False, ALPHA=False, EPS=1e-6)
        out["gdn_x_bf16bits"] = xm.view(torch.int16).numpy().copy()
        out["gdn_cw_bf16bits"] = cw.view(torch.int16).numpy().copy()
        out["gdn_cs_in_bf16bits"] = cs_in.view(torch.int16).numpy().copy()
        out["gdn_cs_out_bf16bits"] = cs.view(torch.int16).numpy().copy()
        out["gdn_a_bf16bits"] = av.view(torch.int16).numpy().copy()
        out["gdn_b_bf16bits"] = bv.view(torch.int16).numpy().copy()
        out["gdn_alog"] = alog.numpy().copy()
        out["gdn_dtb"] = dtb.numpy().copy()
        out["gdn_q_bf16bits"] = qo.view(torch.int16).numpy().copy()
        out["gdn_k_bf16bits"] = ko.view(torch.int16).numpy().copy()
        out["gdn_v_bf16bits"] = vo.view(torch.int16).numpy().copy()
        out["gdn_g"] = go.numpy().copy()
    except Exception as exc:
        print("gdn conv/gates not generated:", repr(exc))

    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    here = os.path.dirname(os.path.abspath(__file__))
    main(sys.argv[1], os.path.join(here, "reference_vectors.npz"))
