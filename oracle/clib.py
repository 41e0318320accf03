"""ctypes binding of liboracle.so, the C twin of the numpy oracle (test / baseline infrastructure)."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "liboracle.so")
_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(PATH):
            subprocess.run(["make", "-C", HERE, "-s"], check=True)
        _lib = C.CDLL(PATH)
        _lib.oracle_threads.restype = C.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def threads() -> int:
    return int(lib().oracle_threads())


def use_all_cores() -> int:
    """Run on every core this process may use, whatever OMP_NUM_THREADS says (torchrun exports 1 for its ranks)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_threads(C.c_int(n))
    return threads()


def gate_logits(x_bits, wr, bias):
    T, H = x_bits.shape
    E = wr.shape[0]
    out = np.empty((T, E), dtype=np.float32)
    lib().oracle_gate_logits(_p(x_bits), _p(wr), None if bias is None else _p(bias), T, H, E, _p(out))
    return out


def topk(logits, K, round_bf16=False):
    T, E = logits.shape
    ids = np.empty((T, K), dtype=np.int32)
    wts = np.empty((T, K), dtype=np.float32)
    lib().oracle_topk(_p(logits), T, E, K, int(round_bf16), _p(ids), _p(wts))
    return ids, wts


def moe_w8a8(x_bits, ids, wts, w13, s13, w2, s2, sh13, shs13, sh2, shs2, gate_w_bits):
    """All arrays C-contiguous numpy: x_bits / gate_w_bits uint16 bf16 patterns.  Returns out bits [T,H]."""
    T, H = x_bits.shape
    K = ids.shape[1]
    I = w2.shape[-1]
    cache = np.empty((T * (K + 1), H), dtype=np.uint16)
    out = np.empty((T, H), dtype=np.uint16)
    lib().oracle_moe_w8a8(_p(x_bits), _p(ids), _p(wts), T, H, I, K, _p(w13), _p(s13), _p(w2), _p(s2), _p(sh13),
                          _p(shs13), _p(sh2), _p(shs2), _p(gate_w_bits), _p(cache), _p(out))
    return out, cache


def e4m3_encode(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint8)
    lib().oracle_e4m3_encode(_p(x), C.c_size_t(x.size), _p(out))
    return out


def quant_fp8_groups(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, n = x.shape
    q = np.empty((rows, n), dtype=np.uint8)
    s = np.empty((rows, n // 128), dtype=np.float32)
    lib().oracle_quant_fp8_groups(_p(x), rows, n, _p(q), _p(s))
    return q, s


def gemm_fp8_blocks(aq, a_s, wq, w_s):
    """out fp32 [M, N]: the block-scaled GEMM with per-128-k promotion (oracle/moe.py gemm_fp8_blocks)."""
    M, K = aq.shape
    N = wq.shape[0]
    out = np.empty((M, N), dtype=np.float32)
    lib().oracle_gemm_fp8_blocks(_p(np.ascontiguousarray(aq)), _p(np.ascontiguousarray(a_s, dtype=np.float32)), M, K,
                                 _p(np.ascontiguousarray(wq)), _p(np.ascontiguousarray(w_s, dtype=np.float32)), N, _p(out))
    return out


def moe_fp8(x_bits, ids, wts, w13, s13, w2, s2, sh13, shs13, sh2, shs2, gate_w_bits):
    """fp8 block-scaled MoE block; all arrays C-contiguous numpy (x_bits / gate_w_bits uint16 bf16 patterns, weights
    uint8 e4m3 codes).  Returns (out bits [T,H], cache bits [T*(K+1),H])."""
    T, H = x_bits.shape
    K = ids.shape[1]
    E = w13.shape[0]
    I = w2.shape[-1]
    cache = np.zeros((T * (K + 1), H), dtype=np.uint16)
    out = np.empty((T, H), dtype=np.uint16)
    lib().oracle_moe_fp8(_p(x_bits), _p(ids), _p(wts), T, H, I, K, E, _p(w13), _p(s13), _p(w2), _p(s2), _p(sh13),
                         _p(shs13), _p(sh2), _p(shs2), _p(gate_w_bits), _p(cache), _p(out))
    return out, cache
