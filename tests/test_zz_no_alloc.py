"""The router entry point for hosts that cannot allocate device memory (`b200_router_static`).

Some callers of the library (a per-step plugin slot of a serving engine, for one) only ever see the
buffers the engine hands them and must not call cudaMalloc.  For them the router keeps its scratch
in an array inside the library.  This test calls that entry point through the C ABI twice in a row
and checks both results against the ordinary entry point, which takes a caller-provided scratch.
It is collected last so that a failure here cannot hide any other test's result.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from bundles_b200 import _lib, ops

pytestmark = pytest.mark.gpu


def _static_router(x, wr, bias, K):
    T, H = x.shape
    E = wr.shape[0]
    logits = torch.empty(T, E, dtype=torch.float32, device=x.device)
    ids = torch.empty(T, K, dtype=torch.int32, device=x.device)
    wts = torch.empty(T, K, dtype=torch.float32, device=x.device)
    p = lambda t: None if t is None else C.c_void_p(t.data_ptr())  # noqa: E731
    rc = _lib.lib().b200_router_static(p(x), p(wr), p(bias), T, H, E, K, 0, p(logits), p(ids), p(wts),
                                       C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, logits, ids, wts


def test_static_router_matches_router_twice_in_a_row():
    dev = torch.device("cuda", 0)
    K = 10
    for call, (T, seed) in enumerate([(64, 901), (17, 902)]):   # the second call reuses the array's old contents
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(T, 2048, generator=g).to(torch.bfloat16).to(dev)
        wr = (torch.randn(512, 2048, generator=g) * 0.02).to(dev)
        bias = torch.randn(512, generator=g).to(dev)
        rc, logits, ids, wts = _static_router(x, wr, bias, K)
        assert rc == 0, _lib.lib().b200_last_error()
        ref_logits, ref_ids, ref_wts = ops.router(x, wr, K, bias)
        torch.cuda.synchronize()
        assert torch.equal(ids, ref_ids), f"call {call}: expert ids differ"
        assert np.array_equal(logits.cpu().numpy().view(np.uint32), ref_logits.cpu().numpy().view(np.uint32))
        np.testing.assert_allclose(wts.cpu().numpy(), ref_wts.cpu().numpy(), rtol=1e-5, atol=1e-8)


def test_static_router_rejects_sizes_beyond_its_array():
    dev = torch.device("cuda", 0)
    lib = _lib.lib()
    cap = lib.b200_router_static_max_scratch_bytes()
    assert lib.b200_router_scratch_bytes(64, 2048, 512) <= cap < lib.b200_router_scratch_bytes(128, 2048, 512)
    x = torch.zeros(256, 2048, dtype=torch.bfloat16, device=dev)
    wr = torch.zeros(512, 2048, device=dev)
    rc, *_ = _static_router(x, wr, None, 10)        # 256 tokens need 8 MiB, the array holds 2 MiB
    assert rc == -3
    assert b"built-in scratch" in lib.b200_last_error()
