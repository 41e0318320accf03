"""CPU checks of the C-ABI library: it loads without a GPU, exports every symbol the public
header declares, and rejects bad arguments with error codes before touching the device."""
import ctypes as C
import os
import re

import pytest

from bundles_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200nodes.h")


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.lib()


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 9
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/b200nodes.h but not exported: {missing}"


def test_prototypes_cover_header(lib):
    assert set(_lib.PROTOTYPES) == set(declared_symbols())


def test_version_and_error_text(lib):
    assert lib.b200_abi_version() == 1
    rc = lib.b200_router(None, None, None, 4, 2048, 512, 10, 0, None, None, None, None, 0, None)
    assert rc == -1
    assert b"b200_router" in lib.b200_last_error()


def test_argument_checks_return_codes(lib):
    one = C.c_void_p(4096)  # never dereferenced: the checks fail first
    # H not a multiple of 128
    assert lib.b200_router(one, one, None, 4, 100, 512, 10, 0, one, one, one, one, 1 << 30, None) == -1
    # K > E
    assert lib.b200_router(one, one, None, 4, 2048, 64, 65, 0, one, one, one, one, 1 << 30, None) == -1
    # misaligned x
    assert lib.b200_router(C.c_void_p(4100), one, None, 4, 2048, 512, 10, 0, one, one, one, one, 1 << 30, None) == -2
    # scratch too small
    assert lib.b200_router(one, one, None, 4, 2048, 512, 10, 0, one, one, one, one, 64, None) == -3
    assert lib.b200_router_scratch_bytes(256, 2048, 512) == 16 * 256 * 512 * 4
    assert lib.b200_moe_max_blocks(256, 10, 512, 128) >= 512 + 20 + 2
    assert lib.b200_moe_w8a8_workspace_bytes(256, 2048, 512, 10) > 256 * 11 * 2048
    assert lib.b200_moe_combine(None, None, None, None, 1, 2048, 10, None, None) == -1
    assert lib.b200_gdn_verify(*([None] * 11), 1e-6, 1, None, None, 0, None, None) == -1
    assert lib.b200_gdn_workspace_bytes(2) == 2 * (16 * 4096 + 32 * 2832) and lib.b200_gdn_workspace_bytes(0) == 0
    # attention verify: null pointers, bad split count, workspace too small, misaligned cache
    assert lib.b200_attn_verify(*([None] * 6), 8, None, 4, None, 2, 0.0625, 1, None, None, 0, None, None) == -1
    av = [one] * 6 + [8, one, 4, one, 2, 0.0625]
    assert lib.b200_attn_verify(*av, 65, one, one, 1 << 30, None, None) == -1
    assert lib.b200_attn_verify(*av, 2, one, one, 64, None, None) == -3
    bad = [one, one, one, one, C.c_void_p(4100), one, 8, one, 4, one, 2, 0.0625]
    assert lib.b200_attn_verify(*bad, 2, one, one, 1 << 30, None, None) == -2
    assert lib.b200_attn_verify_workspace_bytes(2, 3) == 2 * 2 * 3 * (32 * 256 * 4 + 2 * 32 * 4)
    assert lib.b200_attn_verify_splits(0) == 0
    assert lib.b200_moe_combine_norm(None, None, None, None, 1, 2048, 10, None, None, None, 1e-6, None, None) == -1
    assert lib.b200_moe_combine_norm(one, one, None, None, 1, 2047, 10, None, one, one, 1e-6, one, None) == -1
    # GDN verify on the ring layout: null pointers, slot count out of range, misaligned checkpoint
    assert lib.b200_gdn_verify_replay(*([None] * 10), 4, *([None] * 11), 1e-6, 1, None, None, 0, None, None) == -1
    ok = [one] * 10
    assert lib.b200_gdn_verify_replay(*ok, 0, *([one] * 11), 1e-6, 1, one, one, 1 << 30, None, None) == -1
    assert lib.b200_gdn_ring_fold(*([None] * 10), 1, None) == -1
    assert lib.b200_gdn_ring_fold(C.c_void_p(4100), *([one] * 9), 1, None) == -2
    # expert-parallel plumbing
    assert lib.b200_ep_barrier(None, None, 2, 0, 0, 1000, None, None) == -1
    ptrs = (C.c_void_p * 2)(4096, 8192)
    assert lib.b200_ep_barrier(ptrs, one, 9, 0, 0, 1000, None, None) == -1          # more than 8 ranks
    assert lib.b200_ep_barrier(ptrs, one, 2, 0, 4, 1000, None, None) == -1          # channel out of range
    assert lib.b200_ep_barrier(ptrs, one, 2, 0, 0, 0, None, None) == -1             # a barrier without a time limit
    odd = (C.c_void_p * 2)(4096, 8194)
    assert lib.b200_ep_barrier(odd, one, 2, 0, 0, 1000, None, None) == -2
    assert lib.b200_ep_put(one, 6, 0, ptrs, 2, None) == -1                          # not a multiple of 4 bytes
    assert lib.b200_ep_put(one, 0, 0, ptrs, 2, None) == 0                           # nothing to store
    assert lib.b200_moe_fp8_ep(one, 64, 2048, 512, 10, 8, None, None, ptrs, 2, 0, 16, one, 1 << 30, None, None) == -1
    assert lib.b200_selftest_wait_expiry(None, None) == -1
    cols, lds = (C.c_int * 2)(100, 28), (C.c_int * 2)(100, 28)
    assert lib.b200_dense_fp8_split(one, 4, 2048, one, one, 128, 2, cols, ptrs, lds, one, 1 << 30, None, None) == -1
    assert lib.b200_dense_fp8_add_rmsnorm(one, 4, 4000, one, one, 2048, one, one, 1e-6, one, None, one, 1 << 30, None, None) == -1
    assert lib.b200_dense_fp8_add_rmsnorm(one, 4, 4096, one, one, 2048, one, one, 1e-6, one, None, one, 64, None, None) == -3
    assert lib.b200_dense_fp8_add_rmsnorm_workspace_bytes(4, 4096, 2048) > 4 * 2048 * 4
    mis = [one] * 9 + [C.c_void_p(4100)]
    assert lib.b200_gdn_verify_replay(*mis, 4, *([one] * 11), 1e-6, 1, one, one, 1 << 30, None, None) == -2


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()
