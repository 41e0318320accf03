"""Decode-width dense projection (fp8 block-scaled) and add + RMSNorm on the GPU through the C ABI."""
import numpy as np
import pytest
import torch

from bundles_b200 import ops, synth
from oracle import attn_lmhead as oat
from tests.util import bf16_to_np, close_bf16, dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,H,N", [(64, 2048, 12352), (8, 4096, 2048), (1, 2048, 9216), (33, 2048, 200), (150, 2048, 640),
                                   (256, 4096, 2048), (100, 2048, 640), (512, 2048, 256), (600, 2048, 256)])
def test_dense_projection(T, H, N):
    g = torch.Generator().manual_seed(T + N)
    npad = (N + 127) // 128 * 128
    w = torch.zeros(npad, H)
    w[:N] = torch.randn(N, H, generator=g) * 0.02
    codes, scales = synth.quant_fp8_blocks(w)
    codes = codes[:N].contiguous()
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    st = ops.new_status(dev())
    out = ops.dense_fp8(x.to(dev()), codes.to(dev()), scales.to(dev()), status=st)
    torch.cuda.synchronize()
    assert ops.read_status(st) == 0
    ref = oat.dense_fp8(bf16_to_np(x), codes.numpy(), scales.numpy())
    ok, err, nbad = close_bf16(bf16_to_np(out), ref)
    assert ok, (err, nbad)


def test_rows_do_not_depend_on_the_batch_they_are_in():
    # 64-row calls take 64-row chunks, larger calls 128-row chunks: a row's bits are the same in both
    g = torch.Generator().manual_seed(21)
    H, N = 2048, 640
    w = torch.randn(N, H, generator=g) * 0.02
    codes, scales = synth.quant_fp8_blocks(w)
    codes, scales = codes.to(dev()), scales.to(dev())
    x = torch.randn(230, H, generator=g).to(torch.bfloat16).to(dev())
    st = ops.new_status(dev())
    whole = ops.dense_fp8(x, codes, scales, status=st)
    for lo, hi in ((0, 64), (64, 100), (128, 230), (200, 230)):
        part = ops.dense_fp8(x[lo:hi].contiguous(), codes, scales, status=st)
        assert torch.equal(part, whole[lo:hi]), (lo, hi)
    torch.cuda.synchronize()
    assert ops.read_status(st) == 0


def test_split_outputs_equal_the_plain_projection():
    # the GDN in_proj's four consumers get their own buffers; 80 rows run as two launches
    g = torch.Generator().manual_seed(9)
    T, H, widths = 80, 2048, (8192, 4096, 32, 32)
    N = sum(widths)
    npad = (N + 127) // 128 * 128
    w = torch.zeros(npad, H)
    w[:N] = torch.randn(N, H, generator=g) * 0.02
    codes, scales = synth.quant_fp8_blocks(w)
    codes = codes[:N].contiguous().to(dev())
    scales = scales.to(dev())
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev())
    st = ops.new_status(dev())
    whole = ops.dense_fp8(x, codes, scales, status=st)
    parts = ops.dense_fp8_split(x, codes, scales, widths, status=st)
    torch.cuda.synchronize()
    assert ops.read_status(st) == 0
    lo = 0
    for p, wd in zip(parts, widths):
        assert tuple(p.shape) == (T, wd) and torch.equal(p, whole[:, lo:lo + wd])
        lo += wd
    with pytest.raises(ops.B200Error):
        ops.dense_fp8_split(x, codes, scales, (8192, 4100, 28, 32))     # inner boundary not a multiple of 32


@pytest.mark.parametrize("T", [5, 32, 150, 256])
def test_projection_fused_with_add_and_norm(T):
    """The split-K output projection + residual add + norm against the oracle's projection followed by its add + norm
    (the rounded projection within the bf16 tolerance, the add and the norm exact on that projection), and a row's
    result independent of the batch it is in."""
    g = torch.Generator().manual_seed(40 + T)
    K, N = 4096, 2048
    w = torch.randn(N, K, generator=g) * 0.02
    codes, scales = synth.quant_fp8_blocks(w)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    res = torch.randn(T, N, generator=g).to(torch.bfloat16)
    nw = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16)
    st = ops.new_status(dev())
    r_dev = res.to(dev()).clone()
    proj = torch.empty(T, N, dtype=torch.bfloat16, device=dev())
    cd, sd, xd, nd = codes.to(dev()), scales.to(dev()), x.to(dev()), nw.to(dev())
    y = ops.dense_fp8_add_rmsnorm(xd, cd, sd, r_dev, nd, 1e-6, proj_out=proj, status=st)
    torch.cuda.synchronize()
    assert ops.read_status(st) == 0
    ok, err, nbad = close_bf16(bf16_to_np(proj), oat.dense_fp8(bf16_to_np(x), codes.numpy(), scales.numpy()))
    assert ok, (err, nbad)
    ry, rr = oat.add_rmsnorm(bf16_to_np(proj), bf16_to_np(res), bf16_to_np(nw), 1e-6)
    assert np.array_equal(bf16_to_np(r_dev), rr)
    ok, err, nbad = close_bf16(bf16_to_np(y), ry)
    assert ok, (err, nbad)
    if T > 8:   # the first 8 rows alone give the same bits
        r8 = res[:8].to(dev()).clone()
        y8 = ops.dense_fp8_add_rmsnorm(xd[:8].contiguous(), cd, sd, r8, nd, 1e-6, status=st)
        torch.cuda.synchronize()
        assert torch.equal(y8, y[:8]) and torch.equal(r8, r_dev[:8])


def test_add_rmsnorm():
    g = torch.Generator().manual_seed(5)
    T, H = 37, 2048
    proj = torch.randn(T, H, generator=g).to(torch.bfloat16)
    res = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w = (torch.randn(H, generator=g) * 0.1).to(torch.bfloat16)
    r_dev = res.to(dev()).clone()
    y = ops.add_rmsnorm(proj.to(dev()), r_dev, w.to(dev()), 1e-6)
    torch.cuda.synchronize()
    ry, rr = oat.add_rmsnorm(bf16_to_np(proj), bf16_to_np(res), bf16_to_np(w), 1e-6)
    assert np.array_equal(bf16_to_np(r_dev), rr)
    ok, err, nbad = close_bf16(bf16_to_np(y), ry)
    assert ok, (err, nbad)


def test_rows_quantised_by_the_combine_give_the_same_projection_bits():
    # combine + norm leaves the normed rows also as e4m3 + scales; the projections read those instead of quantising again
    g = torch.Generator().manual_seed(33)
    T, H, K = 37, 2048, 10
    cache = (torch.randn(T * (K + 1), H, generator=g) * 0.3).to(torch.bfloat16).to(dev())
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev())
    gate_w = (torch.randn(H, generator=g) * 0.02).to(torch.bfloat16).to(dev())
    norm_w = (torch.randn(H, generator=g) * 0.1).to(torch.bfloat16).to(dev())
    res_a = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev())
    res_b = res_a.clone()
    xq = torch.empty(T, H, dtype=torch.uint8, device=dev())
    xs = torch.empty(T, H // 128, dtype=torch.float32, device=dev())
    out_a, h_a = ops.moe_combine_norm(cache, x, gate_w, K, res_a, norm_w)
    out_b, h_b = ops.moe_combine_norm(cache, x, gate_w, K, res_b, norm_w, quantised=(xq, xs))
    assert torch.equal(out_a, out_b) and torch.equal(h_a, h_b) and torch.equal(res_a, res_b)
    widths = (8192, 4096, 32, 32)
    N = sum(widths)
    w = torch.randn(N, H, generator=g) * 0.02
    codes, scales = synth.quant_fp8_blocks(torch.cat([w, torch.zeros((-N) % 128, H)]))
    codes, scales = codes[:N].contiguous().to(dev()), scales.to(dev())
    st = ops.new_status(dev())
    plain = ops.dense_fp8_split(h_a, codes, scales, widths, status=st)
    pre = ops.dense_fp8_split(h_a, codes, scales, widths, status=st, quantised=(xq, xs))
    torch.cuda.synchronize()
    assert ops.read_status(st) == 0
    for a, b in zip(plain, pre):
        assert torch.equal(a, b)
    with pytest.raises(ops.B200Error):
        ops.moe_combine_norm(cache, x, gate_w, K, res_b, norm_w, quantised=(xq[:, :1024].contiguous(), xs))
