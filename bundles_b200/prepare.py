"""Prepare-time weight quantisers: what the layer and LM-head nodes run once per module to build their private
low-precision copies (the reference quantises its private expert copy at prepare time as well:
i8x_reloc.py:193-241, i8x_kernels.py:112-148, qwen36_lmhead8/lmhead8.py:95-108).  torch tensor code that runs on
whichever device holds the weight; the results are bit-identical on CPU and GPU because every step is an IEEE
operation on fp32 (tensor / tensor divisions, no fused multiply-add).
"""
from __future__ import annotations

import torch


def quant_int8_rows(w: torch.Tensor):
    """Symmetric int8 per row (last dim): scale = amax / 127, round half away from zero, clamp +-127
    (qwen36_lmhead8/lmhead8.py:95-108 `quantize_rows`).  Returns (int8, fp32 scale)."""
    wf = w.float()
    amax = wf.abs().amax(dim=-1)
    # tensor / tensor: an IEEE division on every device (tensor / python scalar is a multiplication by the
    # rounded reciprocal on CUDA, one ulp off amax / 127 now and then)
    scale = amax / torch.full_like(amax, 127.0)
    safe = torch.where(amax > 0, scale, torch.ones_like(scale))
    v = wf / safe.unsqueeze(-1)
    r = torch.where(v >= 0, torch.floor(v + 0.5), -torch.floor(0.5 - v)).clamp_(-127, 127)
    return r.to(torch.int8), scale


def quant_fp8_blocks(w: torch.Tensor, block: int = 128):
    """e4m3 with one fp32 scale per 128 x 128 block: scale = max(amax / 448, 1e-12), y = e4m3(w / scale)
    computed as w * (1 / scale) (fp8.py:21-34 scale rule).  Returns (uint8 codes, fp32 scales)."""
    wf = w.float()
    *lead, n, k = wf.shape
    b = wf.reshape(*lead, n // block, block, k // block, block)
    amax = b.abs().amax(dim=(-3, -1))
    scale = (amax / torch.full_like(amax, 448.0)).clamp_min(1e-12)   # IEEE division, see quant_int8_rows
    inv = torch.ones_like(scale) / scale
    y = (b * inv[..., :, None, :, None]).clamp_(-448.0, 448.0)
    codes = y.reshape(*lead, n, k).to(torch.float8_e4m3fn).view(torch.uint8)
    return codes, scale
