"""Helpers shared by the tests."""
import numpy as np
import torch

from oracle import numerics as num


def bf16_to_np(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> fp32 numpy array holding the same values."""
    return t.detach().cpu().float().numpy()


def np_to_bf16(a: np.ndarray, device="cpu") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).to(device)


def close_bf16(got: np.ndarray, ref: np.ndarray, rtol=2e-2, atol=1e-2):
    """The bf16 output tolerance of the target: 2e-2 relative / 1e-2 absolute."""
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    lim = atol + rtol * np.abs(ref.astype(np.float64))
    bad = err > lim
    return not bad.any(), float(err.max()), int(bad.sum())


def dev():
    return torch.device("cuda", 0)
