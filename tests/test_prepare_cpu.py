"""The prepare-time weight quantisers of the product (bundles_b200/prepare.py, torch) against the oracle's numpy
restatement, which is pinned to the reference's own quantisers (tests/test_oracle_golden.py): bit-identical int8
codes, e4m3 codes and scales, including all-zero rows / blocks, values on rounding ties and saturating values."""
import numpy as np
import torch

from bundles_b200 import prepare
from oracle import numerics as num


def _weights(seed, *shape):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(*shape, generator=g) * 0.02
    return w


def test_int8_rows_equal_the_oracle():
    w = _weights(1, 96, 512)
    w[3] = 0.0                                   # all-zero row: scale 0, divided by 1
    w[5, :8] = torch.tensor([0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 127.0, -127.0]) * (w[5].abs().max() / 127.0)  # ties
    q, s = prepare.quant_int8_rows(w)
    rq, rs = num.quant_int8_rows(w.numpy())
    assert q.dtype == torch.int8 and s.dtype == torch.float32
    assert np.array_equal(q.numpy(), rq)
    assert np.array_equal(s.numpy().view(np.uint32), rs.view(np.uint32))


def test_int8_rows_of_an_expert_stack():
    w = _weights(2, 4, 256, 384)
    q, s = prepare.quant_int8_rows(w)
    for e in range(4):
        rq, rs = num.quant_int8_rows(w[e].numpy())
        assert np.array_equal(q[e].numpy(), rq) and np.array_equal(s[e].numpy(), rs)


def test_fp8_blocks_equal_the_oracle():
    w = _weights(3, 384, 512)
    w[128:256, 128:256] = 0.0                    # all-zero block: scale clamps to 1e-12
    w[0, 0] = 3.0                                # a block whose amax is far above the rest
    q, s = prepare.quant_fp8_blocks(w)
    rq, rs = num.quant_fp8_blocks(w.numpy())
    assert q.dtype == torch.uint8 and tuple(s.shape) == (3, 4)
    assert np.array_equal(q.numpy(), rq)
    assert np.array_equal(s.numpy().view(np.uint32), rs.view(np.uint32))


def test_fp8_blocks_of_an_expert_stack():
    w = _weights(4, 3, 256, 256)
    q, s = prepare.quant_fp8_blocks(w)
    rq, rs = num.quant_fp8_blocks(w.numpy())
    assert np.array_equal(q.numpy(), rq) and np.array_equal(s.numpy(), rs)


def test_synth_uses_the_product_quantisers():
    from bundles_b200 import synth
    assert synth.quant_fp8_blocks is prepare.quant_fp8_blocks and synth.quant_int8_rows is prepare.quant_int8_rows
