"""Number formats and quantisers shared by the oracle (test infrastructure, never shipped).

bf16 and e4m3 are emulated on numpy float32 so that every rounding point is explicit.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


# ----------------------------------------------------------------------------------------------
# bf16
# ----------------------------------------------------------------------------------------------
def bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit pattern (uint16), round to nearest even; NaN stays NaN."""
    u = np.ascontiguousarray(x, dtype=F32).view(np.uint32)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    r = (u + np.uint32(0x7FFF) + lsb) >> np.uint32(16)
    nan = np.isnan(x)
    r = np.where(nan, np.uint32(0x7FC0), r)
    return r.astype(np.uint16)


def bf16_from_bits(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(F32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 value of x after a round trip through bf16 (the reference's explicit rounding points)."""
    return bf16_from_bits(bf16_bits(np.asarray(x, dtype=F32))).reshape(np.shape(x))


# ----------------------------------------------------------------------------------------------
# e4m3 (OCP "fn" flavour: no inf, max 448, NaN = 0x7f)
# ----------------------------------------------------------------------------------------------
def _e4m3_table() -> np.ndarray:
    t = np.zeros(256, dtype=F32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 7
        if e == 0xF and m == 7:
            v = np.nan
        elif e == 0:
            v = s * m * 2.0 ** -9
        else:
            v = s * (1 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = v
    return t


E4M3_TABLE = _e4m3_table()
E4M3_MAX = F32(448.0)


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    return E4M3_TABLE[np.asarray(b, dtype=np.uint8)]


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """fp32 -> e4m3 byte, round to nearest even, saturating to +-448 (PTX cvt.rn.satfinite.e4m3x2.f32,
    the conversion the reference uses for q/k/v: qk_attn_verify.cu:142-146)."""
    x = np.asarray(x, dtype=F32)
    a = np.minimum(np.abs(np.where(np.isnan(x), F32(0.0), x)), E4M3_MAX).astype(np.float64)   # NaN is set at the end
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, -6.0)
    q = np.exp2(e - 3.0)
    r = np.rint(a / q) * q  # rint = ties to even; a / q is exact (power-of-two divisor)
    r = np.minimum(r, 448.0)
    # value -> code: positive codes are monotone in value
    pos = E4M3_TABLE[:127].astype(np.float64)  # 0 .. 448
    code = np.searchsorted(pos, r).astype(np.uint8)
    assert np.all(pos[code] == r), "e4m3 rounding produced a non-representable value"
    sign = (np.signbit(x)).astype(np.uint8) << 7
    out = code | sign
    return np.where(np.isnan(x), np.uint8(0x7F), out).astype(np.uint8)


# ----------------------------------------------------------------------------------------------
# exact fp32 fused multiply-add on numpy arrays
# ----------------------------------------------------------------------------------------------
def fma32(a: np.ndarray, b: np.ndarray, c: np.ndarray) -> np.ndarray:
    """Correctly rounded fp32 fma(a, b, c) (what `fmaf` / `__fmaf_rn` return).

    a*b is exact in float64 (24+24 significand bits).  p + c in float64 is rounded once to 53
    bits; rounding that to fp32 can double-round only when the 53-bit sum sits exactly on an
    fp32 tie while the exact sum does not.  TwoSum recovers the residual and the tie is
    nudged toward it, which makes the final rounding exact.
    """
    p = a.astype(np.float64) * b.astype(np.float64)
    c = c.astype(np.float64)
    s = p + c
    bb = s - p
    err = (p - (s - bb)) + (c - bb)  # exact residual of p + c
    u = s.view(np.uint64)
    tie = (u & np.uint64(0x1FFFFFFF)) == np.uint64(0x10000000)
    fix = tie & (err != 0) & np.isfinite(s)
    if np.any(fix):
        toward = np.where(err > 0, np.inf, -np.inf)
        s = np.where(fix, np.nextafter(s, toward), s)
    return s.astype(F32)


# ----------------------------------------------------------------------------------------------
# quantisers
# ----------------------------------------------------------------------------------------------
def round_half_away(v: np.ndarray) -> np.ndarray:
    """r = v >= 0 ? floor(v + 0.5) : -floor(0.5 - v), in fp32 (qwen36_lmhead8/w8a8.py:21)."""
    v = np.asarray(v, dtype=F32)
    return np.where(v >= 0, np.floor(v + F32(0.5)), -np.floor(F32(0.5) - v)).astype(F32)


def quant_int8_rows(x: np.ndarray):
    """Symmetric int8 per row: scale = amax / 127 (IEEE division), q = round-half-away(x / scale)
    clamped to +-127; an all-zero row gets scale 0 and divides by 1.

    Follows `_round_int8` / `_quant_act_kernel` (qwen36_lmhead8/w8a8.py:15-36), which is also the
    per-output-channel weight convention of `quantize_rows` (qwen36_lmhead8/lmhead8.py:95-108).
    Returns (q int8 [rows, k], scale fp32 [rows]).
    """
    x = np.asarray(x, dtype=F32)
    amax = np.max(np.abs(x), axis=-1)
    scale = (amax / F32(127.0)).astype(F32)
    safe = np.where(amax > 0, scale, F32(1.0)).astype(F32)
    v = (x / safe[..., None]).astype(F32)
    r = np.clip(round_half_away(v), -127.0, 127.0)
    return r.astype(np.int8), scale


def quant_int8_channel_fp16(w: np.ndarray, group: int = 128):
    """The reference's own expert-weight quantiser (i8x_kernels.py:112-125): one scale per row,
    stored as fp16 with one-ulp headroom (x 1.0009765625) and replicated per 128-k group.
    Kept for pinning against the reference at its own format; the target format uses
    `quant_int8_rows` (fp32 scale, no headroom)."""
    w = np.asarray(w, dtype=F32)
    amax = np.max(np.abs(w), axis=-1)
    s16 = ((amax / F32(127.0)).astype(F32) * F32(1.0009765625)).astype(F32).astype(np.float16)
    s = s16.astype(F32)
    v = (w / np.where(s > 0, s, F32(1.0))[..., None]).astype(F32)
    r = np.clip(round_half_away(v), -127.0, 127.0)
    c = np.repeat(s16[..., None], w.shape[-1] // group, axis=-1)
    return r.astype(np.int8), c


def quant_fp8_groups(x: np.ndarray, group: int = 128):
    """Activations -> e4m3 with one fp32 scale per (row, 128-channel group): scale = max(amax / 448,
    1e-12), y = e4m3(x * (1 / scale)).

    The scale and reciprocal-multiply form is the reference's row-wise fp8 quantiser
    (`_rowwise_fp8`, fp8.py:21-34) applied per 128-channel group instead of per row.
    Returns (codes uint8 [rows, k], scale fp32 [rows, k / group]).
    """
    x = np.asarray(x, dtype=F32)
    rows, k = x.shape
    g = x.reshape(rows, k // group, group)
    amax = np.max(np.abs(g), axis=-1)
    scale = np.maximum((amax / F32(448.0)).astype(F32), F32(1e-12)).astype(F32)
    inv = (F32(1.0) / scale).astype(F32)
    y = (g * inv[..., None]).astype(F32)
    return e4m3_encode(y).reshape(rows, k), scale


def quant_fp8_blocks(w: np.ndarray, block: int = 128):
    """Weights -> e4m3 with one fp32 scale per 128 x 128 block (scale = max(block amax / 448, 1e-12)).
    Same scale rule as `quant_fp8_groups`; w is [..., n, k] with n, k multiples of 128.
    Returns (codes uint8 [..., n, k], scale fp32 [..., n/128, k/128])."""
    w = np.asarray(w, dtype=F32)
    *lead, n, k = w.shape
    b = w.reshape(*lead, n // block, block, k // block, block)
    amax = np.max(np.abs(b), axis=(-3, -1))
    scale = np.maximum((amax / F32(448.0)).astype(F32), F32(1e-12)).astype(F32)
    inv = (F32(1.0) / scale).astype(F32)
    y = (b * inv[..., :, None, :, None]).astype(F32)
    return e4m3_encode(y).reshape(*lead, n, k), scale


def silu_mul_bf16(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    """SwiGLU with the reference's rounding points (`_swiglu_store`, i8x_decode.py:151-156):
    g, u rounded to bf16, h = bf16(g / (1 + exp(-g)) * u).  Returns fp32 values on the bf16 grid."""
    g = bf16_round(g)
    u = bf16_round(u)
    with np.errstate(over="ignore"):
        h = (g / (F32(1.0) + np.exp(-g, dtype=F32)) * u).astype(F32)
    return bf16_round(h)
