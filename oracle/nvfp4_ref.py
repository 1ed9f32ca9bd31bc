"""TEST INFRASTRUCTURE ONLY: CPU restatement (numpy) of the NVFP4 weight codec of the reference.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module; the
product path never does.

Format (muse_prefill_layer/nvfp4.py:1-8): value = e2m1 * block_scale(e4m3) * global_scale(fp32);
16-element blocks along the last dim; two 4-bit codes per byte, element 2i in the low nibble
and element 2i+1 in the high nibble; bit 3 of a code is the sign, bits 0-2 index the grid
(0, .5, 1, 1.5, 2, 3, 4, 6) (muse_prefill_layer/nvfp4.py:24-27,40-47).

Parity pin: `tests/test_oracle_golden.py` compares `dequantize` with tensors produced by the
reference's own `nvfp4.dequantize` (stored under tests/golden/).
"""
from __future__ import annotations

import numpy as np

BLOCK = 16
E2M1_GRID = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    """Decode float8_e4m3fn bytes (uint8) to float32. Bias 7, no infinities, 0x7f/0xff = NaN."""
    b = b.astype(np.uint8)
    sign = np.where(b & 0x80, -1.0, 1.0).astype(np.float32)
    e = ((b >> 3) & 0xF).astype(np.int32)
    m = (b & 0x7).astype(np.float32)
    normal = np.ldexp(1.0 + m / 8.0, e - 7)
    sub = np.ldexp(m / 8.0, -6)
    out = np.where(e == 0, sub, normal).astype(np.float32) * sign
    out = np.where((b & 0x7F) == 0x7F, np.float32(np.nan), out)
    return out.astype(np.float32)


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    """uint8 [..., K/2] -> float32 [..., K] (muse_prefill_layer/nvfp4.py:40-47)."""
    p = packed.astype(np.uint8)
    codes = np.stack([p & 0xF, p >> 4], axis=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)
    mag = E2M1_GRID[codes & 7]
    return np.where(codes & 8, -mag, mag).astype(np.float32)


def dequantize(packed: np.ndarray, sf_bytes: np.ndarray, global_scale: float) -> np.ndarray:
    """float32 [..., K]: the block scale times the global scale is rounded to fp32 once, then
    multiplies the E2M1 value (muse_prefill_layer/nvfp4.py:90-97)."""
    vals = unpack_e2m1(packed)
    k = vals.shape[-1]
    scale = e4m3_to_f32(sf_bytes) * np.float32(global_scale)
    out = vals.reshape(*vals.shape[:-1], k // BLOCK, BLOCK) * scale[..., None]
    return out.reshape(vals.shape).astype(np.float32)
