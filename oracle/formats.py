"""Number formats used by the oracle: bf16, fp16, E4M3 (fn), E2M1 — numpy only.

Test infrastructure; see oracle/__init__.py.
"""
import numpy as np

# e2m1 magnitudes, index = low three bits of the code; bit 3 is the sign.
# openpi/nvfp4_packed_plugin/src/nvfp4_packed_kernel.cu:41-44
E2M1_MAGNITUDES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_LUT = np.concatenate([E2M1_MAGNITUDES, -E2M1_MAGNITUDES]).astype(np.float32)
E2M1_MAX = 6.0
E4M3_MAX = 448.0


def round_to_bf16(x):
    """float32 -> nearest-even bf16, returned as float32 values."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    out = rounded.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(x), x, out).astype(np.float32)


def bf16_bits(x):
    """float32 -> bf16 bit pattern (uint16), nearest-even."""
    return (round_to_bf16(x).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_to_fp16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def e4m3_decode(code):
    """E4M3 'fn' byte -> float32 (bias 7, no inf, 0x7f/0xff = NaN)."""
    code = np.asarray(code, dtype=np.uint8).astype(np.int32)
    sign = np.where(code & 0x80, -1.0, 1.0).astype(np.float32)
    e = (code >> 3) & 0xF
    m = code & 0x7
    normal = np.ldexp((8 + m).astype(np.float32), e - 10)
    sub = np.ldexp(m.astype(np.float32), -9)
    val = np.where(e == 0, sub, normal)
    val = np.where((e == 15) & (m == 7), np.nan, val)
    return (sign * val).astype(np.float32)


def e4m3_encode(x):
    """float32 -> E4M3 'fn' byte, round-to-nearest-even, saturating to +-448.

    Same result as `__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3)` used by
    openpi/w4a8_plugin/src/w4a8_gemm_kernel.cu:109,131,358 and, for |x| <= 448,
    as torch's `.to(torch.float8_e4m3fn)` used by
    openpi/src/openpi/models_pytorch/nvfp4_mlp.py:211-212,313.
    """
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float64)
    a = np.where(np.isnan(a), 0.0, a)
    a = np.minimum(a, E4M3_MAX)
    # exponent of the value, clamped to the subnormal range
    _, ex = np.frexp(np.where(a == 0, 1.0, a))  # a = f * 2**ex, f in [0.5,1)
    e = np.maximum(ex - 1, -6)
    quantum = np.ldexp(1.0, e - 3)
    q = np.rint(a / quantum) * quantum  # rint = half-to-even
    q = np.minimum(q, E4M3_MAX)
    _, ex2 = np.frexp(np.where(q == 0, 1.0, q))
    e2 = ex2 - 1
    is_sub = (e2 < -6) | (q == 0)
    mant_sub = np.rint(q * 512.0).astype(np.int64)  # q / 2**-9
    mant_norm = np.rint(q / np.ldexp(1.0, e2) * 8.0).astype(np.int64) - 8
    byte = np.where(is_sub, mant_sub, ((e2 + 7) << 3) | mant_norm).astype(np.uint8)
    return (byte | sign).astype(np.uint8)


def round_to_e4m3(x):
    return e4m3_decode(e4m3_encode(x))


def e2m1_decode(code):
    return E2M1_LUT[np.asarray(code, dtype=np.uint8) & 0xF]


def e2m1_nearest_index(abs_vals):
    """Index of the nearest e2m1 magnitude; ties go to the LOWER index, which is
    what `(abs.unsqueeze(-1) - values).abs().argmin(-1)` returns in
    openpi/nvfp4_packed_plugin/python/nvfp4_packed.py:112-113 and the strict `<`
    scan of openpi/w4a8_plugin/src/w4a8_gemm_kernel.cu:380-388."""
    a = np.asarray(abs_vals, dtype=np.float32)
    d = np.abs(a[..., None] - E2M1_MAGNITUDES)
    return np.argmin(d, axis=-1).astype(np.uint8)
