"""W4A8 oracle: FP8-E4M3 activation quantiser and the FP8 x NVFP4 GEMM.

Test infrastructure; see oracle/__init__.py.
"""
import numpy as np

from .formats import E2M1_LUT, E4M3_MAX, e4m3_decode, e4m3_encode, round_to_bf16


def quantize_activation_fp8(x_bf16):
    """`quantizeToFP8PerRowKernel` (openpi/w4a8_plugin/src/w4a8_gemm_kernel.cu:57-137).

    Per (row, 16-block): scale = max|x|/448 + 1e-12 (fp32), stored as E4M3
    (satfinite); value = E4M3(clamp(x / scale_fp32, +-448)).
    The kernel as launched only reaches the first 32 blocks of a row (its block
    count is capped at 1024 threads, :128-136); the oracle quantises EVERY block,
    which is the stated intent of the routine.
    Returns (values E4M3 bytes (M, K), scales E4M3 bytes (M, K/16))."""
    x = round_to_bf16(x_bf16)
    M, K = x.shape
    xb = x.reshape(M, K // 16, 16)
    bmax = np.abs(xb).max(axis=2).astype(np.float32)
    scale = (bmax / np.float32(E4M3_MAX) + np.float32(1e-12)).astype(np.float32)
    scaled = (xb / scale[:, :, None]).astype(np.float32)
    scaled = np.clip(scaled, -E4M3_MAX, E4M3_MAX)
    return e4m3_encode(scaled).reshape(M, K), e4m3_encode(scale)


def gemm(act_fp8, act_scale, w_packed_t, w_scale_t, alpha=1.0):
    """`w4a8GemmForward` semantics (openpi/w4a8_plugin/src/w4a8_gemm_plugin.h:39-52):
    D[m,n] = alpha * sum_k (A8[m,k] * sA[m,k/16]) * (LUT[code[k,n]] * sW[k/16,n]),
    with the weight operand stored transposed: packed [K/2, N], scales [K/16, N].
    float64 accumulation."""
    a = e4m3_decode(act_fp8).astype(np.float64)
    sa = np.repeat(e4m3_decode(act_scale).astype(np.float64), 16, axis=1)
    p = np.asarray(w_packed_t, dtype=np.uint8)          # (K/2, N)
    Kh, N = p.shape
    codes = np.empty((Kh * 2, N), dtype=np.uint8)
    codes[0::2] = p & 0xF
    codes[1::2] = p >> 4
    w = E2M1_LUT[codes].astype(np.float64)
    sw = np.repeat(e4m3_decode(w_scale_t).astype(np.float64), 16, axis=0)
    return alpha * ((a * sa) @ (w * sw))
