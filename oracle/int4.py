"""INT4 (W4A16) oracle: packers, dequant, GEMV, and the plugin's quantisers.

Test infrastructure; see oracle/__init__.py.  All arithmetic is float32 where
the reference's is float32, float16 where it is float16.
"""
import numpy as np

from .formats import round_to_bf16, round_to_fp16

QUANT_BLOCK = 32  # openpi/src/openpi/utils/w4a16_packer.py:39
INT4_OFFSET = 8   # :44
INT4_RANGE = 7    # :45


def _pack_words(q, layout):
    """q: (N, K) uint8 codes 0..15 -> int32 words, nibble i of a word at bits 4i
    (openpi/src/openpi/utils/w4a16_packer.py:166-172,346-350).

    layout "kblock": (K/32, N, 4)  -- the reference's block-interleaved order
    layout "rowmajor": (N, K/8)    -- 8 codes per word along K
    """
    N, K = q.shape
    words = q.reshape(N, K // 8, 8).astype(np.uint32)
    shifts = (np.arange(8, dtype=np.uint32) * 4)
    packed = (words << shifts).sum(axis=2, dtype=np.uint32)  # (N, K/8)
    if layout == "rowmajor":
        return packed.view(np.int32)
    assert layout == "kblock"
    return np.ascontiguousarray(
        packed.reshape(N, K // 32, 4).transpose(1, 0, 2)).view(np.int32)


def pack_fast(weight, block_size=QUANT_BLOCK, layout="kblock"):
    """`W4A16PackerFast.pack` (openpi/src/openpi/utils/w4a16_packer.py:311-368).

    scale = max|w|/7 clamped to >= 1e-8 (fp32); q = clamp(round(w/scale + 8), 0, 15)
    with the division by the fp32 scale; the scale is stored as fp16 afterwards.
    Returns (weight_packed int32, scales fp16 (K/block, N)).
    With block_size != 32 only layout "rowmajor" is meaningful; scales are then
    returned as (N, K/block).
    """
    w = np.asarray(weight, dtype=np.float32)
    N, K = w.shape
    assert K % block_size == 0
    nb = K // block_size
    wb = w.reshape(N, nb, block_size)
    scales = (np.abs(wb).max(axis=2) / np.float32(INT4_RANGE)).astype(np.float32)
    scales = np.maximum(scales, np.float32(1e-8))
    q = np.rint(wb / scales[:, :, None] + np.float32(INT4_OFFSET))  # half-to-even, as torch.round
    q = np.clip(q, 0, 15).astype(np.uint8).reshape(N, K)
    packed = _pack_words(q, layout)
    if layout == "kblock":
        assert block_size == QUANT_BLOCK
        return packed, np.ascontiguousarray(scales.T).astype(np.float16)
    return packed, scales.astype(np.float16)


def pack_basic(weight, block_size=QUANT_BLOCK):
    """`W4A16Packer._pack_numpy` (openpi/src/openpi/utils/w4a16_packer.py:129-174):
    the scale is rounded to fp16 FIRST (zero -> 1.0) and the division uses it."""
    w = np.asarray(weight, dtype=np.float32)
    N, K = w.shape
    nb = K // block_size
    wb = w.reshape(N, nb, block_size)
    scales = (np.abs(wb).max(axis=2) / INT4_RANGE).astype(np.float16)
    scales = np.where(scales == 0, np.float16(1.0), scales)
    q = np.round(wb / scales[:, :, None] + INT4_OFFSET)
    q = np.clip(q, 0, 15).astype(np.uint8).reshape(N, K)
    return _pack_words(q, "kblock"), np.ascontiguousarray(scales.T).astype(np.float16)


def unpack_codes(weight_packed, layout="kblock"):
    """int32 words -> (N, K) uint8 codes."""
    p = np.asarray(weight_packed).view(np.uint32)
    if layout == "kblock":
        nb, N, _ = p.shape
        p = p.transpose(1, 0, 2).reshape(N, nb * 4)
    N = p.shape[0]
    shifts = (np.arange(8, dtype=np.uint32) * 4)
    return ((p[:, :, None] >> shifts) & 0xF).astype(np.uint8).reshape(N, -1)


def dequantize(weight_packed, scales, layout="kblock", group_size=QUANT_BLOCK):
    """`W4A16Linear._dequantize_weights` (openpi/src/openpi/modules/w4a16_linear.py:174-199):
    ((q - 8) * scale) computed in fp32 from the fp16 scale, stored as fp16.
    Returns float32 values that are exactly representable in fp16."""
    q = unpack_codes(weight_packed, layout).astype(np.float32)
    s = np.asarray(scales, dtype=np.float16).astype(np.float32)
    if layout == "kblock":
        s = s.T  # (N, K/32)
    s = np.repeat(s, group_size, axis=1)
    return round_to_fp16((q - np.float32(8.0)) * s)


def gemv_reference_math(x, weight_packed, scales, layout="kblock", group_size=QUANT_BLOCK):
    """The TVM kernel's arithmetic (openpi/src/openpi/ops/w4a16_gemv.py:83-100):
    w = fp16((fp16(q) - 8) * scale16); p = fp16(a16 * w); C += fp32(p), k ascending.
    x: (1, K) (rounded to fp16 first, as W4A16Linear._forward_w4a16 does,
    w4a16_linear.py:244-245).  Returns (1, N) float32."""
    x16 = np.asarray(x, dtype=np.float32).astype(np.float16)
    q = unpack_codes(weight_packed, layout)
    s = np.asarray(scales, dtype=np.float16)
    if layout == "kblock":
        s = s.T
    s = np.repeat(s, group_size, axis=1)
    w16 = ((q.astype(np.float16) - np.float16(8.0)) * s).astype(np.float16)
    prod = (x16.reshape(1, 1, -1) * w16[None]).astype(np.float16)  # (M, N, K) fp16 products
    # fp32 accumulation in ascending k; pairwise summation would differ in the last bits only
    acc = np.zeros(prod.shape[:2], dtype=np.float32)
    for k in range(prod.shape[2]):
        acc += prod[:, :, k].astype(np.float32)
    return acc


def gemv_dequant_matmul(x, weight_packed, scales, layout="kblock", group_size=QUANT_BLOCK, bias=None):
    """torch dequant-then-matmul path (`W4A16Linear._forward_fallback`,
    openpi/src/openpi/modules/w4a16_linear.py:256-268) in float64 accumulation:
    y = x @ dequant(W)^T (+ bias).  x: (M, K).  Returns float64 (M, N)."""
    w = dequantize(weight_packed, scales, layout, group_size).astype(np.float64)
    y = np.asarray(x, dtype=np.float64) @ w.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)
    return y


# --------------------------------------------------------------------------
# w4a16_plugin's CUDA quantiser / dequantiser (signed codes, byte packed)
# --------------------------------------------------------------------------

def plugin_quantize_int4(weight_bf16, group_size=128):
    """`quantizeToINT4Kernel` (openpi/w4a16_plugin/src/w4a16_gemm_kernel.cu:168-259).

    Per (row, group): scale = max|w|/7 + 1e-12 (fp32; stored as bf16), zero = 0;
    q = clamp(roundf(w / scale_fp32), -8, 7) (roundf = half away from zero);
    byte = (q0 & 0xF) | (q1 & 0xF) << 4, even k in the low nibble.
    Returns (packed int8 (N, K/2), scales bf16-valued f32 (N, K/g), zeros)."""
    w = round_to_bf16(weight_bf16)
    N, K = w.shape
    ng = K // group_size
    wg = w.reshape(N, ng, group_size)
    absmax = np.abs(wg).max(axis=2).astype(np.float32)
    scale = (absmax / np.float32(7.0) + np.float32(1e-12)).astype(np.float32)
    scaled = (wg / scale[:, :, None]).astype(np.float32)
    r = np.where(scaled >= 0, np.floor(scaled + np.float32(0.5)), np.ceil(scaled - np.float32(0.5)))
    # roundf() is exact half-away-from-zero; the +-0.5 form above can be off by one
    # ulp only when scaled+0.5 rounds up in fp32, i.e. for |scaled| >= 2**23: never here.
    q = np.clip(r, -8, 7).astype(np.int8).reshape(N, K)
    nib = (q.astype(np.uint8) & 0xF)
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8).view(np.int8)
    return packed, round_to_bf16(scale), np.zeros_like(scale)


def plugin_dequantize_int4(packed, scales, zeros, group_size=128):
    """`dequantizeINT4Kernel` (openpi/w4a16_plugin/src/w4a16_gemm_kernel.cu:281-308):
    sign-extended nibble * scale + zero in fp32, rounded to bf16."""
    p = np.asarray(packed).view(np.uint8)
    N, Kh = p.shape
    nib = np.empty((N, Kh * 2), dtype=np.int16)
    nib[:, 0::2] = p & 0xF
    nib[:, 1::2] = p >> 4
    q = np.where(nib >= 8, nib - 16, nib).astype(np.float32)
    s = np.repeat(np.asarray(scales, dtype=np.float32), group_size, axis=1)
    z = 0.0 if zeros is None else np.repeat(np.asarray(zeros, dtype=np.float32), group_size, axis=1)
    return round_to_bf16(q * s + z)


def plugin_gemm(x_bf16, packed, scales, zeros, group_size=128, alpha=1.0, beta=0.0, c=None):
    """`w4a16GemmForward` semantics (openpi/w4a16_plugin/src/w4a16_gemm_plugin.h:41-55):
    D = alpha * (A @ dequant(W)^T) + beta * C, fp32/64 accumulate."""
    w = plugin_dequantize_int4(packed, scales, zeros, group_size).astype(np.float64)
    y = alpha * (round_to_bf16(x_bf16).astype(np.float64) @ w.T)
    if c is not None and beta != 0.0:
        y = y + beta * np.asarray(c, dtype=np.float64)
    return y
