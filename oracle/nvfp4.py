"""NVFP4 (e2m1, block-scaled) oracle: quantisers, packers, dequant-then-matmul.

Test infrastructure; see oracle/__init__.py.
"""
import numpy as np

from .formats import (E2M1_LUT, E2M1_MAGNITUDES, E2M1_MAX, E4M3_MAX, e2m1_nearest_index, e4m3_decode,
                      e4m3_encode, round_to_bf16, round_to_e4m3)

BLOCK_SIZE = 32  # openpi/nvfp4_packed_plugin/python/nvfp4_packed.py:29


# --------------------------------------------------------------------------
# nvfp4_packed_plugin (python)
# --------------------------------------------------------------------------

def quantize_to_nvfp4(tensor, block_size=BLOCK_SIZE):
    """`quantize_to_nvfp4` (openpi/nvfp4_packed_plugin/python/nvfp4_packed.py:81-118).

    block_max = max|x| clamped >= 1e-12; scale = block_max / 6;
    scaled = x / block_max * 6 (in that order, fp32), clamped to +-6;
    value = sign(scaled) * nearest magnitude (ties -> lower).
    Returns (quantized values fp32 (M, K), scales fp32 (M, K/block))."""
    x = np.asarray(tensor, dtype=np.float32)
    M, K = x.shape
    nb = K // block_size
    xb = x.reshape(M, nb, block_size)
    block_max = np.maximum(np.abs(xb).max(axis=-1, keepdims=True), np.float32(1e-12)).astype(np.float32)
    scales = (block_max / np.float32(E2M1_MAX)).astype(np.float32)
    scaled = (xb / block_max * np.float32(E2M1_MAX)).astype(np.float32)
    scaled = np.clip(scaled, -E2M1_MAX, E2M1_MAX)
    idx = e2m1_nearest_index(np.abs(scaled))
    q = np.sign(scaled).astype(np.float32) * E2M1_MAGNITUDES[idx]
    return q.reshape(M, K).astype(np.float32), scales[..., 0]


def pack_nvfp4(quantized):
    """`pack_nvfp4` (openpi/nvfp4_packed_plugin/python/nvfp4_packed.py:121-146):
    code = (q < 0) << 3 | index(|q|); byte = even k | odd k << 4.  -0.0 < 0 is
    False, so code 8 is never emitted."""
    q = np.asarray(quantized, dtype=np.float32)
    signs = (q < 0).astype(np.uint8) << 3
    idx = e2m1_nearest_index(np.abs(q))
    enc = signs | idx
    return (enc[:, 0::2] | (enc[:, 1::2] << 4)).astype(np.uint8)


def unpack_codes(packed):
    p = np.asarray(packed, dtype=np.uint8)
    N, Kh = p.shape
    codes = np.empty((N, Kh * 2), dtype=np.uint8)
    codes[:, 0::2] = p & 0xF
    codes[:, 1::2] = p >> 4
    return codes


def unpack_nvfp4(packed):
    """`unpack_nvfp4` (openpi/nvfp4_packed_plugin/python/nvfp4_packed.py:149-163)."""
    return E2M1_LUT[unpack_codes(packed)]


def dequantize(packed, scales, block_size=BLOCK_SIZE, global_scale=1.0, scale_is_e4m3=False):
    """value[n,k] = LUT[code] * scale[n, k/block] (* global scale), fp32
    (openpi/nvfp4_packed_plugin/python/nvfp4_packed.py:316-324)."""
    vals = unpack_nvfp4(packed)
    s = e4m3_decode(scales) if scale_is_e4m3 else np.asarray(scales, dtype=np.float32)
    s = np.repeat(s, block_size, axis=1)
    return (vals * s * np.float32(global_scale)).astype(np.float32)


def gelu_tanh(x):
    """openpi/nvfp4_packed_plugin/src/nvfp4_packed_kernel.cu:70-76 == F.gelu(approximate='tanh')."""
    x = np.asarray(x, dtype=np.float64)
    return 0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def silu(x):
    """openpi/nvfp4_packed_plugin/src/nvfp4_packed_kernel.cu:79-81."""
    x = np.asarray(x, dtype=np.float64)
    return x / (1.0 + np.exp(-x))


def gemv_dequant_matmul(x, packed, scales, bias=None, activation=0, block_size=BLOCK_SIZE,
                        global_scale=1.0, scale_is_e4m3=False):
    """`NVFP4PackedLinear._forward_dequant_gemm`
    (openpi/nvfp4_packed_plugin/python/nvfp4_packed.py:310-335): dequantise, F.linear,
    then GELU-tanh (1) / SiLU (2).  float64 accumulation.  x: (M, K)."""
    w = dequantize(packed, scales, block_size, global_scale, scale_is_e4m3).astype(np.float64)
    y = np.asarray(x, dtype=np.float64) @ w.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)
    if activation == 1:
        y = gelu_tanh(y)
    elif activation == 2:
        y = silu(y)
    return y


# --------------------------------------------------------------------------
# kv_fuse_plugin (python)
# --------------------------------------------------------------------------

def kv_fuse_quantize_to_fp4(tensor, block_size=BLOCK_SIZE):
    """`quantize_to_fp4` (openpi/kv_fuse_plugin/python/kv_fuse.py:72-119):
    abs_max clamped >= 1e-8; scale = abs_max / 6; normalised = x / scale;
    sign from the INPUT (x < 0), index = nearest magnitude (no clamp needed).
    Returns (packed uint8 (N, K/2), scales fp32 (N, K/block))."""
    x = np.asarray(tensor, dtype=np.float32)
    N, K = x.shape
    nb = K // block_size
    xb = x.reshape(N, nb, block_size)
    abs_max = np.maximum(np.abs(xb).max(axis=-1, keepdims=True), np.float32(1e-8)).astype(np.float32)
    scales = (abs_max / np.float32(E2M1_MAX)).astype(np.float32)
    norm = (xb / scales).astype(np.float32).reshape(-1)
    signs = (norm < 0).astype(np.uint8)
    idx = e2m1_nearest_index(np.abs(norm))
    q = (idx + signs * 8).reshape(N, K).astype(np.uint8)
    packed = ((q[:, 0::2] & 0xF) | ((q[:, 1::2] & 0xF) << 4)).astype(np.uint8)
    return packed, scales[..., 0].astype(np.float32)


# --------------------------------------------------------------------------
# w4a8_plugin weight quantiser (CUDA): E4M3 scale per 16, transposed output
# --------------------------------------------------------------------------

def plugin_quantize_weight_nvfp4(weight_bf16):
    """`quantizeWeightToNVFP4Kernel` (openpi/w4a8_plugin/src/w4a8_gemm_kernel.cu:314-412).

    Per (row n, 16-block): scale = max|w|/6 + 1e-12 in fp32; the stored scale is
    that value rounded to E4M3 (satfinite) at [block, n]; the codes come from
    w / scale_fp32 (the UNROUNDED scale, as the kernel does), sign = scaled < 0,
    nearest magnitude with ties to the lower index; packed transposed [K/2, N].
    Returns (packed uint8 (K/2, N), scales E4M3 bytes (K/16, N))."""
    w = round_to_bf16(weight_bf16)
    N, K = w.shape
    nb = K // 16
    wb = w.reshape(N, nb, 16)
    block_max = np.abs(wb).max(axis=2).astype(np.float32)
    scale = (block_max / np.float32(6.0) + np.float32(1e-12)).astype(np.float32)
    scaled = (wb / scale[:, :, None]).astype(np.float32)
    idx = e2m1_nearest_index(np.abs(scaled))
    codes = np.where(scaled < 0, idx | 0x8, idx).astype(np.uint8).reshape(N, K)
    packed_nk = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)  # (N, K/2)
    return np.ascontiguousarray(packed_nk.T), np.ascontiguousarray(e4m3_encode(scale).T)


# --------------------------------------------------------------------------
# NVFP4 "standard" two-level quantisation used by the benchmark configurations:
# E4M3 scale per 16 elements and one fp32 global scale
# --------------------------------------------------------------------------

def quantize_two_level(weight, block_size=16):
    """global = max|w| / (6 * 448); block scale = E4M3(blockmax / 6 / global);
    codes = nearest e2m1 of w / (decoded block scale * global), sign from the
    input, ties to the lower magnitude, |.| clamped to 6.
    Follows the scale recipe of openpi/src/openpi/models_pytorch/nvfp4_mlp.py:129,158
    with the E4M3 rounding of :211-212 applied before the codes are chosen.
    Returns (packed (N, K/2) uint8, scales (N, K/bs) E4M3 bytes, global fp32)."""
    w = np.asarray(weight, dtype=np.float32)
    N, K = w.shape
    amax = np.float32(max(float(np.abs(w).max()), 1e-12))
    g = np.float32(amax / np.float32(E2M1_MAX * E4M3_MAX))
    wb = w.reshape(N, K // block_size, block_size)
    bmax = np.abs(wb).max(axis=2).astype(np.float32)
    sbytes = e4m3_encode(bmax / np.float32(E2M1_MAX) / g)
    s = e4m3_decode(sbytes) * g
    s_safe = np.where(s == 0, np.float32(1.0), s).astype(np.float32)
    scaled = (wb / s_safe[:, :, None]).astype(np.float32)
    idx = e2m1_nearest_index(np.minimum(np.abs(scaled), np.float32(E2M1_MAX)))
    codes = np.where(scaled < 0, idx | 0x8, idx).astype(np.uint8).reshape(N, K)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return packed, sbytes, g


# --------------------------------------------------------------------------
# nvfp4_mlp.py simulation path (prefix GEMM oracle)
# --------------------------------------------------------------------------

def _quantize_block_with_scale(block, scale):
    """openpi/src/openpi/models_pytorch/nvfp4_mlp.py:56-85 (`scale` is the block
    amplitude that maps to 6)."""
    scaled = (block / scale * np.float32(E2M1_MAX)).astype(np.float32)
    scaled = np.clip(scaled, -E2M1_MAX, E2M1_MAX)
    idx = e2m1_nearest_index(np.abs(scaled))
    qs = np.sign(scaled).astype(np.float32) * E2M1_MAGNITUDES[idx]
    return (qs * scale / np.float32(E2M1_MAX)).astype(np.float32)


def quantize_to_nvfp4_sim(tensor, block_size=BLOCK_SIZE, use_mse_search=True, mse_search_steps=10):
    """`quantize_to_nvfp4_sim(use_triton=False)`
    (openpi/src/openpi/models_pytorch/nvfp4_mlp.py:88-173).
    Returns (quantized values fp32 (M, K) in e2m1 units, scale factors fp32 (M, K/block))."""
    x = np.asarray(tensor, dtype=np.float32)
    M, K = x.shape
    nb = K // block_size
    t2 = x.reshape(-1, block_size)
    block_max = np.maximum(np.abs(t2).max(axis=-1, keepdims=True), np.float32(1e-12)).astype(np.float32)
    if use_mse_search:
        best_scales = block_max.copy()
        best_mse = np.full((t2.shape[0],), np.inf, dtype=np.float32)
        # torch.linspace(0.7, 1.0, steps) in fp32
        steps = mse_search_steps
        ratios = _torch_linspace_f32(0.7, 1.0, steps)
        for r in ratios:
            test_scale = (block_max * r).astype(np.float32)
            qt = _quantize_block_with_scale(t2, test_scale)
            mse = ((t2 - qt) ** 2).sum(axis=-1, dtype=np.float32)
            better = mse < best_mse
            best_mse = np.where(better, mse, best_mse)
            best_scales = np.where(better[:, None], test_scale, best_scales)
        sf = (best_scales / np.float32(E2M1_MAX)).reshape(M, nb).astype(np.float32)
    else:
        sf = (block_max / np.float32(E2M1_MAX)).reshape(M, nb).astype(np.float32)
    se = sf.reshape(-1, 1)
    denom = np.maximum(se * np.float32(E2M1_MAX), np.float32(1e-12)).astype(np.float32)
    scaled = (t2 / denom * np.float32(E2M1_MAX)).astype(np.float32)
    scaled = np.clip(scaled, -E2M1_MAX, E2M1_MAX)
    idx = e2m1_nearest_index(np.abs(scaled))
    q = (np.sign(scaled).astype(np.float32) * E2M1_MAGNITUDES[idx]).reshape(M, K)
    return q.astype(np.float32), sf


def _torch_linspace_f32(start, end, steps):
    """torch.linspace in float32: symmetric evaluation from both ends
    (step = (end-start)/(steps-1); first half start + i*step, second half
    end - (steps-1-i)*step), all in fp32."""
    start = np.float32(start)
    end = np.float32(end)
    step = np.float32((end - start) / np.float32(steps - 1))
    out = np.empty(steps, dtype=np.float32)
    half = steps // 2
    for i in range(steps):
        if i < half:
            out[i] = np.float32(start + np.float32(step * np.float32(i)))
        else:
            out[i] = np.float32(end - np.float32(step * np.float32(steps - 1 - i)))
    return out


def dequantize_nvfp4_sim(quantized, scales, block_size=BLOCK_SIZE, use_fp8_scales=False):
    """`dequantize_nvfp4_sim(use_triton=False)`
    (openpi/src/openpi/models_pytorch/nvfp4_mlp.py:176-217)."""
    q = np.asarray(quantized, dtype=np.float32)
    M, K = q.shape
    s = np.asarray(scales, dtype=np.float32)
    if use_fp8_scales:
        s = round_to_e4m3(s)
    return (q.reshape(M, -1, block_size) * s[:, :, None]).reshape(M, K).astype(np.float32)


def pack_nvfp4_data(quantized):
    """`pack_nvfp4_data` (openpi/src/openpi/models_pytorch/nvfp4_mlp.py:400-436)."""
    return pack_nvfp4(quantized)


def linear_sim(x, w_q, w_scales, block_size=BLOCK_SIZE, bias=None, quantize_act=True):
    """`NVFP4Linear._forward_simulation` (openpi/src/openpi/models_pytorch/nvfp4_mlp.py:597-634):
    clamp x to +-2688, quantise it per block (no MSE search), dequantise both sides
    with E4M3-rounded scales, F.linear.  `quantize_act=False` gives the weight-only
    variant (bf16 activations untouched).  float64 accumulation."""
    x = np.asarray(x, dtype=np.float32)
    if quantize_act:
        lim = np.float32(E4M3_MAX * E2M1_MAX)
        xc = np.clip(x, -lim, lim)
        xq, xs = quantize_to_nvfp4_sim(xc, block_size, use_mse_search=False)
        xd = dequantize_nvfp4_sim(xq, xs, block_size, use_fp8_scales=True)
    else:
        xd = x
    wd = dequantize_nvfp4_sim(w_q, w_scales, block_size, use_fp8_scales=True)
    y = xd.astype(np.float64) @ wd.astype(np.float64).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)
    return y


def swizzle_scales_128x4(scales_bytes, kb_multiple=4):
    """Scale-factor bytes (rows, kblocks) -> the 128-row x 4-k-block interleaved atom
    order described in openpi/src/openpi/models_pytorch/nvfp4_mlp.py:224-288: rows
    padded to 128, k-blocks to 4; tile order (k-tile outer... see below), inside a
    tile 32 row-groups x 4 rows-of-32 x 4 k-blocks -> byte offset
    (r % 32) * 16 + (r // 32) * 4 + kb.

    Tiles are laid out row-tile major, k-tile minor (each tile 512 bytes), which
    is the order the tcgen05 scale-factor copy consumes them in.  `kb_multiple`
    pads the k-blocks (16 for the GEMM, whose K stage is 256 elements)."""
    s = np.asarray(scales_bytes, dtype=np.uint8)
    R, KB = s.shape
    Rp = (R + 127) // 128 * 128
    Kp = (KB + kb_multiple - 1) // kb_multiple * kb_multiple
    pad = np.zeros((Rp, Kp), dtype=np.uint8)
    pad[:R, :KB] = s
    t = pad.reshape(Rp // 128, 4, 32, Kp // 4, 4)      # [rt, r//32, r%32, kt, kb]
    t = t.transpose(0, 3, 2, 1, 4)                      # [rt, kt, r%32, r//32, kb]
    return np.ascontiguousarray(t).reshape(-1)
