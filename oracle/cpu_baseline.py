"""The reference's CPU-runnable path for the NVFP4 / INT4 GEMV, in torch CPU ops, for timing.

Test infrastructure; see oracle/__init__.py.  Used by bench.py's cpu_baseline leg and by
`bench.py --impl reference` only.

Restates `NVFP4PackedLinear._forward_dequant_gemm`
(openpi/nvfp4_packed_plugin/python/nvfp4_packed.py:310-335): unpack both nibbles through the
16-entry table into an fp32 [N, K] matrix, expand the block scales with repeat, multiply,
then F.linear -- the weight is dequantised on EVERY call, as the reference does.  The INT4
path restates `W4A16Linear._dequantize_weights` + F.linear
(openpi/src/openpi/modules/w4a16_linear.py:174-199,256-268) in vectorised form.
"""
import torch
import torch.nn.functional as F

_TABLE = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def nvfp4_forward_dequant_gemm(x, weight_packed, weight_scales_f32, block_size, bias=None, activation=0):
    N, Kh = weight_packed.shape
    K = Kh * 2
    low = weight_packed & 0xF
    high = (weight_packed >> 4) & 0xF
    w = torch.zeros(N, K, dtype=torch.float32)
    w[:, 0::2] = _TABLE[low.long()]
    w[:, 1::2] = _TABLE[high.long()]
    s = weight_scales_f32.unsqueeze(-1).repeat(1, 1, block_size).view(N, -1)
    w = w * s
    out = F.linear(x, w.to(x.dtype), bias)
    if activation == 1:
        out = F.gelu(out, approximate="tanh")
    elif activation == 2:
        out = F.silu(out)
    return out


def int4_forward_dequant_gemm(x, words_rowmajor, scales, group_size):
    """words (N, K/8) int32, scales (N, K/group) fp16 -> x @ ((q - 8) * scale)^T in fp32."""
    N = words_rowmajor.shape[0]
    shifts = torch.arange(8, dtype=torch.int32) * 4
    q = ((words_rowmajor.unsqueeze(-1) >> shifts) & 0xF).reshape(N, -1).float()
    w = (q - 8.0) * scales.float().repeat_interleave(group_size, dim=1)
    return F.linear(x.float(), w)
