"""INT4 (W4A16) host side: weight packers and the drop-in Linear.

Mirrors the interface of the reference's
  openpi/src/openpi/utils/w4a16_packer.py   (PackedWeight, W4A16Packer, W4A16PackerFast)
  openpi/src/openpi/modules/w4a16_linear.py (W4A16Linear)
with the GEMV served by the sm_100a kernel (tpb200_w4a16_gemv) for up to 16 tokens
per launch.  Packing runs on whatever device the weight is on, in torch ops.
"""
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import ops
from ._lib import INT4_KBLOCK, INT4_ROWMAJOR

QUANT_BLOCK = 32
INT4_OFFSET = 8
INT4_RANGE = 7


@dataclass
class PackedWeight:
    weight_packed: torch.Tensor            # (K/32, N, 4) int32
    scales: torch.Tensor                   # (K/32, N) float16
    original_shape: Tuple[int, int]        # (N, K)


def _codes_to_words(codes: torch.Tensor) -> torch.Tensor:
    """(N, K) codes 0..15 -> (N, K/8) int32 words, code i of a word at bits 4i."""
    N, K = codes.shape
    c = codes.reshape(N, K // 8, 8).to(torch.int64)
    shifts = torch.arange(8, device=codes.device, dtype=torch.int64) * 4
    words = (c << shifts).sum(dim=2)                       # 0 .. 2**32-1
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    return words.to(torch.int32)


def _quantize_codes(weight: torch.Tensor, block: int, scale_first_to_fp16: bool):
    w = weight.detach().float()
    N, K = w.shape
    if K % block != 0:
        raise ValueError(f"in_features ({K}) must be divisible by the quantisation block ({block})")
    wb = w.reshape(N, K // block, block)
    amax = wb.abs().amax(dim=2)
    if scale_first_to_fp16:
        # W4A16Packer: scale rounded to fp16 before the division, zero -> 1.0 (w4a16_packer.py:149-160)
        scales = (amax / INT4_RANGE).to(torch.float16)
        scales = torch.where(scales == 0, torch.ones_like(scales), scales)
        q = torch.round(wb / scales.float().unsqueeze(2) + INT4_OFFSET)
    else:
        # W4A16PackerFast: fp32 scale clamped at 1e-8, fp16 only when stored (w4a16_packer.py:331-338,356)
        scales32 = (amax / INT4_RANGE).clamp(min=1e-8)
        q = torch.round(wb / scales32.unsqueeze(2) + INT4_OFFSET)
        scales = scales32.to(torch.float16)
    codes = q.clamp(0, 15).to(torch.uint8).reshape(N, K)
    return codes, scales


class W4A16PackerFast:
    """Vectorised packer (the one W4A16Linear uses)."""

    def __init__(self, block_size: int = QUANT_BLOCK):
        self.block_size = block_size

    def pack(self, weight: torch.Tensor, device: Optional[torch.device] = None) -> PackedWeight:
        assert weight.dim() == 2, "Weight must be 2D"
        N, K = weight.shape
        codes, scales = _quantize_codes(weight, self.block_size, scale_first_to_fp16=False)
        words = _codes_to_words(codes)                                    # (N, K/8)
        packed = words.reshape(N, K // 32, 4).permute(1, 0, 2).contiguous()
        device = device or weight.device
        return PackedWeight(packed.to(device), scales.t().contiguous().to(device), (N, K))

    def pack_rowmajor(self, weight: torch.Tensor, group_size: int = 128):
        """(N, K/8) int32 words + (N, K/group) fp16 scales: the row-major layout of the
        sm_100a GEMV (same codes and nibble order, no K-block interleave)."""
        codes, scales = _quantize_codes(weight, group_size, scale_first_to_fp16=False)
        return _codes_to_words(codes), scales.contiguous()


class W4A16Packer(W4A16PackerFast):
    """The reference's basic packer: identical layout; the scale is rounded to fp16
    before the codes are computed."""

    def pack(self, weight: torch.Tensor, device: Optional[torch.device] = None) -> PackedWeight:
        assert weight.dim() == 2, "Weight must be 2D"
        N, K = weight.shape
        codes, scales = _quantize_codes(weight, self.block_size, scale_first_to_fp16=True)
        packed = _codes_to_words(codes).reshape(N, K // 32, 4).permute(1, 0, 2).contiguous()
        device = device or weight.device
        return PackedWeight(packed.to(device), scales.t().contiguous().to(device), (N, K))

    def unpack(self, packed: PackedWeight) -> torch.Tensor:
        return dequantize_kblock(packed.weight_packed, packed.scales)

    def verify(self, original: torch.Tensor, packed: PackedWeight, rtol: float = 0.1, atol: float = 0.1):
        un = self.unpack(packed).float().cpu()
        orig = original.float().cpu()
        cos = torch.nn.functional.cosine_similarity(orig.flatten()[None], un.flatten()[None]).item()
        return torch.allclose(orig, un, rtol=rtol, atol=atol), cos


def pack_linear_weight(weight: torch.Tensor, device: Optional[torch.device] = None) -> PackedWeight:
    return W4A16Packer().pack(weight, device)


def dequantize_kblock(weight_packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """(K/32, N, 4) words + (K/32, N) scales -> (N, K) fp16, ((q - 8) * scale)."""
    nb, N, _ = weight_packed.shape
    words = weight_packed.permute(1, 0, 2).reshape(N, nb * 4).to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(8, device=words.device, dtype=torch.int64) * 4
    codes = ((words.unsqueeze(2) >> shifts) & 0xF).reshape(N, nb * 32).float()
    s = scales.t().float().repeat_interleave(32, dim=1)
    return ((codes - 8.0) * s).to(torch.float16)


class W4A16Linear(nn.Module):
    """nn.Linear replacement with INT4 weights.

    Buffers: weight_packed (K/32, N, 4) int32, scales (K/32, N) fp16 -- the reference's state-dict
    format.  forward() dispatches on the token count: up to 16 tokens run on the decode GEMV, more on
    the tensor-core GEMM that dequantises the same buffers to bf16 inside the kernel (one launch for any
    number of tokens; needs in_features % 128 == 0 and out_features % 8 == 0, otherwise the GEMV runs 16
    rows at a time).  Unlike the reference there is no dequantise-and-F.linear path, so a CUDA device
    is required.
    """

    __constants__ = ["in_features", "out_features"]

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None):
        super().__init__()
        assert in_features % QUANT_BLOCK == 0, f"in_features ({in_features}) must be divisible by {QUANT_BLOCK}"
        self.in_features = in_features
        self.out_features = out_features
        self.num_scale_blocks = in_features // QUANT_BLOCK
        self.register_buffer("weight_packed",
                             torch.zeros(self.num_scale_blocks, out_features, 4, dtype=torch.int32, device=device))
        self.register_buffer("scales",
                             torch.zeros(self.num_scale_blocks, out_features, dtype=torch.float16, device=device))
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device))
        else:
            self.register_parameter("bias", None)
        self._packer = W4A16PackerFast()
        self._original_dtype = dtype or torch.bfloat16

    @property
    def weight(self) -> torch.Tensor:
        """Dequantised fp16 weight, for code that inspects `.weight` (dtype checks, debugging)."""
        return dequantize_kblock(self.weight_packed, self.scales)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        *batch_dims, K = input.shape
        assert K == self.in_features, f"Input last dim ({K}) doesn't match in_features ({self.in_features})"
        x = input.reshape(-1, K)
        if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            x = x.float()
        x = x.contiguous()
        T = x.shape[0]
        out = torch.empty((T, self.out_features), dtype=input.dtype if input.dtype in (
            torch.float16, torch.bfloat16, torch.float32) else torch.float32, device=input.device)
        bias = None if self.bias is None else self.bias.detach().contiguous()
        if bias is not None and bias.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            bias = bias.float()
        if T > 16 and K % 128 == 0 and self.out_features % 8 == 0:
            ops.w4a16_gemm(x, self.weight_packed, self.scales, None, bias, out, INT4_KBLOCK)
            return out.reshape(*batch_dims, self.out_features)
        for t0 in range(0, T, 16):
            t1 = min(T, t0 + 16)
            ops.w4a16_gemv_out(x[t0:t1], self.weight_packed, self.scales, out[t0:t1], bias, 32, INT4_KBLOCK)
        return out.reshape(*batch_dims, self.out_features)

    def pack_weights(self, weight: torch.Tensor) -> None:
        packed = self._packer.pack(weight, device=self.weight_packed.device)
        self.weight_packed.copy_(packed.weight_packed)
        self.scales.copy_(packed.scales)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        # accept an unpacked `weight` and quantise it on load (w4a16_linear.py:286-327)
        key = prefix + "weight"
        if key in state_dict:
            self.pack_weights(state_dict.pop(key))
            for k in (prefix + "weight_packed", prefix + "scales"):
                state_dict.setdefault(k, getattr(self, k[len(prefix):]))
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                      error_msgs)

    @classmethod
    def from_linear(cls, linear: nn.Linear, device=None) -> "W4A16Linear":
        device = device or linear.weight.device
        layer = cls(linear.in_features, linear.out_features, bias=linear.bias is not None, device=device,
                    dtype=linear.weight.dtype)
        layer.pack_weights(linear.weight)
        if linear.bias is not None:
            layer.bias.data.copy_(linear.bias.data)
        return layer

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None}, quant=INT4")
