"""NVFP4 x NVFP4 (W4A4) linear layers for prefix-shaped GEMMs on the tcgen05 kernel.

Mirrors openpi/src/openpi/models_pytorch/nvfp4_mlp.py: quantize_to_nvfp4_sim (with the
MSE scale search used for weights), dequantize_nvfp4_sim, pack_nvfp4_data,
prepare_scales_for_cutlass -> prepare_scales, NVFP4Linear, NVFP4MLP.  The reference's
"simulation" forward (quantise activations per block, dequantise both sides with
E4M3-rounded scales, F.linear) is what the kernel computes, with the products and the
accumulation done by tcgen05.mma kind::mxf4nvf4 instead of a dequantised fp32 matmul.
"""
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from ._lib import ACT_GELU, ACT_NONE
from .nvfp4_packed import NVFP4_MAX, NVFP4_VALUES, _nearest_index, pack_nvfp4

BLOCK_SIZE = 32


def _quantize_block_with_scale(block, scale, values):
    scaled = (block / scale * NVFP4_MAX).clamp(-NVFP4_MAX, NVFP4_MAX)
    q = scaled.sign() * values[_nearest_index(scaled.abs())]
    return q * scale / NVFP4_MAX


def quantize_to_nvfp4_sim(tensor: torch.Tensor, block_size: int = BLOCK_SIZE, use_mse_search: bool = True,
                          mse_search_steps: int = 10) -> Tuple[torch.Tensor, torch.Tensor]:
    """[M, K] -> (values on the e2m1 grid [M, K], fp32 scale factors [M, K/block]).  With
    `use_mse_search` the block amplitude is searched over 0.7..1.0 x blockmax for the lowest
    squared error (offline, weights only)."""
    M, K = tensor.shape
    values = NVFP4_VALUES.to(tensor.device)
    nb = K // block_size
    t2 = tensor.reshape(M, nb, block_size).float().reshape(-1, block_size)
    block_max = t2.abs().amax(dim=-1, keepdim=True).clamp(min=1e-12)
    if use_mse_search:
        best_scales = block_max.clone()
        best_mse = torch.full((t2.shape[0],), float("inf"), device=tensor.device)
        for ratio in torch.linspace(0.7, 1.0, mse_search_steps, device=tensor.device):
            test = block_max * ratio
            mse = ((t2 - _quantize_block_with_scale(t2, test, values)) ** 2).sum(dim=-1)
            better = mse < best_mse
            best_mse = torch.where(better, mse, best_mse)
            best_scales = torch.where(better.unsqueeze(-1), test, best_scales)
        sf = (best_scales / NVFP4_MAX).reshape(M, nb)
    else:
        sf = (block_max / NVFP4_MAX).reshape(M, nb)
    se = sf.reshape(-1, 1)
    scaled = (t2 / (se * NVFP4_MAX).clamp(min=1e-12) * NVFP4_MAX).clamp(-NVFP4_MAX, NVFP4_MAX)
    q = (scaled.sign() * values[_nearest_index(scaled.abs())]).reshape(M, K).to(tensor.dtype)
    return q, sf


def dequantize_nvfp4_sim(quantized: torch.Tensor, scales: torch.Tensor, block_size: int = BLOCK_SIZE,
                         use_fp8_scales: bool = False) -> torch.Tensor:
    M, K = quantized.shape
    if use_fp8_scales:
        scales = scales.to(torch.float8_e4m3fn).to(torch.float32)
    return (quantized.reshape(M, -1, block_size) * scales.unsqueeze(-1)).reshape(M, K)


def pack_nvfp4_data(quantized: torch.Tensor, block_size: int = BLOCK_SIZE) -> torch.Tensor:
    return pack_nvfp4(quantized)


def prepare_scales(scales: torch.Tensor, block_size: int) -> torch.Tensor:
    """fp32 scales [rows, K/block] -> UE4M3 bytes per 16 elements in the kernel's atom layout
    (a block-32 scale covers two 16-blocks).  The counterpart of prepare_scales_for_cutlass."""
    s8 = scales.abs().clamp(max=448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    if block_size == 32:
        s8 = s8.repeat_interleave(2, dim=1)
    elif block_size != 16:
        raise ValueError("block size must be 16 or 32")
    return ops.swizzle_scales(s8.contiguous())


def _pad_rows_to_pitch(packed: torch.Tensor, K: int) -> torch.Tensor:
    pitch = ops.packed_pitch(K)
    if packed.shape[1] == pitch:
        return packed.contiguous()
    out = torch.zeros((packed.shape[0], pitch), dtype=torch.uint8, device=packed.device)
    out[:, :packed.shape[1]] = packed
    return out


class NVFP4Linear(nn.Module):
    """Linear layer with e2m1 weights AND e2m1 activations (both block-scaled).

    from_linear quantises the weight offline (MSE search, block `block_size`), packs it and
    lays its scales out for the kernel.  forward quantises the activations on the device
    (block 16, the kernel's native granularity) and runs the tensor-core GEMM.  Inputs are
    clamped to +-2688 as in the reference so that block scales stay inside E4M3.
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = False, block_size: int = BLOCK_SIZE,
                 activation: int = ACT_NONE):
        super().__init__()
        if in_features % 16 != 0 or out_features % 8 != 0:
            raise ValueError("in_features must be a multiple of 16 and out_features of 8")
        self.in_features = in_features
        self.out_features = out_features
        self.block_size = block_size
        self.activation = activation
        self.weight_scale_multiplier = 1.0   # scales are stored multiplied by this; alpha divides it out
        self.register_buffer("weight_packed", None)
        self.register_buffer("weight_scales_swizzled", None)
        self.register_buffer("weight_q", None)
        self.register_buffer("weight_scales", None)
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features))
        else:
            self.register_parameter("bias", None)

    @classmethod
    def from_linear(cls, linear: nn.Linear, block_size: int = BLOCK_SIZE, use_mse_search: bool = True,
                    keep_sim_weights: bool = False, scale_multiplier: float = 1.0,
                    activation: int = ACT_NONE) -> "NVFP4Linear":
        """`scale_multiplier` = 1 stores E4M3(scale) exactly as the reference does (small weight scales
        then fall into E4M3's subnormals); a power of two such as 256 keeps them in the normal range
        and is divided out through the GEMM's alpha."""
        layer = cls(linear.in_features, linear.out_features, linear.bias is not None, block_size, activation)
        with torch.no_grad():
            w = linear.weight.data.float()
            q, s = quantize_to_nvfp4_sim(w, block_size, use_mse_search=use_mse_search)
            layer.weight_scale_multiplier = float(scale_multiplier)
            layer.weight_packed = _pad_rows_to_pitch(pack_nvfp4_data(q), linear.in_features)
            layer.weight_scales_swizzled = prepare_scales(s * scale_multiplier, block_size)
            if keep_sim_weights:
                layer.weight_q, layer.weight_scales = q, s
            if linear.bias is not None:
                layer.bias.copy_(linear.bias)
        return layer.to(linear.weight.device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        batch_shape = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            x2 = x2.float()
        M = x2.shape[0]
        a, a_sf = ops.nvfp4_quantize_act(x2)
        out_dtype = torch.bfloat16 if x.dtype == torch.bfloat16 else torch.float32
        y = ops.nvfp4_gemm(a, a_sf, self.weight_packed, self.weight_scales_swizzled, M, self.out_features,
                           self.in_features, alpha=1.0 / self.weight_scale_multiplier,
                           bias=None if self.bias is None else self.bias.detach(), activation=self.activation,
                           out_dtype=out_dtype)
        return y.reshape(*batch_shape, self.out_features).to(x.dtype)


class NVFP4MLP(nn.Module):
    """down(gelu_tanh(gate(x)) * up(x)) with NVFP4Linear projections (Gemma's MLP)."""

    def __init__(self, hidden_size: int = 2048, intermediate_size: int = 16384, block_size: int = BLOCK_SIZE):
        super().__init__()
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.block_size = block_size
        self.gate_proj = NVFP4Linear(hidden_size, intermediate_size, False, block_size, ACT_GELU)
        self.up_proj = NVFP4Linear(hidden_size, intermediate_size, False, block_size)
        self.down_proj = NVFP4Linear(intermediate_size, hidden_size, False, block_size)

    @classmethod
    def from_gemma_mlp(cls, mlp: nn.Module, block_size: int = BLOCK_SIZE, use_mse_search: bool = True,
                       scale_multiplier: float = 1.0) -> "NVFP4MLP":
        layer = cls(mlp.gate_proj.in_features, mlp.gate_proj.out_features, block_size)
        layer.gate_proj = NVFP4Linear.from_linear(mlp.gate_proj, block_size, use_mse_search,
                                                  scale_multiplier=scale_multiplier, activation=ACT_GELU)
        layer.up_proj = NVFP4Linear.from_linear(mlp.up_proj, block_size, use_mse_search,
                                                scale_multiplier=scale_multiplier)
        layer.down_proj = NVFP4Linear.from_linear(mlp.down_proj, block_size, use_mse_search,
                                                  scale_multiplier=scale_multiplier)
        return layer

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(self.gate_proj(x) * self.up_proj(x))
