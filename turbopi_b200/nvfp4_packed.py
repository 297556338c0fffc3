"""NVFP4 weight-only host side: quantise / pack helpers and the drop-in modules.

Mirrors openpi/nvfp4_packed_plugin/python/nvfp4_packed.py (quantize_to_nvfp4,
pack_nvfp4, unpack_nvfp4, NVFP4PackedLinear, NVFP4PackedMLP,
replace_mlp_with_nvfp4_packed) with the GEMV served by tpb200_nvfp4_gemv.

Two weight formats are carried:
  "ref"   block 32, fp32 scale per block               (the reference's buffers)
  "nvfp4" block 16, E4M3 scale per block + fp32 global (standard NVFP4; what the
          prefix tensor-core GEMM consumes as well)
"""
from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import ops
from ._lib import ACTIVATIONS

BLOCK_SIZE = 32
NVFP4_MAX = 6.0
E4M3_MAX = 448.0
NVFP4_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
_THRESHOLDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])


def _nearest_index(abs_vals: torch.Tensor) -> torch.Tensor:
    """Index of the nearest e2m1 magnitude; an exact midpoint goes to the lower one
    (same choice as argmin over |a - v|)."""
    return torch.bucketize(abs_vals, _THRESHOLDS.to(abs_vals.device), right=False)


def quantize_to_nvfp4(tensor: torch.Tensor, block_size: int = BLOCK_SIZE) -> Tuple[torch.Tensor, torch.Tensor]:
    """[M, K] -> (values on the e2m1 grid [M, K] fp32, scales [M, K/block] fp32);
    scale = blockmax / 6 (blockmax clamped at 1e-12)."""
    M, K = tensor.shape
    vals = NVFP4_VALUES.to(tensor.device)
    tb = tensor.reshape(M, K // block_size, block_size).float()
    block_max = tb.abs().amax(dim=-1, keepdim=True).clamp(min=1e-12)
    scale = block_max / NVFP4_MAX
    scaled = (tb / block_max * NVFP4_MAX).clamp(-NVFP4_MAX, NVFP4_MAX)
    q = scaled.sign() * vals[_nearest_index(scaled.abs())]
    return q.reshape(M, K), scale.squeeze(-1)


def pack_nvfp4(quantized: torch.Tensor) -> torch.Tensor:
    """values on the e2m1 grid [N, K] -> [N, K/2] uint8, even k in the low nibble;
    code = (v < 0) << 3 | index(|v|)."""
    sign = (quantized < 0).to(torch.uint8) << 3
    enc = sign | _nearest_index(quantized.abs()).to(torch.uint8)
    return (enc[:, 0::2] | (enc[:, 1::2] << 4)).to(torch.uint8)


def unpack_nvfp4(packed: torch.Tensor, N: int, K: int) -> torch.Tensor:
    table = torch.cat([NVFP4_VALUES, -NVFP4_VALUES]).to(packed.device)
    out = torch.empty(N, K, device=packed.device, dtype=torch.float32)
    out[:, 0::2] = table[(packed & 0xF).long()]
    out[:, 1::2] = table[(packed >> 4).long()]
    return out


def quantize_nvfp4_two_level(weight: torch.Tensor, block_size: int = 16):
    """Standard NVFP4: global = max|w| / (6*448); block scale = E4M3(blockmax / 6 / global);
    codes chosen against the DECODED block scale.  Returns (packed [N, K/2] uint8,
    scales [N, K/block] uint8 (E4M3 bytes), global_scale float)."""
    w = weight.detach().float()
    N, K = w.shape
    amax = w.abs().max().clamp(min=1e-12)
    g = (amax / (NVFP4_MAX * E4M3_MAX)).item()
    g = float(torch.tensor(g, dtype=torch.float32))
    wb = w.reshape(N, K // block_size, block_size)
    bmax = wb.abs().amax(dim=2)
    s8 = (bmax / NVFP4_MAX / g).clamp(max=E4M3_MAX).to(torch.float8_e4m3fn)
    s = s8.float() * g
    s_safe = torch.where(s == 0, torch.ones_like(s), s)
    scaled = wb / s_safe.unsqueeze(2)
    idx = _nearest_index(scaled.abs().clamp(max=NVFP4_MAX)).to(torch.uint8)
    codes = torch.where(scaled < 0, idx | 0x8, idx).reshape(N, K)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).to(torch.uint8)
    return packed, s8.view(torch.uint8), g


class NVFP4PackedLinear(nn.Module):
    """Linear layer over packed e2m1 weights with fused bias + GELU-tanh / SiLU.

    Buffers follow the reference: weight_packed [N, K/2] uint8 and weight_scales
    [N, K/block] (fp32 for the "ref" format, uint8 E4M3 bytes + `global_scale` for
    "nvfp4").  forward() accepts any leading shape; rows go through the kernel 16
    at a time.  There is no dequantise-and-matmul path.
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = False, block_size: int = BLOCK_SIZE,
                 activation: str = "none"):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.block_size = block_size
        self.activation = activation
        self.global_scale = 1.0
        self.register_buffer("weight_packed", None)
        self.register_buffer("weight_scales", None)
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features))
        else:
            self.register_parameter("bias", None)

    @classmethod
    def from_linear(cls, linear: nn.Linear, block_size: int = BLOCK_SIZE, activation: str = "none",
                    fmt: str = "ref") -> "NVFP4PackedLinear":
        if fmt == "nvfp4":
            block_size = 16
        layer = cls(linear.in_features, linear.out_features, bias=linear.bias is not None, block_size=block_size,
                    activation=activation)
        with torch.no_grad():
            w = linear.weight.data
            if fmt == "ref":
                q, s = quantize_to_nvfp4(w, block_size)
                layer.weight_packed = pack_nvfp4(q)
                layer.weight_scales = s
            elif fmt == "nvfp4":
                layer.weight_packed, layer.weight_scales, layer.global_scale = quantize_nvfp4_two_level(w, 16)
            else:
                raise ValueError(f"unknown format {fmt!r}")
            if linear.bias is not None:
                layer.bias.copy_(linear.bias)
        return layer.to(linear.weight.device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        batch_shape = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            x2 = x2.float()
        x2 = x2.contiguous()
        T = x2.shape[0]
        out = torch.empty((T, self.out_features), dtype=x2.dtype, device=x2.device)
        act = ACTIVATIONS.get(self.activation, 0)
        bias = None if self.bias is None else self.bias.detach().float().contiguous()
        for t0 in range(0, T, 16):
            t1 = min(T, t0 + 16)
            ops.nvfp4_gemv_out(x2[t0:t1], self.weight_packed, self.weight_scales, out[t0:t1], bias, act,
                               self.block_size, self.global_scale)
        return out.reshape(*batch_shape, self.out_features).to(x.dtype)

    @property
    def weight(self) -> torch.Tensor:
        """Placeholder for code that only looks at `.weight.dtype` / `.device`."""
        return torch.empty(1, dtype=torch.bfloat16, device=self.weight_packed.device)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None}, activation={self.activation}")


class NVFP4PackedMLP(nn.Module):
    """Gated MLP down(act(gate(x)) * up(x)).  `gate_activation` defaults to the
    reference module's 'silu'; Gemma's own MLP uses 'gelu' (tanh form)."""

    def __init__(self, hidden_size: int, intermediate_size: int, block_size: int = BLOCK_SIZE,
                 gate_activation: str = "silu"):
        super().__init__()
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.block_size = block_size
        self.gate_proj = NVFP4PackedLinear(hidden_size, intermediate_size, False, block_size, gate_activation)
        self.up_proj = NVFP4PackedLinear(hidden_size, intermediate_size, False, block_size, "none")
        self.down_proj = NVFP4PackedLinear(intermediate_size, hidden_size, False, block_size, "none")

    @classmethod
    def from_gemma_mlp(cls, mlp: nn.Module, block_size: int = BLOCK_SIZE, gate_activation: str = "silu",
                       fmt: str = "ref") -> "NVFP4PackedMLP":
        layer = cls(mlp.gate_proj.in_features, mlp.gate_proj.out_features, block_size, gate_activation)
        layer.gate_proj = NVFP4PackedLinear.from_linear(mlp.gate_proj, block_size, gate_activation, fmt)
        layer.up_proj = NVFP4PackedLinear.from_linear(mlp.up_proj, block_size, "none", fmt)
        layer.down_proj = NVFP4PackedLinear.from_linear(mlp.down_proj, block_size, "none", fmt)
        return layer

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(self.gate_proj(x) * self.up_proj(x))


def replace_mlp_with_nvfp4_packed(model, block_size: int = BLOCK_SIZE, target_layers: Optional[list] = None,
                                  gate_activation: str = "silu") -> int:
    """Swap every `layer.mlp` of model.paligemma_with_expert.paligemma.language_model for an
    NVFP4PackedMLP; returns the number replaced."""
    try:
        lm = model.paligemma_with_expert.paligemma.language_model
    except AttributeError:
        return 0
    count = 0
    for idx, layer in enumerate(lm.layers):
        if target_layers is not None and idx not in target_layers:
            continue
        if getattr(layer, "mlp", None) is not None:
            device = next(layer.mlp.parameters()).device
            layer.mlp = NVFP4PackedMLP.from_gemma_mlp(layer.mlp, block_size, gate_activation).to(device)
            count += 1
    return count
