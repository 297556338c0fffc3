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

from . import _lib, ops
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


def _operand_buffer(module, T, K, device):
    """The tiled A operand of `module`'s GEMM for T tokens, kept on the module: allocating (and zero-filling) 3 x T x K / 2
    bytes per call costs more than the quantiser that fills them.  Padding rows and columns are never written, so
    they stay zero from one call to the next.  (Calls on one module are expected in stream order, as with any
    module that owns scratch.)"""
    cache = module.__dict__.setdefault("_operands", {})
    key = (int(T), int(K), str(device))
    q = cache.get(key)
    if q is None:
        if len(cache) >= 4:
            cache.clear()
        q = cache[key] = ops.QuantBuf(T, K, 3, device)
    return q


def _split_k_scratch(module, T, N, K, device):
    """Zeroed split-K scratch of `module`'s GEMM, as large as the launch planner wants for T tokens (a scratch
    that is too small makes the planner cut K less and leaves SMs idle: 712 x 2048 x 16384 runs on 48 CTAs
    without it).  Grown when a larger token count arrives; owned by the module, so calls on different modules
    never share counters."""
    need = ops.nvfp4_gemm_workspace_size(T, N, K, 3, ops.OPERANDS_TILED)
    ws = module.__dict__.get("_gemm_ws")
    if ws is None or ws.numel() < need or ws.device != torch.device(device):
        ws = module.__dict__["_gemm_ws"] = ops.gemm_workspace(device, max(int(need), 1 << 20))
    return ws


class NVFP4PackedLinear(nn.Module):
    """Linear layer over packed e2m1 weights with fused bias + GELU-tanh / SiLU.

    Buffers follow the reference: weight_packed [N, K/2] uint8 and weight_scales
    [N, K/block] (fp32 for the "ref" format, uint8 E4M3 bytes + `global_scale` for
    "nvfp4").  forward() accepts any leading shape and dispatches on the token count:

      "nvfp4" weights   <= 4 tokens: the CUDA-core GEMV on the packed rows as stored; 5..16 tokens: one
                        tensor-core GEMV launch behind a quantiser launch; more tokens: the tcgen05
                        block-scaled GEMM on the tiled weight image (bf16 activations as three residual
                        e2m1 pieces).  The tiled image is built once, on the first forward that needs it,
                        and serves both tensor-core kernels.
      "ref" weights     fp32 scales per 32 are not an operand format of the block-scaled tensor cores:
                        rows go through the CUDA-core GEMV 16 at a time, exactly as stored.

    There is no dequantise-and-matmul path.
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

    # ------------------------------------------------------------------ tensor-core path ("nvfp4" format)
    def tensor_core_ready(self) -> bool:
        """True if the weights are standard NVFP4 (E4M3 scale per 16 + global scale) on a CUDA device."""
        return (self.block_size == 16 and self.weight_scales is not None and self.weight_scales.dtype == torch.uint8
                and self.weight_packed.is_cuda and self.in_features % 16 == 0)

    def _tc_state(self):
        """(tiled weight image, GEMV scratch), built on first use and whenever the packed
        weights were replaced (load_state_dict, .to(device))."""
        key = (self.weight_packed.data_ptr(), self.weight_scales.data_ptr(), str(self.weight_packed.device))
        st = getattr(self, "_tc", None)
        if st is None or st[0] != key:
            N, K = self.out_features, self.in_features
            dev = self.weight_packed.device
            b = torch.zeros((N, ops.packed_pitch(K)), dtype=torch.uint8, device=dev)
            b[:, :K // 2] = self.weight_packed
            image = ops.tile_weights(b, ops.swizzle_scales(self.weight_scales.contiguous()), N, K)
            st = (key, image, ops.tc_gemv_workspace(N, K, dev))
            self._tc = st
        return st[1], st[2]

    def _forward_tensor_cores(self, x2, act, bias):
        T = x2.shape[0]
        out = torch.empty((T, self.out_features), dtype=x2.dtype, device=x2.device)
        if T <= 4 and self.in_features % 32 == 0 and self.weight_packed.is_contiguous():
            # one matrix, a few tokens: the CUDA-core GEMV streams the packed rows as stored and has no
            # split-K hand-over at the end (4.5-12 us against 9-27 us for the tensor-core kernel, whose
            # ground is many matrices per launch)
            return ops.nvfp4_gemv_out(x2, self.weight_packed, self.weight_scales, out, bias, act, 16, self.global_scale)
        image, gemv_ws = self._tc_state()
        if T <= 16:
            return ops.tc_gemv(x2, image, self.out_features, out, self.global_scale, bias, act, 3, gemv_ws)
        xb = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
        q = _operand_buffer(self, T, self.in_features, x2.device)
        # the quantiser and the GEMM are chained by programmatic dependent launch: the weights are static, so
        # the GEMM may fetch them while the quantiser still runs
        with ops.launch_flags(ops.FLAG_PDL):
            ops.rowop(_lib.ROW_NONE, xb, self.in_features, q)
            args = _lib.GemmArgs(a_packed=ops._ptr(q.packed), a_pieces=3, a_row_scale=ops._ptr(q.row_scale),
                                 b_packed=ops._ptr(image), alpha=float(self.global_scale), bias=ops._ptr(bias),
                                 activation=int(act), out=ops._ptr(out), out_dtype=ops._dt(out), ldo=out.stride(0), M=T,
                                 N=self.out_features, K=self.in_features, layout=ops.OPERANDS_TILED)
            ops._gemm_ex(args, x2.device, _split_k_scratch(self, T, self.out_features, self.in_features, x2.device))
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        batch_shape = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            x2 = x2.float()
        x2 = x2.contiguous()
        T = x2.shape[0]
        act = ACTIVATIONS.get(self.activation, 0)
        bias = None if self.bias is None else self.bias.detach().float().contiguous()
        if self.tensor_core_ready():
            return self._forward_tensor_cores(x2, act, bias).reshape(*batch_shape, self.out_features).to(x.dtype)
        out = torch.empty((T, self.out_features), dtype=x2.dtype, device=x2.device)
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
    reference module's 'silu'; Gemma's own MLP uses 'gelu' (tanh form).

    With "nvfp4" weights the forward is three or four launches whatever the token count: gate and up run as
    ONE stacked [2I, K] matrix (one GEMV launch for <= 16 tokens, one tensor-core GEMM otherwise), the row
    kernel applies act(gate) * up with the module's roundings (and, for the GEMM, writes the down
    projection's operand), then the down projection."""

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
        if fmt == "nvfp4":
            # gate and up are quantised as ONE [2I, K] matrix (a common global scale), so that they can run as one launch
            with torch.no_grad():
                w = torch.cat([mlp.gate_proj.weight.data, mlp.up_proj.weight.data], 0)
                packed, scales, gs = quantize_nvfp4_two_level(w, 16)
                I = mlp.gate_proj.out_features
                dev = mlp.gate_proj.weight.device
                for lin, sl in ((layer.gate_proj, slice(0, I)), (layer.up_proj, slice(I, 2 * I))):
                    lin.weight_packed, lin.weight_scales, lin.global_scale = packed[sl].contiguous().to(dev), scales[sl].contiguous().to(dev), gs
        return layer

    def _stacked_gate_up(self):
        """Tiled image of [W_gate; W_up] under ONE global scale, or None if the projections do not share one
        (each was quantised on its own: the stacked launch needs a common fp32 multiplier)."""
        g, u = self.gate_proj, self.up_proj
        key = (g.weight_packed.data_ptr(), u.weight_packed.data_ptr())
        st = getattr(self, "_gu", None)
        if st is None or st[0] != key:
            if g.global_scale != u.global_scale:
                st = (key, None)
            else:
                dev = g.weight_packed.device
                N, K = 2 * self.intermediate_size, self.hidden_size
                b = torch.zeros((N, ops.packed_pitch(K)), dtype=torch.uint8, device=dev)
                b[:, :K // 2] = torch.cat([g.weight_packed, u.weight_packed], 0)
                sc = torch.cat([g.weight_scales, u.weight_scales], 0).contiguous()
                st = (key, ops.tile_weights(b, ops.swizzle_scales(sc), N, K), ops.tc_gemv_workspace(N, K, dev))
            self._gu = st
        return st

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        g, u, d = self.gate_proj, self.up_proj, self.down_proj
        fast = (g.tensor_core_ready() and u.tensor_core_ready() and d.tensor_core_ready() and g.bias is None
                and u.bias is None and g.activation in ("gelu", "silu") and self.intermediate_size % 16 == 0)
        st = self._stacked_gate_up() if fast else None
        if st is None or st[1] is None:
            return self.down_proj(self.gate_proj(x) * self.up_proj(x))
        from . import _lib
        _, gu_image, gu_gemv_ws = st
        batch_shape = x.shape[:-1]
        x2 = x.reshape(-1, self.hidden_size).contiguous()
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        T, I = x2.shape[0], self.intermediate_size
        gu = torch.empty((T, 2 * I), dtype=torch.bfloat16, device=x2.device)
        mode = _lib.ROW_GELU_MUL if g.activation == "gelu" else _lib.ROW_SILU_MUL
        d_image, d_gemv_ws = d._tc_state()
        d_bias = None if d.bias is None else d.bias.detach().float().contiguous()
        out = torch.empty((T, self.hidden_size), dtype=torch.bfloat16, device=x2.device)
        if T <= 16:
            ops.tc_gemv(x2, gu_image, 2 * I, gu, g.global_scale, None, 0, 3, gu_gemv_ws)
            h = torch.empty((T, I), dtype=torch.bfloat16, device=x2.device)
            ops.rowop(mode, gu, I, None, y_out=h, M=T)
            if T <= 4 and d.in_features % 32 == 0 and d.weight_packed.is_contiguous():
                ops.nvfp4_gemv_out(h, d.weight_packed, d.weight_scales, out, d_bias, 0, 16, d.global_scale)
            else:
                ops.tc_gemv(h, d_image, self.hidden_size, out, d.global_scale, d_bias, 0, 3, d_gemv_ws)
        else:
            qx = _operand_buffer(g, T, self.hidden_size, x2.device)
            q = _operand_buffer(d, T, I, x2.device)
            with ops.launch_flags(ops.FLAG_PDL):     # four launches chained by programmatic dependent launch
                ops.rowop(_lib.ROW_NONE, x2, self.hidden_size, qx)
                args = _lib.GemmArgs(a_packed=ops._ptr(qx.packed), a_pieces=3, a_row_scale=ops._ptr(qx.row_scale),
                                     b_packed=ops._ptr(gu_image), alpha=float(g.global_scale), out=ops._ptr(gu),
                                     out_dtype=ops._dt(gu), ldo=gu.stride(0), M=T, N=2 * I, K=self.hidden_size,
                                     layout=ops.OPERANDS_TILED)
                ops._gemm_ex(args, x2.device, _split_k_scratch(g, T, 2 * I, self.hidden_size, x2.device))
                ops.rowop(mode, gu, I, q, M=T)
                args = _lib.GemmArgs(a_packed=ops._ptr(q.packed), a_pieces=3, a_row_scale=ops._ptr(q.row_scale),
                                     b_packed=ops._ptr(d_image), alpha=float(d.global_scale), bias=ops._ptr(d_bias),
                                     out=ops._ptr(out), out_dtype=ops._dt(out), ldo=out.stride(0), M=T, N=self.hidden_size,
                                     K=I, layout=ops.OPERANDS_TILED)
                ops._gemm_ex(args, x2.device, _split_k_scratch(d, T, self.hidden_size, I, x2.device))
        return out.reshape(*batch_shape, self.hidden_size).to(x.dtype)


def replace_mlp_with_nvfp4_packed(model, block_size: int = BLOCK_SIZE, target_layers: Optional[list] = None,
                                  gate_activation: str = "silu", fmt: str = "nvfp4") -> int:
    """Swap every `layer.mlp` of model.paligemma_with_expert.paligemma.language_model for an
    NVFP4PackedMLP; returns the number replaced.  `fmt="nvfp4"` (default) stores standard NVFP4, which the
    tensor-core kernels consume; `fmt="ref"` keeps the reference's block-32 fp32-scale buffers (CUDA-core
    GEMV only)."""
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
            layer.mlp = NVFP4PackedMLP.from_gemma_mlp(layer.mlp, block_size, gate_activation, fmt).to(device)
            count += 1
    return count
