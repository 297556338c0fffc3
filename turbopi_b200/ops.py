"""Tensor-level wrappers over the C ABI.

The functions keep the names, argument order and return conventions of the
reference's pybind / torch.library surfaces:

  w4a16_gemv(input, weight_packed, scales)            openpi/src/openpi/ops/w4a16_gemv.py:244-294
  nvfp4_gemv_v6 / nvfp4_gemv_w4a16 / nvfp4_gemv       openpi/nvfp4_packed_plugin/src/nvfp4_gemv_v5.cu:566-602,
                                                       openpi/nvfp4_packed_plugin/src/nvfp4_packed_torch.cu:296-319

and add the B200-native forms (bf16 in/out, E4M3 block-16 scales, grouped launch).
Every tensor must live on a CUDA device; nothing here computes on the CPU.
"""
import ctypes

import torch

from . import _lib
from ._lib import (ACT_NONE, BF16, F16, F32, FLAG_NONE, FLAG_PDL, INT4_KBLOCK, INT4_PLUGIN, INT4_ROWMAJOR, SCALE_E4M3,
                   SCALE_F16, SCALE_BF16, SCALE_F32, TurboPiError)

_DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


def _dt(t):
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TurboPiError(f"unsupported dtype {t.dtype}") from None


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise TurboPiError("turbopi_b200 kernels need CUDA tensors (there is no CPU path)")


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _scale_kind(scales):
    if scales.dtype == torch.float32:
        return SCALE_F32
    if scales.dtype in (torch.uint8, torch.float8_e4m3fn):
        return SCALE_E4M3
    if scales.dtype == torch.float16:
        return SCALE_F16
    if scales.dtype == torch.bfloat16:
        return SCALE_BF16
    raise TurboPiError(f"unsupported scale dtype {scales.dtype}")


# ------------------------------------------------------------------------------------- INT4
def w4a16_gemv_out(input, weight_packed, scales, out, bias=None, group_size=32, layout=INT4_KBLOCK, pdl=False):
    """out[M, N] = input[M, K] @ dequant(W)^T (+ bias); M <= 16.  Writes into `out`."""
    _cuda(input, weight_packed, scales, out, bias)
    M, K = input.shape
    N = out.shape[1]
    with torch.cuda.device(input.device):
        st = _lib.load().tpb200_w4a16_gemv(
            _ptr(input), _dt(input), _ptr(weight_packed), _ptr(scales), _scale_kind(scales), _ptr(bias),
            _dt(bias) if bias is not None else F32, _ptr(out), _dt(out), M, N, K, group_size, layout,
            FLAG_PDL if pdl else FLAG_NONE, _stream(input))
    _lib.check(st, "tpb200_w4a16_gemv")
    return out


def w4a16_gemv(input, weight_packed, scales):
    """Same contract as torch.ops.openpi.w4a16_gemv: input (1, K) fp16 CUDA, weight_packed
    (K/32, N, 4) int32, scales (K/32, N) fp16; returns (1, N) float32.  Raises ValueError
    for more than one row, as the reference does."""
    if not input.is_cuda:
        raise TurboPiError("Input must be on CUDA")
    if input.size(0) > 1:
        raise ValueError("W4A16 GEMV only supports seq_len=1. Use F.linear for seq_len > 1.")
    nb, N, four = weight_packed.shape
    if four != 4 or input.shape[1] != nb * 32:
        raise TurboPiError(f"shape mismatch: input {tuple(input.shape)}, weight_packed {tuple(weight_packed.shape)}")
    out = torch.empty((input.size(0), N), dtype=torch.float32, device=input.device)
    return w4a16_gemv_out(input.contiguous(), weight_packed.contiguous(), scales.contiguous(), out)


def w4a16_gemm(x, weight, scales, zeros=None, bias=None, out=None, layout=INT4_KBLOCK, alpha=1.0, beta=0.0,
               out_dtype=torch.bfloat16):
    """out[M, N] = alpha * x @ dequant(W)^T + bias + beta * out for any M on the tensor cores (INT4 weights
    dequantised to bf16 inside the kernel).  layout INT4_KBLOCK: weight (K/32, N, 4) int32 + fp16 scales
    (K/32, N); INT4_PLUGIN: weight [N, K/2] int8 + bf16 scales / zeros [N, K/128].  x is converted to bf16."""
    _cuda(x, weight, scales, zeros, bias, out)
    M, K = x.shape
    N = weight.shape[1] if layout == INT4_KBLOCK else weight.shape[0]
    xb = x.to(torch.bfloat16).contiguous()
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if bias is not None:
        bias = bias.float().contiguous()
    with torch.cuda.device(x.device):
        st = _lib.load().tpb200_w4a16_gemm(_ptr(xb), _ptr(weight), _ptr(scales), _ptr(zeros), _ptr(bias), F32, _ptr(out),
                                           _dt(out), M, N, K, out.stride(0), int(layout), float(alpha), float(beta),
                                           _launch_flags, _stream(x))
    _lib.check(st, "tpb200_w4a16_gemm")
    return out


# ------------------------------------------------------------------------------------- NVFP4
def nvfp4_gemv_out(x, weight_packed, weight_scales, out, bias=None, activation=ACT_NONE, block_size=32,
                   global_scale=1.0, x_scales=None, pdl=False):
    """out[M, N] = act(gs * x @ dequant(W)^T + bias); M <= 16.  Writes into `out`."""
    _cuda(x, weight_packed, weight_scales, out, bias, x_scales)
    M, K = x.shape
    N = out.shape[1]
    with torch.cuda.device(x.device):
        st = _lib.load().tpb200_nvfp4_gemv(
            _ptr(x), _dt(x), _ptr(x_scales), _ptr(weight_packed), _ptr(weight_scales), _scale_kind(weight_scales),
            block_size, float(global_scale), _ptr(bias), _dt(bias) if bias is not None else F32, _ptr(out),
            _dt(out), M, N, K, int(activation), FLAG_PDL if pdl else FLAG_NONE, _stream(x))
    _lib.check(st, "tpb200_nvfp4_gemv")
    return out


def _nvfp4_gemv_ref_signature(activation, weight_packed, scale_W, bias, M, N, K, activation_type, scale_A=None):
    activation = activation.to(torch.float32).contiguous()
    weight_packed = weight_packed.contiguous()
    scale_W = scale_W.to(torch.float32).contiguous()
    if bias is not None and bias.numel() > 0:
        bias = bias.to(torch.float32).contiguous()
    else:
        bias = None
    if scale_A is not None:
        scale_A = scale_A.to(torch.float32).contiguous()
    if tuple(activation.shape) != (M, K) or tuple(weight_packed.shape) != (N, K // 2):
        raise TurboPiError("nvfp4_gemv: tensor shapes do not match M, N, K")
    out = torch.empty((M, N), dtype=torch.float32, device=activation.device)
    for m0 in range(0, M, 16):                       # the kernel takes up to 16 rows per launch
        m1 = min(M, m0 + 16)
        nvfp4_gemv_out(activation[m0:m1], weight_packed, scale_W, out[m0:m1], bias, activation_type, 32, 1.0,
                       None if scale_A is None else scale_A[m0:m1])
    return out


def nvfp4_gemv_v6(activation, weight_packed, scale_W, bias, M, N, K, activation_type):
    """nvfp4_gemv_v6(activation, weight_packed uint8[N,K/2], scale_W f32[N,K/32], bias|None, M, N, K, act)
    -> f32[M, N]  (openpi/nvfp4_packed_plugin/src/nvfp4_gemv_v5.cu:430-476)."""
    return _nvfp4_gemv_ref_signature(activation, weight_packed, scale_W, bias, M, N, K, activation_type)


nvfp4_gemv_w4a16 = nvfp4_gemv_v6  # openpi/nvfp4_packed_plugin/src/nvfp4_packed_torch.cu:232-290


def nvfp4_gemv(activation, weight_packed, scale_A, scale_W, bias, M, N, K, activation_type):
    """W4A4-style variant with per-block activation scales
    (openpi/nvfp4_packed_plugin/src/nvfp4_packed_torch.cu:173-230)."""
    return _nvfp4_gemv_ref_signature(activation, weight_packed, scale_W, bias, M, N, K, activation_type, scale_A)


class GroupedGemv:
    """A fixed list of independent NVFP4 GEMVs launched as ONE kernel.  The problem table is
    built once (host memory only); `launch()` enqueues the kernel on the current stream."""

    def __init__(self, problems, block_size, activation=ACT_NONE, pdl=False):
        # problems: list of dicts with x, weight_packed, weight_scales, out, optional bias, global_scale
        if not 1 <= len(problems) <= _lib.MAX_GROUP:
            raise TurboPiError(f"1..{_lib.MAX_GROUP} problems per grouped launch")
        p0 = problems[0]
        self._keep = problems
        self.M = p0["x"].shape[0]
        self.x_dtype = _dt(p0["x"])
        self.out_dtype = _dt(p0["out"])
        self.scale_kind = _scale_kind(p0["weight_scales"])
        self.bias_dtype = _dt(p0["bias"]) if p0.get("bias") is not None else F32
        self.block_size = block_size
        self.activation = int(activation)
        self.flags = FLAG_PDL if pdl else FLAG_NONE
        self.device = p0["x"].device
        arr = (_lib.GemvProblem * len(problems))()
        for i, p in enumerate(problems):
            _cuda(p["x"], p["weight_packed"], p["weight_scales"], p["out"], p.get("bias"))
            N, Kh = p["weight_packed"].shape
            arr[i] = _lib.GemvProblem(_ptr(p["x"]), _ptr(p["weight_packed"]), _ptr(p["weight_scales"]),
                                      _ptr(p.get("bias")), _ptr(p["out"]), N, Kh * 2,
                                      float(p.get("global_scale", 1.0)), p["out"].stride(0))
        self._arr = arr

    def launch(self):
        with torch.cuda.device(self.device):
            st = _lib.load().tpb200_nvfp4_gemv_grouped(
                self._arr, len(self._arr), self.x_dtype, self.scale_kind, self.block_size, self.bias_dtype,
                self.out_dtype, self.M, self.activation, self.flags,
                torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(st, "tpb200_nvfp4_gemv_grouped")


# ------------------------------------------------------------------------------------- plugin quantisers
def quantize_weight_to_int4(weight_bf16, group_size=128):
    """quantizeWeightToINT4: bf16 [N, K] -> (int8 [N, K/2], bf16 scales [N, K/g], bf16 zeros)."""
    _cuda(weight_bf16)
    w = weight_bf16.to(torch.bfloat16).contiguous()
    N, K = w.shape
    packed = torch.empty((N, K // 2), dtype=torch.int8, device=w.device)
    scales = torch.empty((N, K // group_size), dtype=torch.bfloat16, device=w.device)
    zeros = torch.empty_like(scales)
    with torch.cuda.device(w.device):
        _lib.load().quantizeWeightToINT4(_ptr(w), _ptr(packed), _ptr(scales), _ptr(zeros), N, K, group_size, _stream(w))
    _lib.check_void("quantizeWeightToINT4")
    return packed, scales, zeros


def dequantize_int4_to_bf16(packed, scales, zeros, group_size=128):
    _cuda(packed, scales, zeros)
    N, Kh = packed.shape
    out = torch.empty((N, Kh * 2), dtype=torch.bfloat16, device=packed.device)
    with torch.cuda.device(packed.device):
        _lib.load().dequantizeINT4ToBF16(_ptr(packed), _ptr(scales), _ptr(zeros), _ptr(out), N, Kh * 2, group_size,
                                         _stream(packed))
    _lib.check_void("dequantizeINT4ToBF16")
    return out


def quantize_activation_to_fp8(x_bf16):
    """quantizeActivationToFP8: bf16 [M, K] -> (E4M3 bytes [M, K], E4M3 scale bytes [M, K/16])."""
    _cuda(x_bf16)
    x = x_bf16.to(torch.bfloat16).contiguous()
    M, K = x.shape
    out = torch.empty((M, K), dtype=torch.uint8, device=x.device)
    scales = torch.empty((M, K // 16), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _lib.load().quantizeActivationToFP8(_ptr(x), _ptr(out), _ptr(scales), M, K, _stream(x))
    _lib.check_void("quantizeActivationToFP8")
    return out, scales


def quantize_weight_to_nvfp4(weight_bf16):
    """quantizeWeightToNVFP4: bf16 [N, K] -> (packed [K/2, N] uint8, E4M3 scale bytes [K/16, N])."""
    _cuda(weight_bf16)
    w = weight_bf16.to(torch.bfloat16).contiguous()
    N, K = w.shape
    packed = torch.empty((K // 2, N), dtype=torch.uint8, device=w.device)
    scales = torch.empty((K // 16, N), dtype=torch.uint8, device=w.device)
    with torch.cuda.device(w.device):
        _lib.load().quantizeWeightToNVFP4(_ptr(w), _ptr(packed), _ptr(scales), N, K, _stream(w))
    _lib.check_void("quantizeWeightToNVFP4")
    return packed, scales


# ------------------------------------------------------------------------------------- NVFP4 tensor-core GEMM
def nvfp4_sf_bytes(rows, K):
    return int(_lib.load().tpb200_nvfp4_sf_bytes(int(rows), int(K)))


def packed_pitch(K):
    """Row pitch in bytes of a packed e2m1 matrix: K/2 rounded up to 16 bytes."""
    return (K // 2 + 15) // 16 * 16


def swizzle_scales(sf_bytes):
    """UE4M3 scale bytes [rows, K/16] -> the GEMM's atom layout (flat uint8): rows padded to 128,
    K-blocks to 16, atoms of 128 rows x 4 blocks ordered [row tile][K atom], byte
    (r % 32) * 16 + (r // 32) * 4 + kb inside an atom.  Pure index shuffle (host-side weight prep)."""
    R, KB = sf_bytes.shape
    Rp, Kp = (R + 127) // 128 * 128, (KB + 15) // 16 * 16
    pad = torch.zeros((Rp, Kp), dtype=torch.uint8, device=sf_bytes.device)
    pad[:R, :KB] = sf_bytes
    t = pad.reshape(Rp // 128, 4, 32, Kp // 4, 4).permute(0, 3, 2, 1, 4)
    return t.contiguous().reshape(-1)


def nvfp4_quantize_act(x, packed=None, sf=None):
    """x [M, K] (bf16/fp16/fp32, CUDA) -> (packed [M, pitch] uint8, swizzled UE4M3 scales)."""
    _cuda(x)
    M, K = x.shape
    x = x.contiguous()
    pitch = packed_pitch(K)
    if packed is None:
        packed = torch.empty((M, pitch), dtype=torch.uint8, device=x.device)
    if sf is None:
        sf = torch.empty(nvfp4_sf_bytes(M, K), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        st = _lib.load().tpb200_nvfp4_quantize_act(_ptr(x), _dt(x), K, _ptr(packed), pitch, _ptr(sf), M, K, _stream(x))
    _lib.check(st, "tpb200_nvfp4_quantize_act")
    return packed, sf


def nvfp4_gemm(a_packed, a_sf, b_packed, b_sf, M, N, K, alpha=1.0, bias=None, activation=ACT_NONE, out=None,
               out_dtype=torch.bfloat16):
    """out[M, N] = act(alpha * A @ B^T + bias) with A, B packed e2m1 + swizzled UE4M3 scales."""
    _cuda(a_packed, a_sf, b_packed, b_sf, bias, out)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a_packed.device)
    if bias is not None:
        bias = bias.float().contiguous()
    with torch.cuda.device(a_packed.device):
        st = _lib.load().tpb200_nvfp4_gemm(
            _ptr(a_packed), a_packed.stride(0), _ptr(a_sf), _ptr(b_packed), b_packed.stride(0), _ptr(b_sf),
            float(alpha), _ptr(bias), int(activation), _ptr(out), _dt(out), out.stride(0), M, N, K, FLAG_NONE,
            _stream(a_packed))
    _lib.check(st, "tpb200_nvfp4_gemm")
    return out


def nvfp4_quantize_act_pieces(x, pieces=3):
    """bf16/fp16/fp32 x [M, K] -> `pieces` residual e2m1 operands stacked along rows (piece p of row m at
    row p * piece_rows + m), their swizzled UE4M3 scales, and the per-row multiplier that undoes the
    power-of-two pre-scale.  Returns (packed, sf, row_scale, piece_rows)."""
    _cuda(x)
    M, K = x.shape
    x = x.contiguous()
    pitch = packed_pitch(K)
    piece_rows = (M + 127) // 128 * 128
    packed = torch.empty((pieces * piece_rows, pitch), dtype=torch.uint8, device=x.device)
    sf = torch.empty(nvfp4_sf_bytes(pieces * piece_rows, K), dtype=torch.uint8, device=x.device)
    row_scale = torch.empty((M,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        st = _lib.load().tpb200_nvfp4_quantize_act_pieces(_ptr(x), _dt(x), K, _ptr(packed), pitch, _ptr(sf),
                                                          _ptr(row_scale), M, K, pieces, piece_rows, _stream(x))
    _lib.check(st, "tpb200_nvfp4_quantize_act_pieces")
    return packed, sf, row_scale, piece_rows


def gemm_workspace(device, nbytes=32 << 20):
    """Zeroed split-K scratch for the tensor-core GEMM.  One buffer serves any number of launches that
    run one after another on a stream; launches that may overlap need a buffer each."""
    return torch.zeros(nbytes, dtype=torch.uint8, device=device)


def nvfp4_gemm_workspace_size(M, N, K, pieces=1, layout=0):
    return int(_lib.load().tpb200_nvfp4_gemm_workspace_size(M, N, K, pieces, layout))


# Launch flags applied to the tensor-core GEMM and the row kernel (see `launch_flags`)
_launch_flags = FLAG_NONE


class launch_flags:
    """Context manager: `with ops.launch_flags(ops.FLAG_PDL): ...` launches every GEMM and row kernel inside
    with programmatic stream serialisation, so that each kernel's set-up overlaps its predecessor's tail."""

    def __init__(self, flags):
        self.flags = int(flags)

    def __enter__(self):
        global _launch_flags
        self.prev, _launch_flags = _launch_flags, self.flags
        return self

    def __exit__(self, *exc):
        global _launch_flags
        _launch_flags = self.prev
        return False


def _gemm_ex(args, device, workspace=None):
    args.flags = _launch_flags
    if workspace is not None:
        _cuda(workspace)
        args.workspace = _ptr(workspace)
        args.workspace_bytes = workspace.numel() * workspace.element_size()
    with torch.cuda.device(device):
        st = _lib.load().tpb200_nvfp4_gemm_ex(ctypes.byref(args), torch.cuda.current_stream(device).cuda_stream)
    _lib.check(st, "tpb200_nvfp4_gemm_ex")


def nvfp4_gemm_w4a16(x, b_packed, b_sf, N, alpha=1.0, bias=None, activation=ACT_NONE, pieces=3, out=None,
                     out_dtype=torch.bfloat16, workspace=None):
    """Weight-only semantics on the tensor-core path: out = act(alpha * x @ dequant(W)^T + bias) with the
    bf16 activations carried as `pieces` residual e2m1 operands (3 pieces keep ~bf16 precision)."""
    M, K = x.shape
    a, a_sf, row_scale, piece_rows = nvfp4_quantize_act_pieces(x, pieces)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if bias is not None:
        bias = bias.float().contiguous()
    args = _lib.GemmArgs(a_packed=_ptr(a), a_pitch=a.stride(0), a_sf=_ptr(a_sf), a_pieces=pieces,
                         a_piece_rows=piece_rows, a_row_scale=_ptr(row_scale), b_packed=_ptr(b_packed),
                         b_pitch=b_packed.stride(0), b_sf=_ptr(b_sf), alpha=float(alpha), bias=_ptr(bias),
                         activation=int(activation), out=_ptr(out), out_dtype=_dt(out), ldo=out.stride(0),
                         M=M, N=N, K=K)
    _gemm_ex(args, x.device, workspace)
    return out


def qkv_tile_permutation(q_dim, head_dim=256):
    """Row order of the stacked [Wq; Wk; Wv] the fused-QKV kernel expects: every 128-row tile holds 64
    rows of one head's first half followed by their rotate-half partners (+ head_dim / 2)."""
    if head_dim != 256:
        raise TurboPiError("the fused QKV kernel is built for head_dim 256")
    heads = q_dim // 256 + 2
    idx = []
    for h in range(heads):
        for half in range(2):
            base = h * 256 + half * 64
            idx += list(range(base, base + 64)) + list(range(base + 128, base + 192))
    return torch.tensor(idx, dtype=torch.long)


def geglu_row_permutation(inter):
    """Row order of a stacked [W_gate; W_up] ([2 * inter, K]) for the gated-GELU epilogue: every 256-row
    block holds 128 gate rows followed by the 128 matching up rows."""
    if inter % 128:
        raise TurboPiError("the gated-GELU epilogue needs an intermediate size that is a multiple of 128")
    t = torch.arange(inter // 128)[:, None, None] * 128
    r = torch.arange(128)[None, None, :]
    half = torch.tensor([0, inter])[None, :, None]
    return (t + half + r).reshape(-1)


def rope_tables(num_positions, head_dim=256, theta=10000.0, device="cuda"):
    """cos / sin tables [positions, head_dim / 2] in bf16, computed the way the model does:
    inv_freq in fp32 rounded to bf16, pos * inv_freq in fp32, cos / sin rounded to bf16."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    inv = inv.to(torch.bfloat16).float()
    f = torch.arange(num_positions, dtype=torch.float32)[:, None] * inv[None, :]
    return f.cos().to(torch.bfloat16).to(device).contiguous(), f.sin().to(torch.bfloat16).to(device).contiguous()


def fused_qkv_rope_append(x, w_packed, w_sf, q_dim, k_rows, v_rows, positions, rope_cos, rope_sin, alpha=1.0,
                          pieces=3, q_out=None, workspace=None, check_positions=True):
    """q = RoPE(x Wq^T), cache K rows <- RoPE(x Wk^T), cache V rows <- x Wv^T in ONE kernel.
    x [M, H] bf16; w_packed / w_sf: tile-permuted stacked [Wq; Wk; Wv] (qkv_tile_permutation) in NVFP4;
    k_rows / v_rows: views of the cache whose row 0 is the first token's row, row stride 256 (bf16);
    positions int32 [M], each inside the RoPE table (`check_positions` reads them back to verify, which
    synchronises: switch it off inside a stream capture).  Returns q [M, q_dim] bf16."""
    _cuda(x, w_packed, w_sf, k_rows, v_rows, positions, rope_cos, rope_sin)
    M, K = x.shape
    N = q_dim + 512
    if (k_rows.stride(0) != 256 or v_rows.stride(0) != 256 or k_rows.dtype != torch.bfloat16
            or v_rows.dtype != torch.bfloat16):
        raise TurboPiError("cache rows must be bf16 with a row stride of 256 elements")
    if k_rows.shape[0] < M or v_rows.shape[0] < M:
        raise TurboPiError(f"cache views hold {min(k_rows.shape[0], v_rows.shape[0])} rows, {M} tokens to append")
    if positions.dtype != torch.int32 or positions.numel() < M:
        raise TurboPiError("positions must be int32 with one entry per token")
    if rope_cos.shape != rope_sin.shape or rope_cos.dtype != torch.bfloat16 or rope_cos.shape[1] != 128:
        raise TurboPiError("RoPE tables must be bf16 [positions, 128]")
    if check_positions and (int(positions[:M].min()) < 0 or int(positions[:M].max()) >= rope_cos.shape[0]):
        raise TurboPiError("a position lies outside the RoPE table")
    if q_out is None:
        q_out = torch.empty((M, q_dim), dtype=torch.bfloat16, device=x.device)
    if w_sf is None:
        # w_packed is the tiled image of the permuted weight (tile_weights)
        q = QuantBuf(M, K, pieces, x.device, tiled=True)
        rowop(_lib.ROW_NONE, x.contiguous(), K, q)
        args = _lib.GemmArgs(a_packed=_ptr(q.packed), a_pieces=pieces, a_row_scale=_ptr(q.row_scale),
                             b_packed=_ptr(w_packed), layout=1)
    else:
        a, a_sf, row_scale, piece_rows = nvfp4_quantize_act_pieces(x, pieces)
        args = _lib.GemmArgs(a_packed=_ptr(a), a_pitch=a.stride(0), a_sf=_ptr(a_sf), a_pieces=pieces,
                             a_piece_rows=piece_rows, a_row_scale=_ptr(row_scale), b_packed=_ptr(w_packed),
                             b_pitch=w_packed.stride(0), b_sf=_ptr(w_sf))
    args.alpha, args.M, args.N, args.K = float(alpha), M, N, K
    args.qkv_q_out, args.qkv_ldq, args.qkv_q_dim = _ptr(q_out), q_out.stride(0), q_dim
    args.qkv_k_rows, args.qkv_v_rows, args.qkv_positions = _ptr(k_rows), _ptr(v_rows), _ptr(positions)
    args.qkv_rope_cos, args.qkv_rope_sin = _ptr(rope_cos), _ptr(rope_sin)
    _gemm_ex(args, x.device, workspace)
    return q_out


# ------------------------------------------------------------------------- tiled operands for the GEMM
OPERANDS_ROWMAJOR, OPERANDS_TILED = 0, 1


def tile_weights(b_packed, b_sf, N, K):
    """Row-major GEMM B operand (codes [N, pitch] + swizzled scales) -> the tiled image of the fast path:
    blocks [ceil(N/256)][ceil(K/256)] of 36 KB that carry codes and scales of 256 rows for one K stage."""
    _cuda(b_packed, b_sf)
    image = torch.empty(int(_lib.load().tpb200_nvfp4_tiled_b_bytes(N, K)), dtype=torch.uint8, device=b_packed.device)
    with torch.cuda.device(b_packed.device):
        st = _lib.load().tpb200_nvfp4_tile_weights(_ptr(b_packed), b_packed.stride(0), _ptr(b_sf), _ptr(image), N, K,
                                                   _stream(b_packed))
    _lib.check(st, "tpb200_nvfp4_tile_weights")
    # weight preparation is a one-off: finish it here, so that a following launch with FLAG_PDL (which reads
    # weights before it waits for its predecessor) can never start on an incomplete image
    torch.cuda.current_stream(b_packed.device).synchronize()
    return image


class QuantBuf:
    """Pre-allocated A operand of the GEMM for an [M, K] activation: residual pieces + scales + row
    multipliers, as the tiled image (default) or the row-major operand.  Allocated zeroed: padding rows
    and padding K keep zero scales because the quantiser never writes them."""

    def __init__(self, M, K, pieces, device, tiled=True):
        self.M, self.K, self.pieces, self.tiled = M, K, pieces, tiled
        self.piece_rows = (M + 127) // 128 * 128
        self.row_scale = torch.ones((M,), dtype=torch.float32, device=device)
        if tiled:
            self.pitch = 0
            self.packed = torch.zeros(int(_lib.load().tpb200_nvfp4_tiled_a_bytes(M, K, pieces)), dtype=torch.uint8,
                                      device=device)
            self.sf = None
        else:
            self.pitch = packed_pitch(K)
            self.packed = torch.zeros((pieces * self.piece_rows, self.pitch), dtype=torch.uint8, device=device)
            self.sf = torch.zeros(nvfp4_sf_bytes(pieces * self.piece_rows, K), dtype=torch.uint8, device=device)

    @property
    def layout(self):
        return OPERANDS_TILED if self.tiled else OPERANDS_ROWMAJOR


def rowop(mode, x, K, q=None, res_in=None, gate=None, h_out=None, w0=None, w1=None, eps=1e-6, y_out=None, M=None):
    """tpb200_row_transform_quantize: optional gated residual, a norm (or GELU(gate) * up), an optional
    bf16 copy, and the residual-piece quantisation into `q` (a QuantBuf)."""
    M = x.shape[0] if M is None else M
    p = _ptr
    a = _lib.RowOpArgs(mode=mode, M=M, K=K, x=p(x), ldx=x.stride(0), res_in=p(res_in), gate=p(gate), h_out=p(h_out),
                       w0=p(w0), w1=p(w1), eps=float(eps), y_out=p(y_out),
                       packed=p(q.packed) if q is not None else 0, pitch=q.pitch if q is not None else 0,
                       sf=p(q.sf) if q is not None else 0, row_scale=p(q.row_scale) if q is not None else 0,
                       pieces=q.pieces if q is not None else 0, piece_rows=q.piece_rows if q is not None else 0,
                       layout=q.layout if q is not None else 0, flags=_launch_flags)
    with torch.cuda.device(x.device):
        st = _lib.load().tpb200_row_transform_quantize(ctypes.byref(a), torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(st, "tpb200_row_transform_quantize")


def nvfp4_gemm_w4a16_tiled(x, b_image, N, alpha=1.0, bias=None, activation=ACT_NONE, pieces=3, out=None,
                           out_dtype=torch.bfloat16, workspace=None):
    """nvfp4_gemm_w4a16 on the tiled operand images: x bf16 [M, K] is quantised straight into the A image
    (tpb200_row_transform_quantize), b_image comes from tile_weights()."""
    _cuda(x, b_image, bias, out)
    M, K = x.shape
    q = QuantBuf(M, K, pieces, x.device, tiled=True)
    rowop(_lib.ROW_NONE, x.contiguous(), K, q)
    if out is None:
        out = torch.empty((M, N // 2 if activation == _lib.ACT_GEGLU else N), dtype=out_dtype, device=x.device)
    if bias is not None:
        bias = bias.float().contiguous()
    args = _lib.GemmArgs(a_packed=_ptr(q.packed), a_pieces=pieces, a_row_scale=_ptr(q.row_scale),
                         b_packed=_ptr(b_image), alpha=float(alpha), bias=_ptr(bias), activation=int(activation),
                         out=_ptr(out), out_dtype=_dt(out), ldo=out.stride(0), M=M, N=N, K=K, layout=OPERANDS_TILED)
    _gemm_ex(args, x.device, workspace)
    return out


# ------------------------------------------------------------------------------------- attention
def attention_workspace(n_rows, n_keys, head_dim, groups, device):
    """Scratch for `attention` (partial results of the key tiles); needs no initialisation."""
    n = int(_lib.load().tpb200_attention_workspace_size(int(n_rows), int(n_keys), int(head_dim), int(groups)))
    if n == 0:
        raise TurboPiError("attention: unsupported shape")
    return torch.empty(n, dtype=torch.uint8, device=device)


def attention(q, k, v, out, scale, key_bias=None, workspace=None, quant=None, rows_per_token=1):
    """out = softmax(scale * q k^T + key_bias) v on the tensor cores; bf16 tensors.
    q / out: [rows, D] or [A, B, rows, D] views (any strides with a unit last stride); k / v: [keys, D] or
    [A, B, keys, D].  Gemma's grouped heads: pass q as the [tokens * heads, 256] view of the projection.
    `quant` (a tiled QuantBuf of [rows / rows_per_token, rows_per_token * D]): the result is also, or with
    out=None only, written as the operand of the next tensor-core GEMM -- what rowop(ROW_NONE, out, ...) would
    produce, without that launch (2-D problems only)."""
    _cuda(q, k, v, out, key_bias, workspace)
    if q.dim() == 2:
        q, k, v = q[None, None], k[None, None], v[None, None]
        out = None if out is None else out[None, None]
    if out is None and quant is None:
        raise TurboPiError("attention: neither out nor quant given")
    if not (q.dim() == k.dim() == v.dim() == 4 and (out is None or out.dim() == 4)):
        raise TurboPiError("attention: q, k, v, out must all be 2-D or all 4-D")
    for t in (q, k, v, out):
        if t is not None and (t.dtype != torch.bfloat16 or t.stride(3) != 1):
            raise TurboPiError("attention: bf16 tensors with a contiguous last dimension")
    A, B, R, D = q.shape
    S = k.shape[2]
    if tuple(k.shape) != (A, B, S, D) or tuple(v.shape) != (A, B, S, D) or (out is not None and tuple(out.shape) != (A, B, R, D)):
        raise TurboPiError("attention: shapes of q, k, v, out do not agree")
    if key_bias is not None and (key_bias.dtype != torch.bfloat16 or key_bias.numel() < S or not key_bias.is_contiguous()):
        raise TurboPiError("attention: key_bias must be a contiguous bf16 vector with one entry per key")
    if quant is not None:
        if A * B != 1 or R % rows_per_token or quant.M != R // rows_per_token or quant.K != rows_per_token * D:
            raise TurboPiError("attention: quant must be a QuantBuf of [rows / rows_per_token, rows_per_token * D]")
    if workspace is None:
        workspace = attention_workspace(R, S, D, A * B, q.device)
    two = ctypes.c_longlong * 2
    o = q if out is None else out          # strides only; the pointer stays NULL without `out`
    args = _lib.AttentionArgs(q=_ptr(q), k=_ptr(k), v=_ptr(v), out=_ptr(out), key_bias=_ptr(key_bias), n_rows=R, n_keys=S,
                              head_dim=D, ldq=q.stride(2), ldk=k.stride(2), ldv=v.stride(2), ldo=o.stride(2),
                              groups_outer=A, groups_inner=B, q_stride=two(q.stride(0), q.stride(1)),
                              k_stride=two(k.stride(0), k.stride(1)), v_stride=two(v.stride(0), v.stride(1)),
                              o_stride=two(o.stride(0), o.stride(1)), scale=float(scale), workspace=_ptr(workspace),
                              workspace_bytes=workspace.numel(), flags=_launch_flags,
                              quant_image=_ptr(quant.packed) if quant is not None else None,
                              quant_row_scale=_ptr(quant.row_scale) if quant is not None else None,
                              quant_pieces=quant.pieces if quant is not None else 0, quant_rows_per_token=rows_per_token,
                              quant_sf=_ptr(quant.sf) if quant is not None and not quant.tiled else None,
                              quant_pitch=quant.pitch if quant is not None else 0,
                              quant_piece_rows=quant.piece_rows if quant is not None else 0)
    with torch.cuda.device(q.device):
        st = _lib.load().tpb200_attention(ctypes.byref(args), torch.cuda.current_stream(q.device).cuda_stream)
    _lib.check(st, "tpb200_attention")
    return out


# ------------------------------------------------------------------------------------- tensor-core GEMV
class TcGemv:
    """NVFP4 weight-only GEMV(s) for M <= 16 tokens on the tensor cores.  Built once from a list of
    problems (dicts: weight_packed [N, K/2] uint8, weight_scales [N, K/16] E4M3 bytes, global_scale,
    x [M, K], out [M, N], optional bias; or `w_image` = the tiled weight image of tile_weights(), the
    same one the tensor-core GEMM streams); weights are tiled at construction.

    `fused=True` (default): `launch()` is ONE kernel, which quantises the activations it needs inside the
    launch.  `fused=False`: `launch()` first writes every distinct activation tensor as residual pieces to
    an image in global memory (one quantiser launch), then runs the GEMV on those."""

    def __init__(self, problems, pieces=3, activation=ACT_NONE, pdl=False, fused=True):
        if not 1 <= len(problems) <= _lib.MAX_GROUP:
            raise TurboPiError(f"1..{_lib.MAX_GROUP} problems per launch")
        p0 = problems[0]
        self.device = p0["x"].device
        self.M = p0["x"].shape[0]
        self.pieces = pieces
        self.fused = fused
        self.activation = int(activation)
        self.flags = FLAG_PDL if pdl else FLAG_NONE
        self.out_dtype = _dt(p0["out"])
        self.x_dtype = _dt(p0["x"])
        self.bias_dtype = _dt(p0["bias"]) if p0.get("bias") is not None else F32
        self._keep = []
        self._acts = {}           # x.data_ptr() -> (x, image, row_scale, K)
        lib = _lib.load()
        arr = ((_lib.GemvTcFusedProblem if fused else _lib.GemvTcProblem) * len(problems))()
        for i, p in enumerate(problems):
            x, out = p["x"], p["out"]
            _cuda(x, out, p.get("bias"))
            if x.shape[0] != self.M or _dt(x) != self.x_dtype or x.stride(1) != 1:
                raise TurboPiError("every problem of a launch takes [M, K] activations of one dtype")
            K = x.shape[1]
            if "w_image" in p:
                w_image, N = p["w_image"], out.shape[1]
                _cuda(w_image)
            else:
                w, ws = p["weight_packed"], p["weight_scales"]
                _cuda(w, ws)
                N = w.shape[0]
                b = torch.zeros((N, packed_pitch(K)), dtype=torch.uint8, device=self.device)
                b[:, :K // 2] = w[:, :K // 2]
                w_image = tile_weights(b, swizzle_scales(ws.view(torch.uint8)), N, K)
            self._keep.append((w_image, x, out, p.get("bias")))
            gs = float(p.get("global_scale", 1.0))
            if fused:
                arr[i] = _lib.GemvTcFusedProblem(_ptr(w_image), _ptr(x), x.stride(0), _ptr(p.get("bias")), _ptr(out), N, K,
                                                 out.stride(0), gs)
            else:
                key = x.data_ptr()
                if key not in self._acts:
                    nbytes = int(lib.tpb200_nvfp4_gemv_tc_x_image_bytes(K, pieces))
                    self._acts[key] = (x, torch.empty(nbytes, dtype=torch.uint8, device=self.device),
                                       torch.empty(16, dtype=torch.float32, device=self.device), K)
                _, xi, rs, _ = self._acts[key]
                arr[i] = _lib.GemvTcProblem(_ptr(w_image), _ptr(xi), _ptr(rs), _ptr(p.get("bias")), _ptr(out), N, K,
                                            out.stride(0), gs)
        self._arr = arr
        with torch.cuda.device(self.device):
            size = lib.tpb200_nvfp4_gemv_tc_fused_workspace_size if fused else lib.tpb200_nvfp4_gemv_tc_workspace_size
            nbytes = int(size(arr, len(arr)))
        if nbytes == 0:
            raise TurboPiError("the launch cannot be planned (unsupported shape or too many tiles for one launch)")
        self.workspace = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=self.device)

    def quantize(self):
        if self.fused:
            return
        lib = _lib.load()
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            acts = list(self._acts.values())
            for i in range(0, len(acts), 8):          # up to 8 activation tensors per launch
                chunk = acts[i:i + 8]
                arr = (_lib.ActTc * len(chunk))(*[_lib.ActTc(_ptr(x), x.stride(0), K, _ptr(xi), _ptr(rs))
                                                  for (x, xi, rs, K) in chunk])
                st = lib.tpb200_nvfp4_quantize_acts_tc(arr, len(chunk), _dt(chunk[0][0]), self.M, self.pieces,
                                                       self.flags, stream)
                _lib.check(st, "tpb200_nvfp4_quantize_acts_tc")

    def gemv(self):
        lib = _lib.load()
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            if self.fused:
                st = lib.tpb200_nvfp4_gemv_tc_fused(self._arr, len(self._arr), self.M, self.pieces, self.x_dtype,
                                                    self.bias_dtype, self.out_dtype, self.activation,
                                                    _ptr(self.workspace), self.workspace.numel(), self.flags, stream)
            else:
                st = lib.tpb200_nvfp4_gemv_tc(self._arr, len(self._arr), self.M, self.pieces, self.bias_dtype,
                                              self.out_dtype, self.activation, _ptr(self.workspace),
                                              self.workspace.numel(), self.flags, stream)
        _lib.check(st, "tpb200_nvfp4_gemv_tc")

    def gemv_static(self):
        """The GEMV through the entry point that uses the library's built-in scratch instead of
        `self.workspace` (for hosts that cannot allocate device memory); pre-tiled activations only."""
        if self.fused:
            raise TurboPiError("gemv_static takes pre-tiled activations: build the TcGemv with fused=False")
        with torch.cuda.device(self.device):
            st = _lib.load().tpb200_nvfp4_gemv_tc_static(self._arr, len(self._arr), self.M, self.pieces,
                                                         self.bias_dtype, self.out_dtype, self.activation, self.flags,
                                                         torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(st, "tpb200_nvfp4_gemv_tc_static")

    def launch(self):
        self.quantize()
        self.gemv()


def tc_gemv(x, w_image, N, out, global_scale=1.0, bias=None, activation=ACT_NONE, pieces=3, workspace=None, pdl=False):
    """One tensor-core GEMV launch without a prepared problem table: out[M, N] = act(gs * x @ W^T + bias)
    for M <= 16 rows, W given as its tiled image.  M <= 4 quantises the activations inside the launch; larger
    M goes through the stand-alone quantiser first (the in-launch quantiser keeps pace with the weight stream
    only for a few rows).  `workspace`: zeroed scratch of tc_gemv_workspace() bytes, reusable across calls
    that do not overlap; allocated here when omitted."""
    _cuda(x, w_image, out, bias, workspace)
    M, K = x.shape
    if not 1 <= M <= 16 or x.stride(1) != 1:
        raise TurboPiError("tc_gemv: 1..16 rows with a contiguous last dimension")
    lib = _lib.load()
    flags = FLAG_PDL if pdl else FLAG_NONE
    bias_dtype = _dt(bias) if bias is not None else F32
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        if M <= 4:
            arr = (_lib.GemvTcFusedProblem * 1)(_lib.GemvTcFusedProblem(_ptr(w_image), _ptr(x), x.stride(0), _ptr(bias), _ptr(out),
                                                                          N, K, out.stride(0), float(global_scale)))
            if workspace is None:
                workspace = torch.zeros(int(lib.tpb200_nvfp4_gemv_tc_fused_workspace_size(arr, 1)), dtype=torch.uint8,
                                        device=x.device)
            st = lib.tpb200_nvfp4_gemv_tc_fused(arr, 1, M, pieces, _dt(x), bias_dtype, _dt(out), int(activation),
                                                _ptr(workspace), workspace.numel(), flags, stream)
            _lib.check(st, "tpb200_nvfp4_gemv_tc_fused")
        else:
            xi = torch.empty(int(lib.tpb200_nvfp4_gemv_tc_x_image_bytes(K, pieces)), dtype=torch.uint8, device=x.device)
            rs = torch.empty(16, dtype=torch.float32, device=x.device)
            st = lib.tpb200_nvfp4_quantize_act_tc(_ptr(x), _dt(x), x.stride(0), _ptr(xi), _ptr(rs), M, K, pieces, flags, stream)
            _lib.check(st, "tpb200_nvfp4_quantize_act_tc")
            arr = (_lib.GemvTcProblem * 1)(_lib.GemvTcProblem(_ptr(w_image), _ptr(xi), _ptr(rs), _ptr(bias), _ptr(out), N, K,
                                                              out.stride(0), float(global_scale)))
            if workspace is None:
                workspace = torch.zeros(int(lib.tpb200_nvfp4_gemv_tc_workspace_size(arr, 1)), dtype=torch.uint8,
                                        device=x.device)
            st = lib.tpb200_nvfp4_gemv_tc(arr, 1, M, pieces, bias_dtype, _dt(out), int(activation), _ptr(workspace),
                                          workspace.numel(), flags, stream)
            _lib.check(st, "tpb200_nvfp4_gemv_tc")
    return out


def tc_gemv_workspace(N, K, device):
    """Zeroed scratch for tc_gemv() on an [N, K] weight (the plan does not depend on the row count)."""
    arr = (_lib.GemvTcFusedProblem * 1)(_lib.GemvTcFusedProblem(0, 0, 0, 0, 0, N, K, 0, 1.0))
    with torch.cuda.device(device):
        n = int(_lib.load().tpb200_nvfp4_gemv_tc_fused_workspace_size(arr, 1))
    return torch.zeros(max(n, 256), dtype=torch.uint8, device=device)
