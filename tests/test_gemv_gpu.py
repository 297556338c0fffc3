"""Parity of the decode-shaped 4-bit GEMV kernels (through the C ABI) with the CPU oracle.

Tolerances are the ones the path is specified with: max|y - ref| / max|ref| <= 1e-2 and
cosine >= 0.999 against the dequantise-then-matmul reference (fp32 accumulation on the
device, float64 in the oracle).  Packing and decode are checked bit-exactly.
"""
import numpy as np
import pytest
import torch

from conftest import cosine, rel_err
from oracle import formats, int4, nvfp4

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2
COS_TOL = 0.999


def _check(y, ref):
    assert np.isfinite(y).all()
    assert rel_err(y, ref) <= REL_TOL, rel_err(y, ref)
    assert cosine(y, ref) >= COS_TOL, cosine(y, ref)


def _dev(a, device, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return t if dtype is None else t.to(dtype)


def _bf16(a):
    return formats.round_to_bf16(np.asarray(a, dtype=np.float32))


def _canary_out(M, N, dtype, device):
    """Output buffer framed by sentinel rows to catch out-of-bounds stores."""
    buf = torch.full((M + 32, N), -12345.0, dtype=dtype, device=device)   # 16 rows in front keep `out` 16-byte aligned
    return buf, buf[16:16 + M]


def _canary_ok(buf):
    M = buf.shape[0] - 32
    return bool((buf[:16] == -12345.0).all() and (buf[16 + M:] == -12345.0).all())


# --------------------------------------------------------------------------- decode tables
def test_e2m1_decode_all_byte_values_exact(cuda_device):
    from turbopi_b200 import ops
    N, K = 256, 32
    packed = np.zeros((N, K // 2), dtype=np.uint8)
    packed[:, 0] = np.arange(256)
    packed[:, 7] = np.arange(256)[::-1]
    x = np.zeros((1, K), dtype=np.float32)
    x[0, 0], x[0, 1], x[0, 14], x[0, 15] = 1.0, 16.0, 256.0, 4096.0
    scales = np.ones((N, 1), dtype=np.float32)
    out = torch.empty((1, N), dtype=torch.float32, device=cuda_device)
    ops.nvfp4_gemv_out(_dev(x, cuda_device), _dev(packed, cuda_device), _dev(scales, cuda_device), out, block_size=32)
    ref = nvfp4.gemv_dequant_matmul(x, packed, scales, block_size=32)
    assert np.array_equal(out.cpu().numpy().astype(np.float64), ref)   # small integers and halves: exact


def test_int4_decode_all_codes_exact(cuda_device):
    from turbopi_b200 import ops
    N, K = 16, 32
    codes = np.zeros((N, K), dtype=np.uint8)
    for n in range(N):
        codes[n] = (np.arange(K) + n) % 16
    words = int4._pack_words(codes, "rowmajor")
    scales = np.ones((N, 1), dtype=np.float16)
    for pos in range(K):
        x = np.zeros((1, K), dtype=np.float16)
        x[0, pos] = 1.0
        out = torch.empty((1, N), dtype=torch.float32, device=cuda_device)
        ops.w4a16_gemv_out(_dev(x, cuda_device), _dev(words, cuda_device), _dev(scales, cuda_device), out,
                           group_size=32, layout=1)
        assert np.array_equal(out.cpu().numpy()[0], codes[:, pos].astype(np.float32) - 8.0), pos
    kb = int4._pack_words(codes, "kblock")
    for pos in (0, 5, 12, 31):
        x = np.zeros((1, K), dtype=np.float16)
        x[0, pos] = 2.0
        out = torch.empty((1, N), dtype=torch.float32, device=cuda_device)
        ops.w4a16_gemv_out(_dev(x, cuda_device), _dev(kb, cuda_device), _dev(scales.T.copy(), cuda_device), out,
                           group_size=32, layout=0)
        assert np.array_equal(out.cpu().numpy()[0], 2.0 * (codes[:, pos].astype(np.float32) - 8.0)), pos


# --------------------------------------------------------------------------- W4A16 INT4
def test_w4a16_benchmark_config_rowmajor_g128(cuda_device):
    """x bf16 [1,2048] N(0,1); codes uniform 0..15, 8 per int32 along K, N=16384; fp16 scale per
    (n, 128 group) uniform [0.005, 0.02]; zero point 8; bf16 output."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(0)
    N, K, G = 16384, 2048, 128
    codes = rng.integers(0, 16, size=(N, K), dtype=np.uint8)
    words = int4._pack_words(codes, "rowmajor")
    scales = rng.uniform(0.005, 0.02, size=(N, K // G)).astype(np.float16)
    x = _bf16(rng.normal(size=(1, K)))
    buf, out = _canary_out(1, N, torch.bfloat16, cuda_device)
    ops.w4a16_gemv_out(_dev(x, cuda_device, torch.bfloat16), _dev(words, cuda_device), _dev(scales, cuda_device), out,
                       group_size=G, layout=1)
    ref = int4.gemv_dequant_matmul(x, words, scales, "rowmajor", G)
    _check(out.float().cpu().numpy(), ref)
    assert _canary_ok(buf)


@pytest.mark.parametrize("N,K,G", [(256, 2048, 128), (4096, 1024, 32), (48, 4096, 64), (1600, 2048, 2048), (16, 1024, 128),
                                   (9600, 1024, 64), (9488, 2048, 128)])     # the last two: several tiles per CTA
@pytest.mark.parametrize("xdt,sdt,with_bias", [(torch.bfloat16, np.float16, False), (torch.float16, np.float16, True),
                                               (torch.float32, "bf16", True)])
def test_w4a16_one_token_rowmajor_kernel(cuda_device, N, K, G, xdt, sdt, with_bias):
    """The single-token row-major kernel (K of 1024 / 2048 / 4096, any group that is a multiple of 32, fp16 or bf16
    scales, every activation dtype, optional bias, PDL flag) against the dequantise-then-matmul oracle; the words past
    the output stay untouched."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(N + K + G)
    codes = rng.integers(0, 16, size=(N, K), dtype=np.uint8)
    words = int4._pack_words(codes, "rowmajor")
    scales = rng.uniform(0.005, 0.02, size=(N, K // G)).astype(np.float32)
    if sdt == "bf16":
        scales = _bf16(scales)
        sc_dev = _dev(scales, cuda_device, torch.bfloat16)
    else:
        scales = scales.astype(np.float16)
        sc_dev = _dev(scales, cuda_device)
    x = rng.normal(size=(1, K)).astype(np.float32)
    x = _bf16(x) if xdt == torch.bfloat16 else x.astype(np.float16).astype(np.float32) if xdt == torch.float16 else x
    bias = rng.normal(size=(N,)).astype(np.float32) if with_bias else None
    ref = int4.gemv_dequant_matmul(x, words, scales.astype(np.float32), "rowmajor", G, bias)
    for pdl in (False, True):
        buf, out = _canary_out(1, N, torch.bfloat16, cuda_device)
        ops.w4a16_gemv_out(_dev(x, cuda_device, xdt), _dev(words, cuda_device), sc_dev, out,
                           bias=_dev(bias, cuda_device) if with_bias else None, group_size=G, layout=1, pdl=pdl)
        _check(out.float().cpu().numpy(), ref)
        assert _canary_ok(buf)


@pytest.mark.parametrize("N,K", [(16384, 2048), (2048, 16384), (100, 64), (64, 32), (1000, 4096)])
def test_w4a16_reference_layout_kblock(cuda_device, N, K):
    """The reference op's contract: fp16 (1,K) x (K/32,N,4) int32 + (K/32,N) fp16 -> fp32 (1,N)."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(N + K)
    w = rng.normal(size=(N, K)).astype(np.float32)
    packed, scales = int4.pack_fast(w)
    x = rng.normal(size=(1, K)).astype(np.float16)
    y = ops.w4a16_gemv(_dev(x, cuda_device), _dev(packed, cuda_device), _dev(scales, cuda_device))
    assert y.dtype == torch.float32 and tuple(y.shape) == (1, N)
    ref = int4.gemv_dequant_matmul(x, packed, scales, "kblock")
    _check(y.cpu().numpy(), ref)
    if N * K <= 100 * 64:     # the TVM kernel's own fp16 arithmetic, where the loop oracle is cheap
        _check(y.cpu().numpy(), int4.gemv_reference_math(x, packed, scales, "kblock"))
    with pytest.raises(ValueError):
        ops.w4a16_gemv(_dev(np.zeros((2, K), np.float16), cuda_device), _dev(packed, cuda_device),
                       _dev(scales, cuda_device))


@pytest.mark.parametrize("M", [1, 2, 3, 4, 7, 16])
@pytest.mark.parametrize("layout", [0, 1])
def test_w4a16_batched_rows_and_bias(cuda_device, M, layout):
    from turbopi_b200 import ops
    rng = np.random.default_rng(10 * M + layout)
    N, K = 520, 1024                  # N is not a multiple of any tile size
    w = rng.normal(size=(N, K)).astype(np.float32)
    name = "kblock" if layout == 0 else "rowmajor"
    packed, scales = int4.pack_fast(w, 32, name)
    x = _bf16(rng.normal(size=(M, K)))
    bias = rng.normal(size=(N,)).astype(np.float32)
    buf, out = _canary_out(M, N, torch.float32, cuda_device)
    ops.w4a16_gemv_out(_dev(x, cuda_device, torch.bfloat16), _dev(packed, cuda_device), _dev(scales, cuda_device), out,
                       bias=_dev(bias, cuda_device), group_size=32, layout=layout)
    ref = int4.gemv_dequant_matmul(x, packed, scales, name, 32, bias)
    _check(out.cpu().numpy(), ref)
    assert _canary_ok(buf)


# --------------------------------------------------------------------------- NVFP4
def _cfg2_weights(rng, N, K):
    """Benchmark configuration 2: E4M3 scale per 16 = blockamax/6 of an underlying N(0, 0.02)
    matrix (over an fp32 global scale); the codes themselves uniform over the 16 codes."""
    base = (rng.normal(size=(N, K)) * 0.02).astype(np.float32)
    _, sbytes, g = nvfp4.quantize_two_level(base, 16)
    packed = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    return packed, sbytes, float(g)


@pytest.mark.parametrize("M", [1, 4, 16])
@pytest.mark.parametrize("N,K", [(4096, 1024), (1024, 4096)])
def test_nvfp4_benchmark_config_action_expert_mlp(cuda_device, M, N, K):
    from turbopi_b200 import ops
    rng = np.random.default_rng(M * 7 + N)
    packed, sbytes, g = _cfg2_weights(rng, N, K)
    x = _bf16(rng.normal(size=(M, K)))
    buf, out = _canary_out(M, N, torch.bfloat16, cuda_device)
    ops.nvfp4_gemv_out(_dev(x, cuda_device, torch.bfloat16), _dev(packed, cuda_device), _dev(sbytes, cuda_device), out,
                       block_size=16, global_scale=g)
    ref = nvfp4.gemv_dequant_matmul(x, packed, sbytes, None, 0, 16, g, scale_is_e4m3=True)
    _check(out.float().cpu().numpy(), ref)
    assert _canary_ok(buf)


@pytest.mark.parametrize("N,K,M", [(16384, 2048, 1), (2048, 16384, 2), (2560, 2048, 1), (3072, 3072, 1),
                                   (37, 32, 5), (1, 64, 1), (333, 1056, 3), (8192, 8192, 4), (100, 32768, 1)])
def test_nvfp4_shapes_edge_cases(cuda_device, N, K, M):
    from turbopi_b200 import ops
    rng = np.random.default_rng(N * 3 + K + M)
    packed, sbytes, g = _cfg2_weights(rng, N, K)
    x = _bf16(rng.normal(size=(M, K)))
    buf, out = _canary_out(M, N, torch.float32, cuda_device)
    ops.nvfp4_gemv_out(_dev(x, cuda_device, torch.bfloat16), _dev(packed, cuda_device), _dev(sbytes, cuda_device), out,
                       block_size=16, global_scale=g)
    ref = nvfp4.gemv_dequant_matmul(x, packed, sbytes, None, 0, 16, g, scale_is_e4m3=True)
    _check(out.cpu().numpy(), ref)
    assert _canary_ok(buf)


@pytest.mark.parametrize("act", [0, 1, 2])
@pytest.mark.parametrize("xdt", [torch.float32, torch.float16, torch.bfloat16])
def test_nvfp4_reference_format_bias_activation(cuda_device, act, xdt):
    """block 32 + fp32 scales (the reference's buffers), fused bias + GELU-tanh / SiLU."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(act)
    N, K, M = 3072, 3072, 2
    w = (rng.normal(size=(N, K)) * 0.02).astype(np.float32)
    q, s = nvfp4.quantize_to_nvfp4(w, 32)
    packed = nvfp4.pack_nvfp4(q)
    x = rng.normal(size=(M, K)).astype(np.float32)
    xt = _dev(x, cuda_device, xdt)
    xr = xt.float().cpu().numpy()
    bias = (rng.normal(size=(N,)) * 0.5).astype(np.float32)
    out = torch.empty((M, N), dtype=torch.float32, device=cuda_device)
    ops.nvfp4_gemv_out(xt, _dev(packed, cuda_device), _dev(s, cuda_device), out, _dev(bias, cuda_device), act, 32)
    ref = nvfp4.gemv_dequant_matmul(xr, packed, s, bias, act, 32)
    _check(out.cpu().numpy(), ref)


def test_nvfp4_golden_vectors_from_reference(cuda_device, golden):
    """The reference's own _forward_dequant_gemm outputs on its own quantised weights."""
    from turbopi_b200 import ops
    g = golden("nvfp4_packed")
    for act in (0, 1, 2):
        y = ops.nvfp4_gemv_v6(_dev(g["x"], cuda_device), _dev(g["packed"], cuda_device), _dev(g["scales"], cuda_device),
                              _dev(g["bias"], cuda_device), 5, 40, 128, act)
        _check(y.cpu().numpy(), g[f"out_act{act}"])


def test_nvfp4_plugin_abi_and_activation_scales(cuda_device):
    """nvfp4_gemv_forward (void, reference signature) with per-block activation scales."""
    from turbopi_b200 import _lib, ops
    rng = np.random.default_rng(11)
    N, K, M = 512, 1024, 3
    w = (rng.normal(size=(N, K)) * 0.02).astype(np.float32)
    q, s = nvfp4.quantize_to_nvfp4(w, 32)
    packed = nvfp4.pack_nvfp4(q)
    xq, xs = nvfp4.quantize_to_nvfp4(rng.normal(size=(M, K)).astype(np.float32), 32)
    y = ops.nvfp4_gemv(_dev(xq, cuda_device), _dev(packed, cuda_device), _dev(xs, cuda_device), _dev(s, cuda_device),
                       None, M, N, K, 0)
    x_full = xq * np.repeat(xs, 32, axis=1)
    ref = nvfp4.gemv_dequant_matmul(x_full, packed, s, None, 0, 32)
    _check(y.cpu().numpy(), ref)
    out = torch.empty((M, N), dtype=torch.float32, device=cuda_device)
    a, p, sa, sw = (_dev(v, cuda_device) for v in (xq, packed, xs, s))
    _lib.load().nvfp4_gemv_forward(a.data_ptr(), p.data_ptr(), sa.data_ptr(), sw.data_ptr(), None, out.data_ptr(),
                                   M, N, K, 0, 0, torch.cuda.current_stream().cuda_stream)
    _lib.check_void("nvfp4_gemv_forward")
    assert torch.equal(out, y)
    assert _lib.load().nvfp4_gemv_workspace_size(M, N, K) == 0


def test_grouped_launch_and_pdl_chain_match_single_launches(cuda_device):
    from turbopi_b200 import ops
    rng = np.random.default_rng(21)
    shapes = [(4096, 1024), (4096, 1024), (1024, 4096)] * 3
    xs = {1024: _dev(_bf16(rng.normal(size=(1, 1024))), cuda_device, torch.bfloat16),
          4096: _dev(_bf16(rng.normal(size=(1, 4096))), cuda_device, torch.bfloat16)}
    probs, singles = [], []
    for N, K in shapes:
        packed, sbytes, g = _cfg2_weights(rng, N, K)
        p = dict(x=xs[K], weight_packed=_dev(packed, cuda_device), weight_scales=_dev(sbytes, cuda_device),
                 out=torch.zeros((1, N), dtype=torch.bfloat16, device=cuda_device), global_scale=g)
        probs.append(p)
        o = torch.empty((1, N), dtype=torch.bfloat16, device=cuda_device)
        ops.nvfp4_gemv_out(p["x"], p["weight_packed"], p["weight_scales"], o, block_size=16, global_scale=g)
        singles.append(o)
        ref = nvfp4.gemv_dequant_matmul(p["x"].float().cpu().numpy(), packed, sbytes, None, 0, 16, g, True)
        _check(o.float().cpu().numpy(), ref)
    ops.GroupedGemv(probs, 16).launch()
    for p, o in zip(probs, singles):
        assert rel_err(p["out"].float().cpu().numpy(), o.float().cpu().numpy()) < 4e-3   # bf16 rounding of a re-ordered sum
    # a dependent chain under programmatic dependent launch gives the same bytes as without it
    outs_pdl = [torch.empty_like(o) for o in singles]
    for p, o in zip(probs, outs_pdl):
        ops.nvfp4_gemv_out(p["x"], p["weight_packed"], p["weight_scales"], o, block_size=16,
                           global_scale=p["global_scale"], pdl=True)
    torch.cuda.synchronize()
    for a, b in zip(outs_pdl, singles):
        assert torch.equal(a, b)


@torch.no_grad()
def test_modules_forward_through_kernels(cuda_device):
    from turbopi_b200 import nvfp4_packed, w4a16
    torch.manual_seed(3)
    lin = torch.nn.Linear(1024, 768, bias=True).to(cuda_device)
    x = torch.randn(2, 21, 1024, device=cuda_device, dtype=torch.bfloat16)      # 42 tokens: three launches
    q = w4a16.W4A16Linear.from_linear(lin)
    y = q(x)
    assert y.shape == (2, 21, 768) and y.dtype == torch.bfloat16
    ref = torch.nn.functional.linear(x.float(), q.weight.float(), lin.bias.float())
    _check(y.float().cpu().numpy(), ref.cpu().numpy())
    for fmt in ("ref", "nvfp4"):
        n = nvfp4_packed.NVFP4PackedLinear.from_linear(lin, activation="gelu", fmt=fmt)
        y = n(x)
        sc = n.weight_scales.cpu().numpy()
        wd = nvfp4.dequantize(n.weight_packed.cpu().numpy(), sc, n.block_size, n.global_scale, fmt == "nvfp4")
        ref = torch.nn.functional.gelu(
            torch.nn.functional.linear(x.float().cpu(), torch.from_numpy(wd), lin.bias.float().cpu()),
            approximate="tanh")
        _check(y.float().cpu().numpy(), ref.numpy())
    mlp = torch.nn.Module()
    mlp.gate_proj = torch.nn.Linear(1024, 4096, bias=False).to(cuda_device)
    mlp.up_proj = torch.nn.Linear(1024, 4096, bias=False).to(cuda_device)
    mlp.down_proj = torch.nn.Linear(4096, 1024, bias=False).to(cuda_device)
    pm = nvfp4_packed.NVFP4PackedMLP.from_gemma_mlp(mlp, gate_activation="gelu", fmt="nvfp4")
    xin = torch.randn(1, 1024, device=cuda_device, dtype=torch.bfloat16)
    y = pm(xin)

    def deq(l):
        return torch.from_numpy(nvfp4.dequantize(l.weight_packed.cpu().numpy(), l.weight_scales.cpu().numpy(), 16,
                                                 l.global_scale, True))
    xf = xin.float().cpu()
    gate = torch.nn.functional.gelu(xf @ deq(pm.gate_proj).T, approximate="tanh").to(torch.bfloat16).float()
    up = (xf @ deq(pm.up_proj).T).to(torch.bfloat16).float()
    ref = ((gate * up).to(torch.bfloat16).float() @ deq(pm.down_proj).T)
    _check(y.float().cpu().numpy(), ref.numpy())


def test_no_kernel_gave_up_on_a_wait(cuda_device):
    from turbopi_b200 import _lib
    assert _lib.load().tpb200_device_error(0) == 0


def test_kv_fuse_module_matches_reference_golden(cuda_device, golden):
    """FusedQKVProjection on the reference's own quantised weights: Q and the cache rows against the output
    of its fallback path; every other cache row keeps the sentinel bit for bit."""
    from turbopi_b200 import kv_fuse
    g = golden("kv_fuse")
    mod = kv_fuse.FusedQKVProjection(64, 2, 1, 32, max_seq_len=6)
    for n in ("q", "k", "v"):
        setattr(mod, f"W{n}_packed", _dev(g[f"W{n}_packed"], cuda_device))
        setattr(mod, f"scale_W{n}", _dev(g[f"scale_W{n}"], cuda_device))
    # the packer is the reference's, bit for bit (sign from the input: code 8 appears)
    pk, sc = kv_fuse.quantize_to_fp4(torch.from_numpy(g["Wk"]), 32)
    assert np.array_equal(pk.numpy(), g["Wk_packed"]) and np.array_equal(sc.numpy(), g["scale_Wk"])
    Kc = torch.full((3, 6, 1, 32), -7.0, device=cuda_device)
    Vc = torch.full((3, 6, 1, 32), -7.0, device=cuda_device)
    pos = int(g["cache_pos"])
    Q, Kc2, Vc2 = mod(_dev(g["x"], cuda_device), Kc, Vc, pos)
    assert Kc2 is Kc and Vc2 is Vc                                  # updated in place
    _check(Q.cpu().numpy(), g["Q"])
    _check(Kc[:, pos].cpu().numpy(), g["K_cache"][:, pos])
    _check(Vc[:, pos].cpu().numpy(), g["V_cache"][:, pos])
    other = [i for i in range(6) if i != pos]
    assert (Kc[:, other] == -7.0).all() and (Vc[:, other] == -7.0).all()
