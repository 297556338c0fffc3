"""Plugin quantisers against the REFERENCE's own CUDA kernels, bit for bit.

oracle/_ref/libref_w4a16.so and libref_w4a8.so are the reference's translation units
(openpi/w4a16_plugin/src/w4a16_gemm_kernel.cu, openpi/w4a8_plugin/src/w4a8_gemm_kernel.cu) compiled unmodified
by oracle/build_ref.py.  Only their plain-CUDA quantiser entry points are called here; both libraries export
the same symbol names as ours, so each is loaded into its own namespace."""
import ctypes
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
REF = Path(__file__).resolve().parent.parent / "oracle" / "_ref"
P = ctypes.c_void_p


def _ref(name):
    path = REF / name
    if not path.exists():
        pytest.skip(f"{path} not built (oracle/build_ref.py needs the reference checkout)")
    return ctypes.CDLL(str(path), mode=ctypes.RTLD_LOCAL)


def _weights(N, K, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.05
    w[1, :128] = 0.0                                    # an all-zero group
    w[2, 5] = 0.35                                      # a group dominated by one value
    w[3, :128] = torch.linspace(-0.7, 0.7, 128)         # exact ties after scaling by max / 7
    return w.to(torch.bfloat16)


@pytest.mark.parametrize("N,K,group", [(16, 256, 128), (48, 1024, 128), (8, 512, 64)])
def test_int4_weight_quantiser_and_dequantiser_equal_reference_cuda(cuda_device, N, K, group):
    from turbopi_b200 import _lib
    ref, ours = _ref("libref_w4a16.so"), _lib.load()
    w = _weights(N, K, N + K).to(cuda_device)
    G = K // group
    stream = torch.cuda.current_stream().cuda_stream
    out = {}
    for tag, lib in (("ref", ref), ("ours", ours)):
        packed = torch.zeros((N, K // 2), dtype=torch.int8, device=cuda_device)
        scales = torch.zeros((N, G), dtype=torch.bfloat16, device=cuda_device)
        zeros = torch.full((N, G), 9.0, dtype=torch.bfloat16, device=cuda_device)
        deq = torch.zeros((N, K), dtype=torch.bfloat16, device=cuda_device)
        q, d = lib.quantizeWeightToINT4, lib.dequantizeINT4ToBF16
        q.restype = d.restype = None
        q.argtypes = [P, P, P, P, ctypes.c_int, ctypes.c_int, ctypes.c_int, P]
        d.argtypes = [P, P, P, P, ctypes.c_int, ctypes.c_int, ctypes.c_int, P]
        q(w.data_ptr(), packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(), N, K, group, stream)
        d(packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(), deq.data_ptr(), N, K, group, stream)
        torch.cuda.synchronize()
        out[tag] = (packed.cpu(), scales.cpu(), zeros.cpu(), deq.cpu())
    for a, b, what in zip(out["ref"], out["ours"], ("codes", "scales", "zeros", "dequantised")):
        assert torch.equal(a, b), what


@pytest.mark.parametrize("M,K", [(4, 256), (33, 512)])
def test_fp8_activation_quantiser_equals_reference_cuda(cuda_device, M, K):
    """K <= 512: the reference's launch covers only the first 32 blocks of a row; ours covers every block and
    must agree with it on those it does cover."""
    from turbopi_b200 import _lib
    ref, ours = _ref("libref_w4a8.so"), _lib.load()
    g = torch.Generator().manual_seed(M * K)
    x = (torch.randn(M, K, generator=g) * torch.rand(M, 1, generator=g) * 8).to(torch.bfloat16).to(cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    got = {}
    for tag, lib in (("ref", ref), ("ours", ours)):
        vals = torch.zeros((M, K), dtype=torch.uint8, device=cuda_device)
        sc = torch.zeros((M, K // 16), dtype=torch.uint8, device=cuda_device)
        f = lib.quantizeActivationToFP8
        f.restype = None
        f.argtypes = [P, P, P, ctypes.c_int, ctypes.c_int, P]
        f(x.data_ptr(), vals.data_ptr(), sc.data_ptr(), M, K, stream)
        torch.cuda.synchronize()
        got[tag] = (vals.cpu(), sc.cpu())
    assert torch.equal(got["ref"][1], got["ours"][1]), "scales"
    assert torch.equal(got["ref"][0], got["ours"][0]), "values"


@pytest.mark.parametrize("N,K", [(64, 256), (200, 1024)])
def test_nvfp4_weight_quantiser_equals_reference_cuda(cuda_device, N, K):
    from turbopi_b200 import _lib
    ref, ours = _ref("libref_w4a8.so"), _lib.load()
    w = _weights(N, K, 7 * N + K).to(cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    got = {}
    for tag, lib in (("ref", ref), ("ours", ours)):
        packed = torch.zeros((K // 2, N), dtype=torch.uint8, device=cuda_device)
        sc = torch.zeros((K // 16, N), dtype=torch.uint8, device=cuda_device)
        f = lib.quantizeWeightToNVFP4
        f.restype = None
        f.argtypes = [P, P, P, ctypes.c_int, ctypes.c_int, P]
        f(w.data_ptr(), packed.data_ptr(), sc.data_ptr(), N, K, stream)
        torch.cuda.synchronize()
        got[tag] = (packed.cpu(), sc.cpu())
    assert torch.equal(got["ref"][1], got["ours"][1]), "scales"
    assert torch.equal(got["ref"][0], got["ours"][0]), "codes"


@pytest.mark.parametrize("M,N,K", [(1, 512, 1024), (3, 4096, 1024), (2, 1024, 4096)])
@pytest.mark.parametrize("act,with_bias", [(0, False), (0, True), (1, True), (2, True)])
def test_nvfp4_gemv_forward_equals_reference_cuda(cuda_device, M, N, K, act, with_bias):
    """nvfp4_gemv_forward (the TensorRT plugin's launcher, fp32 tensors, fp32 block-32 scales on weights AND
    activations, optional bias + GELU / SiLU) against the reference's own kernels
    (openpi/nvfp4_packed_plugin/src/nvfp4_packed_kernel.cu, compiled unmodified).  The reference multiplies in
    fp32; the kernel here carries scaled activations as fp16 pairs (relative rounding 2^-11 per product, fp32
    sums), so the outputs agree to a few 1e-4 of the largest output -- far inside the 1e-2 bound of the
    specification, but not bit for bit.  Prints both kernels' device times on this GPU."""
    from oracle import nvfp4
    from turbopi_b200 import _lib
    ref, ours = _ref("libref_nvfp4_packed.so"), _lib.load()
    rng = np.random.default_rng(M * 7 + N + K + act)
    q, s = nvfp4.quantize_to_nvfp4((rng.normal(size=(N, K)) * 0.02).astype(np.float32), 32)
    packed = torch.from_numpy(nvfp4.pack_nvfp4(q)).to(cuda_device)
    sw = torch.from_numpy(s).to(cuda_device)
    xq, xs = nvfp4.quantize_to_nvfp4(rng.normal(size=(M, K)).astype(np.float32), 32)
    a, sa = torch.from_numpy(xq).to(cuda_device), torch.from_numpy(xs).to(cuda_device)
    bias = torch.from_numpy(rng.normal(size=(N,)).astype(np.float32)).to(cuda_device) if with_bias else None
    stream = torch.cuda.current_stream().cuda_stream
    outs, times = {}, {}
    for tag, lib in (("ref", ref), ("ours", ours)):
        f = lib.nvfp4_gemv_forward
        f.restype = None
        f.argtypes = [P, P, P, P, P, P, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, P]
        out = torch.zeros((M, N), dtype=torch.float32, device=cuda_device)
        call = lambda: f(a.data_ptr(), packed.data_ptr(), sa.data_ptr(), sw.data_ptr(),
                         bias.data_ptr() if bias is not None else None, out.data_ptr(), M, N, K, act, 0, stream)
        call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            call()
        e1.record()
        torch.cuda.synchronize()
        outs[tag], times[tag] = out.cpu().numpy(), e0.elapsed_time(e1) / 20 * 1e3
    assert ours.tpb200_last_error() == 0 and ours.tpb200_device_error(0) == 0
    scale = np.abs(outs["ref"]).max()
    assert np.abs(outs["ours"] - outs["ref"]).max() <= 2e-3 * scale
    print(f"nvfp4_gemv_forward M={M} N={N} K={K} act={act}: reference kernel {times['ref']:.1f} us, ours {times['ours']:.1f} us")


def _ref_ext(name):
    from oracle import build_ref
    mod = build_ref.load_torch_ext(name)
    if mod is None:
        pytest.skip(f"oracle/_ref/{name} not built (oracle/build_ref.py needs the reference checkout)")
    return mod


@pytest.mark.parametrize("M,N,K", [(1, 4096, 1024), (1, 1024, 4096), (4, 512, 2048), (16, 256, 1024)])
@pytest.mark.parametrize("act", [0, 1, 2])
def test_nvfp4_gemv_v6_equals_reference_extension(cuda_device, M, N, K, act):
    """ops.nvfp4_gemv_v6 against the reference's production GEMV (nvfp4_gemv_v6 of
    openpi/nvfp4_packed_plugin/src/nvfp4_gemv_v5.cu, built unmodified with its --use_fast_math): same argument
    list, same fp32 [M, N] result to a few 1e-4 of the largest output (fp16 activation pairs here, fp32 there)."""
    from oracle import nvfp4
    from turbopi_b200 import _lib, ops
    ext = _ref_ext("ref_nvfp4_gemv_v5")
    rng = np.random.default_rng(M + N + K + act)
    q, s = nvfp4.quantize_to_nvfp4((rng.normal(size=(N, K)) * 0.02).astype(np.float32), 32)
    packed = torch.from_numpy(nvfp4.pack_nvfp4(q)).to(cuda_device)
    sw = torch.from_numpy(s).to(cuda_device)
    x = torch.from_numpy(rng.normal(size=(M, K)).astype(np.float32)).to(cuda_device)
    bias = torch.from_numpy(rng.normal(size=(N,)).astype(np.float32)).to(cuda_device)
    want = ext.nvfp4_gemv_v6(x, packed, sw, bias, M, N, K, act)
    got = ops.nvfp4_gemv_v6(x, packed, sw, bias, M, N, K, act)
    torch.cuda.synchronize()
    assert _lib.load().tpb200_device_error(0) == 0
    assert got.shape == want.shape and got.dtype == want.dtype == torch.float32
    assert (got - want).abs().max().item() <= 2e-3 * want.abs().max().item()


@pytest.mark.parametrize("hidden", [2048, 1024])
def test_fused_qkv_fp4_equals_reference_extension(cuda_device, hidden):
    """kv_fuse.fused_qkv_fp4 (Q returned, K / V rows written in place at cache[b, cache_pos, 0, :], no RoPE, fp32)
    against the reference's kernel (openpi/kv_fuse_plugin/src/fused_qkv_fp4.cu, built unmodified): Q and the
    caches agree, and nothing but the addressed cache rows changes."""
    from turbopi_b200 import kv_fuse
    ext = _ref_ext("ref_fused_qkv_fp4")
    B, H, KVH, D, S, pos = 2, 8, 1, 256, 16, 5
    g = torch.Generator().manual_seed(hidden)
    ws = []
    for n in (H * D, KVH * D, KVH * D):
        packed, sc = kv_fuse.quantize_to_fp4(torch.randn(n, hidden, generator=g) * 0.02)
        ws += [packed.to(cuda_device), sc.to(cuda_device)]
    x = torch.randn(B, hidden, generator=g).to(cuda_device)
    res = {}
    for tag, fn in (("ref", ext.fused_qkv_fp4), ("ours", kv_fuse.fused_qkv_fp4)):
        kc = torch.full((B, S, KVH, D), -7.0, device=cuda_device)
        vc = torch.full((B, S, KVH, D), -7.0, device=cuda_device)
        qo = fn(x, *ws, kc, vc, hidden, H, KVH, D, pos)
        torch.cuda.synchronize()
        res[tag] = (qo.float().cpu(), kc.cpu(), vc.cpu())
    for a, b in zip(res["ref"], res["ours"]):
        assert (a - b).abs().max().item() <= 2e-3 * a.abs().max().item()
    for t in res["ours"][1:]:
        mask = torch.ones_like(t, dtype=torch.bool)
        mask[:, pos] = False
        assert (t[mask] == -7.0).all()


@pytest.mark.parametrize("M,N,K", [(1, 2048, 1024), (3, 512, 4096)])
@pytest.mark.parametrize("act", [0, 1, 2])
def test_nvfp4_gemv_torch_variants_equal_reference_extension(cuda_device, M, N, K, act):
    """ops.nvfp4_gemv (per-block activation scales) and ops.nvfp4_gemv_w4a16 against the reference's
    nvfp4_packed_torch.cu extension (openpi/nvfp4_packed_plugin/src/nvfp4_packed_torch.cu:173-290), built unmodified."""
    from oracle import nvfp4
    from turbopi_b200 import ops
    ext = _ref_ext("ref_nvfp4_packed_torch")
    rng = np.random.default_rng(M * 31 + N + K + act)
    q, s = nvfp4.quantize_to_nvfp4((rng.normal(size=(N, K)) * 0.02).astype(np.float32), 32)
    packed = torch.from_numpy(nvfp4.pack_nvfp4(q)).to(cuda_device)
    sw = torch.from_numpy(s).to(cuda_device)
    bias = torch.from_numpy(rng.normal(size=(N,)).astype(np.float32)).to(cuda_device)
    x = torch.from_numpy(rng.normal(size=(M, K)).astype(np.float32)).to(cuda_device)
    xq, xs = nvfp4.quantize_to_nvfp4(rng.normal(size=(M, K)).astype(np.float32), 32)
    a, sa = torch.from_numpy(xq).to(cuda_device), torch.from_numpy(xs).to(cuda_device)
    pairs = [(ext.nvfp4_gemv_w4a16(x, packed, sw, bias, M, N, K, act), ops.nvfp4_gemv_w4a16(x, packed, sw, bias, M, N, K, act)),
             (ext.nvfp4_gemv(a, packed, sa, sw, bias, M, N, K, act), ops.nvfp4_gemv(a, packed, sa, sw, bias, M, N, K, act))]
    torch.cuda.synchronize()
    for want, got in pairs:
        assert got.shape == want.shape
        assert (got.float() - want.float()).abs().max().item() <= 2e-3 * want.float().abs().max().item()
