"""The reference-named TensorRT-plugin launchers (void, caller-owned workspace) against the oracle."""
import numpy as np
import pytest
import torch

from conftest import cosine, rel_err
from oracle import formats, int4, nvfp4, w4a8

pytestmark = pytest.mark.gpu


def _dev(a, device, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return t if dtype is None else t.to(dtype)


def test_int4_quantise_dequantise_kernels(cuda_device):
    from turbopi_b200 import ops
    rng = np.random.default_rng(0)
    w = formats.round_to_bf16(rng.uniform(-1, 1, size=(96, 512)).astype(np.float32))
    packed, scales, zeros = ops.quantize_weight_to_int4(_dev(w, cuda_device, torch.bfloat16), 128)
    op, os_, oz = int4.plugin_quantize_int4(w, 128)
    assert np.array_equal(scales.float().cpu().numpy(), os_)
    assert np.array_equal(packed.cpu().numpy(), op)                     # every code, every nibble
    assert (zeros.float() == 0).all()
    deq = ops.dequantize_int4_to_bf16(packed, scales, zeros, 128)
    assert np.array_equal(deq.float().cpu().numpy(), int4.plugin_dequantize_int4(op, os_, oz, 128))


def test_nvfp4_and_fp8_quantiser_kernels(cuda_device):
    from turbopi_b200 import ops
    rng = np.random.default_rng(1)
    w = formats.round_to_bf16((rng.normal(size=(72, 256)) * 0.02).astype(np.float32))
    w[3, :16] = 0.0
    pt, st = ops.quantize_weight_to_nvfp4(_dev(w, cuda_device, torch.bfloat16))
    opt, ost = nvfp4.plugin_quantize_weight_nvfp4(w)
    assert np.array_equal(pt.cpu().numpy(), opt) and np.array_equal(st.cpu().numpy(), ost)
    x = formats.round_to_bf16(rng.normal(size=(9, 1024)).astype(np.float32))       # 64 blocks per row
    v, s = ops.quantize_activation_to_fp8(_dev(x, cuda_device, torch.bfloat16))
    ov, os_ = w4a8.quantize_activation_fp8(x)
    assert np.array_equal(s.cpu().numpy(), os_) and np.array_equal(v.cpu().numpy(), ov)


@pytest.mark.parametrize("M,use_zero,beta", [(1, False, 0.0), (20, False, 0.0), (5, True, 0.5), (256, False, 0.0)])
def test_w4a16_gemm_forward(cuda_device, M, use_zero, beta):
    from turbopi_b200 import _lib, ops
    lib = _lib.load()
    rng = np.random.default_rng(M)
    N, K = 640, 1024
    w = formats.round_to_bf16(rng.uniform(-1, 1, size=(N, K)).astype(np.float32))
    packed, scales, zeros = int4.plugin_quantize_int4(w, 128)
    if use_zero:
        zeros = formats.round_to_bf16(rng.normal(size=zeros.shape).astype(np.float32) * 0.05)
    x = formats.round_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    c0 = formats.round_to_bf16(rng.normal(size=(M, N)).astype(np.float32))
    out = _dev(c0, cuda_device, torch.bfloat16)
    d = dict(x=_dev(x, cuda_device, torch.bfloat16), p=_dev(packed.view(np.uint8), cuda_device),
             s=_dev(scales, cuda_device, torch.bfloat16), z=_dev(zeros, cuda_device, torch.bfloat16))
    nws = lib.getW4A16GemmWorkspaceSize(M, N, K)
    ws = torch.empty(nws, dtype=torch.uint8, device=cuda_device)
    lib.w4a16GemmForward(d["x"].data_ptr(), d["p"].data_ptr(), d["s"].data_ptr(), d["z"].data_ptr() if use_zero else None,
                         out.data_ptr(), M, N, K, 0.75, beta, ws.data_ptr(), nws, torch.cuda.current_stream().cuda_stream)
    _lib.check_void("w4a16GemmForward")
    ref = int4.plugin_gemm(x, packed, scales, zeros if use_zero else None, 128, 0.75, beta, c0)
    y = out.float().cpu().numpy()
    assert rel_err(y, ref) <= 1e-2 and cosine(y, ref) >= 0.999


@pytest.mark.parametrize("M,N,K", [(64, 256, 512), (300, 2048, 2048), (7, 136, 272)])
def test_w4a8_gemm_forward(cuda_device, M, N, K):
    from turbopi_b200 import _lib, ops
    lib = _lib.load()
    rng = np.random.default_rng(M + N)
    w = formats.round_to_bf16((rng.normal(size=(N, K)) * 0.05).astype(np.float32))
    x = formats.round_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    wp_t, ws_t = ops.quantize_weight_to_nvfp4(_dev(w, cuda_device, torch.bfloat16))
    a8, sa = ops.quantize_activation_to_fp8(_dev(x, cuda_device, torch.bfloat16))
    out = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_device)
    nws = lib.getW4A8GemmWorkspaceSize(M, N, K)
    ws = torch.empty(nws, dtype=torch.uint8, device=cuda_device)
    lib.w4a8GemmForward(a8.data_ptr(), sa.data_ptr(), wp_t.data_ptr(), ws_t.data_ptr(), out.data_ptr(), M, N, K, 0.5,
                        ws.data_ptr(), nws, torch.cuda.current_stream().cuda_stream)
    _lib.check_void("w4a8GemmForward")
    assert lib.tpb200_device_error(0) == 0
    ref = w4a8.gemm(a8.cpu().numpy(), sa.cpu().numpy(), wp_t.cpu().numpy(), ws_t.cpu().numpy(), 0.5)
    y = out.float().cpu().numpy()
    assert rel_err(y, ref) <= 1e-2 and cosine(y, ref) >= 0.999
