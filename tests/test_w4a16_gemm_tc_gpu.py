"""INT4 x bf16 GEMM on the tensor cores (weights dequantised to bf16 inside the kernel) against the oracle:
the plugin launcher `w4a16GemmForward` at prefill sizes (openpi/w4a16_plugin/src/w4a16_gemm_plugin.h:41-59),
with zero points, alpha and beta, and `W4A16Linear` on the reference packer's buffers
(openpi/src/openpi/modules/w4a16_linear.py:201-268)."""
import numpy as np
import pytest
import torch

from conftest import cosine, rel_err
from oracle import formats, int4

pytestmark = pytest.mark.gpu


def _dev(a, device, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return t if dtype is None else t.to(dtype)


@pytest.mark.parametrize("M,N,K,use_zero,beta", [(64, 640, 1024, False, 0.0), (256, 384, 2048, True, 0.0), (712, 2048, 2048, False, 0.0),
                                                 (712, 512, 1024, True, 0.5), (17, 128, 128, False, 0.0), (300, 136, 256, False, 1.0)])
def test_plugin_gemm_forward_on_tensor_cores(cuda_device, M, N, K, use_zero, beta):
    from turbopi_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(M + N + K)
    w = formats.round_to_bf16(rng.uniform(-1, 1, size=(N, K)).astype(np.float32))
    packed, scales, zeros = int4.plugin_quantize_int4(w, 128)
    if use_zero:
        zeros = formats.round_to_bf16(rng.normal(size=zeros.shape).astype(np.float32) * 0.05)
    x = formats.round_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    c0 = formats.round_to_bf16(rng.normal(size=(M, N)).astype(np.float32))
    out = _dev(c0, cuda_device, torch.bfloat16)
    d = dict(x=_dev(x, cuda_device, torch.bfloat16), p=_dev(packed.view(np.uint8), cuda_device),
             s=_dev(scales, cuda_device, torch.bfloat16), z=_dev(zeros, cuda_device, torch.bfloat16))
    lib.w4a16GemmForward(d["x"].data_ptr(), d["p"].data_ptr(), d["s"].data_ptr(), d["z"].data_ptr() if use_zero else None,
                         out.data_ptr(), M, N, K, 0.75, beta, None, 0, torch.cuda.current_stream().cuda_stream)
    _lib.check_void("w4a16GemmForward")
    torch.cuda.synchronize()
    assert lib.tpb200_device_error(0) == 0
    ref = int4.plugin_gemm(x, packed, scales, zeros if use_zero else None, 128, 0.75, beta, c0)
    y = out.float().cpu().numpy()
    err = np.abs(y - ref).max(axis=1) / np.abs(ref).max(axis=1)         # per token row
    assert err.max() <= 1e-2, err.max()
    assert cosine(y, ref) >= 0.999


@torch.no_grad()
@pytest.mark.parametrize("T", [1, 16, 17, 200, 712])
def test_w4a16_linear_dispatches_on_token_count(cuda_device, T):
    """Same module, same buffers: decode GEMV up to 16 tokens, one tensor-core GEMM launch beyond."""
    from turbopi_b200 import _lib
    from turbopi_b200.w4a16 import W4A16Linear
    g = torch.Generator().manual_seed(T)
    lin = torch.nn.Linear(1024, 768, bias=True)
    lin.weight.data = torch.randn(768, 1024, generator=g) * 0.05
    lin.bias.data = torch.randn(768, generator=g) * 0.1
    layer = W4A16Linear.from_linear(lin.to(cuda_device))
    x = torch.randn(T, 1024, generator=g).to(torch.bfloat16)
    y = layer(x.to(cuda_device))
    assert y.shape == (T, 768) and y.dtype == torch.bfloat16
    assert _lib.load().tpb200_device_error(0) == 0
    ref = int4.gemv_dequant_matmul(x.float().numpy(), layer.weight_packed.cpu().numpy(), layer.scales.cpu().numpy(), "kblock")
    ref = ref + lin.bias.data.cpu().numpy()[None, :]
    assert rel_err(y.float().cpu().numpy(), ref) <= 1e-2
    assert cosine(y.float().cpu().numpy(), ref) >= 0.999


def test_w4a16_gemm_refuses_bad_shapes(cuda_device):
    from turbopi_b200 import ops
    from turbopi_b200._lib import TurboPiError
    x = torch.zeros((32, 96), dtype=torch.bfloat16, device=cuda_device)          # K not a multiple of 128
    w = torch.zeros((3, 64, 4), dtype=torch.int32, device=cuda_device)
    s = torch.zeros((3, 64), dtype=torch.float16, device=cuda_device)
    with pytest.raises(TurboPiError):
        ops.w4a16_gemm(x, w, s)
