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
