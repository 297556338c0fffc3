"""The allocation-free variant of the tensor-core GEMV (scratch built into the library) must give
what the workspace-taking entry point gives.  Collected last on purpose: if it fails, every other test
has already run."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


def _problem(rng, N, K, M, device):
    packed = torch.from_numpy(rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)).to(device)
    scales = torch.from_numpy(rng.integers(40, 120, size=(N, K // 16), dtype=np.uint8)).to(device)
    x = torch.from_numpy(rng.normal(size=(M, K)).astype(np.float32)).to(device).to(torch.bfloat16)
    return dict(x=x, weight_packed=packed, weight_scales=scales, global_scale=1e-3,
                out=torch.zeros((M, N), dtype=torch.float32, device=device))


def test_static_scratch_entry_matches_workspace_entry(cuda_device):
    from turbopi_b200 import _lib, ops
    lib = _lib.load()
    assert lib.tpb200_nvfp4_gemv_tc_static_capacity() == 16 << 20
    rng = np.random.default_rng(77)
    # two problems in one launch; the second one's K is split across CTAs, so the scratch is really used
    probs = [_problem(rng, 4096, 1024, 2, cuda_device), _problem(rng, 1024, 4096, 2, cuda_device)]
    tc = ops.TcGemv(probs, pieces=3)
    tc.quantize()
    tc.gemv()                                             # existing entry point, caller-provided workspace
    torch.cuda.synchronize()
    want = [p["out"].cpu().numpy().copy() for p in probs]
    for call in range(2):                                 # twice in a row: the array keeps the last call's contents
        for p in probs:
            p["out"].fill_(-1.0)
        tc.gemv_static()
        torch.cuda.synchronize()
        for p, w in zip(probs, want):
            got = p["out"].cpu().numpy()
            assert rel_err(got, w) <= 1e-2, (call, rel_err(got, w))
            assert np.array_equal(got, w), call           # same kernel, same plan: the same bytes
    assert lib.tpb200_device_error(0) == 0


def test_static_scratch_entry_refuses_what_does_not_fit(cuda_device):
    """A plan that needs more than the built-in 16 MiB is rejected on the host, nothing is launched."""
    from turbopi_b200 import _lib
    lib = _lib.load()
    # 1024 row tiles, 8 K-splits of 16 token rows each: 262144 x 16384 needs far more than 16 MiB;
    # the pointers are never dereferenced because the size check comes first
    arr = (_lib.GemvTcProblem * 1)()
    arr[0] = _lib.GemvTcProblem(256, 256, 256, 0, 256, 262144, 16384, 0, 1.0)
    st = lib.tpb200_nvfp4_gemv_tc_static(arr, 1, 1, 3, 0, 2, 0, 0, None)
    assert st == -6 and b"workspace" in lib.tpb200_status_string(st)
