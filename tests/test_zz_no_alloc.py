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
    assert lib.tpb200_nvfp4_gemv_tc_static_capacity() == 4 << 20
    rng = np.random.default_rng(77)
    # two problems in one launch; the second one's K is split across CTAs, so the scratch is really used
    probs = [_problem(rng, 4096, 1024, 2, cuda_device), _problem(rng, 1024, 4096, 2, cuda_device)]
    tc = ops.TcGemv(probs, pieces=3, fused=False)
    assert tc.workspace.numel() > 4096                    # the plan cuts tiles: partial sums go through scratch
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
    """A plan that needs more than the built-in 4 MiB is rejected on the host and nothing is launched.
    Every buffer is real, so a planner that stopped refusing would compute, not fault."""
    from turbopi_b200 import _lib, ops
    lib = _lib.load()
    N, K, M = 25600, 16384, 1       # 100 tiles of 64 K stages: the plan cuts every tile four ways
    image = torch.zeros(int(lib.tpb200_nvfp4_tiled_b_bytes(N, K)), dtype=torch.uint8, device=cuda_device)
    x = torch.ones((M, K), dtype=torch.bfloat16, device=cuda_device)
    out = torch.full((M, N), 7.0, dtype=torch.float32, device=cuda_device)
    tc = ops.TcGemv([dict(x=x, w_image=image, global_scale=1.0, out=out)], pieces=3, fused=False)
    assert tc.workspace.numel() > lib.tpb200_nvfp4_gemv_tc_static_capacity()
    tc.quantize()
    with pytest.raises(_lib.TurboPiError) as e:
        tc.gemv_static()
    assert "workspace" in str(e.value)
    torch.cuda.synchronize()
    assert (out == 7.0).all()
    tc.gemv()                                             # the same launch with a caller-provided workspace runs
    torch.cuda.synchronize()
    assert (out == 0.0).all()
    assert lib.tpb200_device_error(0) == 0
