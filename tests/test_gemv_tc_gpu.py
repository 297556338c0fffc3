"""Parity of the tensor-core NVFP4 GEMV (weights as the MMA's 128-row operand, residual-piece
activations quantised inside the launch or read from a pre-tiled image, host-planned schedule with
K cuts through scratch where a launch has few tiles) with the CPU oracle and with the CUDA-core GEMV."""
import numpy as np
import pytest
import torch

from conftest import cosine, rel_err
from oracle import formats, nvfp4

pytestmark = pytest.mark.gpu


def _dev(a, device, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return t if dtype is None else t.to(dtype)


def _weights(rng, N, K):
    base = (rng.normal(size=(N, K)) * 0.02).astype(np.float32)
    _, sbytes, g = nvfp4.quantize_two_level(base, 16)
    packed = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    return packed, sbytes, float(g)


def test_weight_tiling_is_the_swizzled_image(cuda_device):
    """tile_weights: block (n // 256, k_stage) of 36864 bytes = 256 rows x 128 B with 16-byte chunk c of row
    r at c ^ (r & 7), then the scale slabs of rows 0..127 and 128..255; padding rows are zero."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(1)
    N, K = 328, 1024 + 512
    packed = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    sbytes = rng.integers(1, 120, size=(N, K // 16), dtype=np.uint8)
    sf = nvfp4.swizzle_scales_128x4(sbytes, 16)
    image = ops.tile_weights(_dev(packed, cuda_device), _dev(sf, cuda_device), N, K).cpu().numpy().reshape(2, 6, 36864)
    codes = image[:, :, :32768].reshape(2, 6, 256, 8, 16)
    slabs = image[:, :, 32768:].reshape(2, 6, 2, 4, 32, 4, 4)      # [half][K atom][r % 32][r // 32][k block]
    for (n, kbyte) in [(0, 0), (1, 17), (129, 300), (327, 767), (77, 640), (300, 5)]:
        nb, r = divmod(n, 256)
        ks, within = divmod(kbyte, 128)
        c, b = divmod(within, 16)
        assert codes[nb, ks, r, c ^ (r & 7), b] == packed[n, kbyte]
        kb = kbyte // 8                                  # 16-element block index
        rr = r % 128
        assert slabs[nb, ks, r // 128, (kb % 16) // 4, rr % 32, rr // 32, kb % 4] == sbytes[n, kb]
    assert codes[1, :, 72:, :, :].sum() == 0          # padded rows are zero codes
    assert slabs[1, :, 1].sum() == 0                   # ... with zero scales


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("M", [1, 4, 16])
@pytest.mark.parametrize("N,K", [(4096, 1024), (1024, 4096), (16384, 2048), (2048, 16384), (200, 272), (2560, 2048)])
def test_tc_gemv_matches_oracle(cuda_device, M, N, K, fused):
    from turbopi_b200 import _lib, ops
    rng = np.random.default_rng(M + N + K)
    packed, sbytes, g = _weights(rng, N, K)
    x = formats.round_to_bf16((rng.normal(size=(M, K)) * rng.choice([0.1, 1.0, 10.0], size=(M, 1))).astype(np.float32))
    bias = rng.normal(size=(N,)).astype(np.float32)
    buf = torch.full((M + 32, N), -5.0, dtype=torch.float32, device=cuda_device)
    out = buf[16:16 + M]
    tc = ops.TcGemv([dict(x=_dev(x, cuda_device, torch.bfloat16), weight_packed=_dev(packed, cuda_device),
                          weight_scales=_dev(sbytes, cuda_device), global_scale=g, out=out,
                          bias=_dev(bias, cuda_device))], pieces=3, fused=fused)
    tc.launch()
    tc.launch()                       # the counters are back at zero: a second launch gives the same bytes
    y1 = out.cpu().numpy().copy()
    tc.launch()
    assert np.array_equal(out.cpu().numpy(), y1)
    assert _lib.load().tpb200_device_error(0) == 0
    ref = nvfp4.gemv_dequant_matmul(x, packed, sbytes, bias, 0, 16, g, True)
    err = np.abs(y1 - ref).max(axis=1) / np.abs(ref).max(axis=1)
    assert err.max() <= 1e-2, err.max()
    assert cosine(y1, ref) >= 0.999
    assert (buf[:16] == -5.0).all() and (buf[16 + M:] == -5.0).all()


def test_tc_grouped_matches_cuda_core_gemv(cuda_device):
    from turbopi_b200 import ops
    rng = np.random.default_rng(3)
    shapes = [(4096, 1024), (4096, 1024), (1024, 4096)] * 2
    xs = {K: _dev(formats.round_to_bf16(rng.normal(size=(1, K)).astype(np.float32)), cuda_device, torch.bfloat16)
          for K in (1024, 4096)}
    probs, refs = [], []
    for N, K in shapes:
        packed, sbytes, g = _weights(rng, N, K)
        p = dict(x=xs[K], weight_packed=_dev(packed, cuda_device), weight_scales=_dev(sbytes, cuda_device),
                 global_scale=g, out=torch.zeros((1, N), dtype=torch.bfloat16, device=cuda_device))
        probs.append(p)
        o = torch.empty((1, N), dtype=torch.bfloat16, device=cuda_device)
        ops.nvfp4_gemv_out(p["x"], p["weight_packed"], p["weight_scales"], o, block_size=16, global_scale=g)
        refs.append(o)
    ops.TcGemv(probs, pieces=3, activation=0).launch()
    for p, o in zip(probs, refs):
        assert rel_err(p["out"].float().cpu().numpy(), o.float().cpu().numpy()) <= 1e-2


@pytest.mark.parametrize("fused", [True, False])
def test_tc_gemv_chain_under_programmatic_dependent_launch(cuda_device, fused):
    """GEMV -> GEMV ... (or quantiser -> GEMV -> quantiser -> GEMV ...) launched with programmatic stream
    serialisation (a GEMV requests its first weight blocks while its predecessor still runs): same bytes
    as the plain launches, also when the chain is captured in a CUDA graph and replayed."""
    from turbopi_b200 import _lib, ops
    rng = np.random.default_rng(77)
    specs = [(4096, 1024), (4096, 1024), (1024, 4096)] * 3
    xs = {K: _dev(formats.round_to_bf16(rng.normal(size=(1, K)).astype(np.float32)), cuda_device, torch.bfloat16)
          for K in (1024, 4096)}
    mats = [_weights(rng, N, K) for (N, K) in specs]

    def build(pdl):
        outs = [torch.zeros((1, N), dtype=torch.bfloat16, device=cuda_device) for (N, K) in specs]
        tc = ops.TcGemv([dict(x=xs[K], weight_packed=_dev(p, cuda_device), weight_scales=_dev(s, cuda_device),
                              global_scale=g, out=o) for (N, K), (p, s, g), o in zip(specs, mats, outs)],
                        pieces=3, pdl=pdl, fused=fused)
        return tc, outs

    plain, want = build(False)
    plain.launch()
    chained, got = build(True)
    for _ in range(3):
        chained.launch()
    torch.cuda.synchronize()
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    side = torch.cuda.Stream(device=cuda_device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        chained.launch()
        chained.launch()
    for o in got:
        o.zero_()
    graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert _lib.load().tpb200_device_error(0) == 0


def test_tc_gemv_reads_the_gemm_weight_image(cuda_device):
    """One tiled weight image serves prefill and decode: the GEMV given `w_image` (what tile_weights makes for
    the tensor-core GEMM) returns the same bytes as the GEMV that tiles the packed weights itself."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(91)
    N, K = 1152, 2048
    packed, sbytes, g = _weights(rng, N, K)
    x = _dev(formats.round_to_bf16(rng.normal(size=(2, K)).astype(np.float32)), cuda_device, torch.bfloat16)
    b = torch.zeros((N, ops.packed_pitch(K)), dtype=torch.uint8, device=cuda_device)
    b[:, :K // 2] = _dev(packed, cuda_device)
    image = ops.tile_weights(b, ops.swizzle_scales(_dev(sbytes, cuda_device)), N, K)
    y1 = torch.zeros((2, N), dtype=torch.float32, device=cuda_device)
    y2 = torch.zeros((2, N), dtype=torch.float32, device=cuda_device)
    ops.TcGemv([dict(x=x, w_image=image, global_scale=g, out=y1)], pieces=3).launch()
    ops.TcGemv([dict(x=x, weight_packed=_dev(packed, cuda_device), weight_scales=_dev(sbytes, cuda_device),
                     global_scale=g, out=y2)], pieces=3).launch()
    assert torch.equal(y1, y2)
    ref = nvfp4.gemv_dequant_matmul(x.float().cpu().numpy(), packed, sbytes, None, 0, 16, g, True)
    assert rel_err(y1.cpu().numpy(), ref) <= 1e-2


@pytest.mark.parametrize("M", [1, 3, 16])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_fused_quantiser_equals_stand_alone_quantiser(cuda_device, M, dtype):
    """The activation pieces made inside the GEMV launch are the ones the stand-alone quantiser writes:
    both forms return the same bytes, for every activation dtype, for a grouped launch whose problems
    share activation tensors and for a K that ends inside a 256-wide stage."""
    from turbopi_b200 import _lib, ops
    rng = np.random.default_rng(5 + M)
    shapes = [(512, 1024), (512, 1024), (768, 4096), (300, 1104), (256, 4096)]
    xs = {K: (torch.from_numpy(rng.normal(size=(M, K)).astype(np.float32)) * 3.0).to(cuda_device).to(dtype)
          for K in (1024, 4096, 1104)}
    mats = [_weights(rng, N, K) for (N, K) in shapes]

    def run(fused):
        outs = [torch.zeros((M, N), dtype=torch.float32, device=cuda_device) for (N, K) in shapes]
        tc = ops.TcGemv([dict(x=xs[K], weight_packed=_dev(p, cuda_device), weight_scales=_dev(s, cuda_device),
                              global_scale=g, out=o) for (N, K), (p, s, g), o in zip(shapes, mats, outs)],
                        pieces=3, fused=fused)
        tc.launch()
        torch.cuda.synchronize()
        return outs

    a, b = run(True), run(False)
    assert _lib.load().tpb200_device_error(0) == 0
    for (N, K), ya, yb, (p, s, g) in zip(shapes, a, b, mats):
        assert torch.equal(ya, yb), (N, K)
        ref = nvfp4.gemv_dequant_matmul(xs[K].float().cpu().numpy(), p, s, None, 0, 16, g, True)
        assert rel_err(ya.cpu().numpy(), ref) <= 1e-2


def test_tc_gemv_strided_activations_and_outputs(cuda_device):
    """Activation rows and output rows with a pitch larger than their width (views into wider buffers)."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(12)
    N, K, M = 640, 2048, 5
    packed, sbytes, g = _weights(rng, N, K)
    xbuf = torch.from_numpy(rng.normal(size=(M, K + 64)).astype(np.float32)).to(cuda_device).to(torch.bfloat16)
    obuf = torch.full((M, N + 32), 9.0, dtype=torch.float32, device=cuda_device)
    x, out = xbuf[:, :K], obuf[:, :N]
    ops.TcGemv([dict(x=x, weight_packed=_dev(packed, cuda_device), weight_scales=_dev(sbytes, cuda_device),
                     global_scale=g, out=out)], pieces=3).launch()
    ref = nvfp4.gemv_dequant_matmul(x.float().cpu().numpy(), packed, sbytes, None, 0, 16, g, True)
    assert rel_err(out.cpu().numpy(), ref) <= 1e-2
    assert (obuf[:, N:] == 9.0).all()


def test_tc_gemv_54_matrix_step_matches_oracle(cuda_device):
    """The benchmark's step: 18 x (gate, up 1024 -> 4096; down 4096 -> 1024) in one launch (648 whole tiles
    dealt to the CTAs, no tile cut), spot-checked against the oracle on three matrices."""
    from turbopi_b200 import _lib, ops
    rng = np.random.default_rng(54)
    shapes = [(4096, 1024), (4096, 1024), (1024, 4096)] * 18
    xs = {K: _dev(formats.round_to_bf16(rng.normal(size=(1, K)).astype(np.float32)), cuda_device, torch.bfloat16)
          for K in (1024, 4096)}
    mats = [_weights(rng, N, K) for (N, K) in shapes]
    outs = [torch.zeros((1, N), dtype=torch.bfloat16, device=cuda_device) for (N, K) in shapes]
    tc = ops.TcGemv([dict(x=xs[K], weight_packed=_dev(p, cuda_device), weight_scales=_dev(s, cuda_device),
                          global_scale=g, out=o) for (N, K), (p, s, g), o in zip(shapes, mats, outs)], pieces=3)
    assert tc.workspace.numel() <= 512            # nothing is cut: no partial sums
    tc.launch()
    torch.cuda.synchronize()
    assert _lib.load().tpb200_device_error(0) == 0
    for i in (0, 26, 53):
        (N, K), (p, s, g) = shapes[i], mats[i]
        ref = nvfp4.gemv_dequant_matmul(xs[K].float().cpu().numpy(), p, s, None, 0, 16, g, True)
        assert rel_err(outs[i].float().cpu().numpy(), ref) <= 1e-2, i
