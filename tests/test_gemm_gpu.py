"""Parity of the tcgen05 NVFP4 x NVFP4 GEMM and its activation quantiser with the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import cosine, rel_err
from oracle import formats, nvfp4

pytestmark = pytest.mark.gpu


def _dev(a, device, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return t if dtype is None else t.to(dtype)


def _pack_padded(codes_packed, pitch):
    R, Kh = codes_packed.shape
    out = np.zeros((R, pitch), dtype=np.uint8)
    out[:, :Kh] = codes_packed
    return out


def _operand(rng, rows, K, scale):
    """Random block-16 NVFP4 operand: (packed codes, UE4M3 scale bytes, dequantised float64)."""
    vals = (rng.normal(size=(rows, K)) * scale).astype(np.float32)
    q, s = nvfp4.quantize_to_nvfp4(vals, 16)
    sb = formats.e4m3_encode(s)
    packed = nvfp4.pack_nvfp4(q)
    deq = nvfp4.dequantize(packed, sb, 16, 1.0, scale_is_e4m3=True).astype(np.float64)
    return packed, sb, deq


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (128, 128, 64), (1, 8, 16), (200, 264, 1024), (712, 2048, 2048),
                                   (512, 1152, 4304), (512, 4304, 1152), (37, 4096, 1024), (712, 384, 16384)])
def test_gemm_matches_oracle(cuda_device, M, N, K):
    from turbopi_b200 import _lib, ops
    rng = np.random.default_rng(M + N + K)
    ap, asf, ad = _operand(rng, M, K, 1.0)
    bp, bsf, bd = _operand(rng, N, K, 0.5)
    pitch = ops.packed_pitch(K)
    a = _dev(_pack_padded(ap, pitch), cuda_device)
    b = _dev(_pack_padded(bp, pitch), cuda_device)
    a_sf = _dev(nvfp4.swizzle_scales_128x4(asf, 16), cuda_device)
    b_sf = _dev(nvfp4.swizzle_scales_128x4(bsf, 16), cuda_device)
    assert a_sf.numel() == ops.nvfp4_sf_bytes(M, K) and b_sf.numel() == ops.nvfp4_sf_bytes(N, K)
    assert np.array_equal(ops.swizzle_scales(_dev(bsf, cuda_device)).cpu().numpy(), b_sf.cpu().numpy())
    bias = rng.normal(size=(N,)).astype(np.float32)
    buf = torch.full((M + 2, N), -777.0, dtype=torch.float32, device=cuda_device)
    out = ops.nvfp4_gemm(a, a_sf, b, b_sf, M, N, K, alpha=0.125, bias=_dev(bias, cuda_device), out=buf[1:M + 1])
    ref = 0.125 * (ad @ bd.T) + bias
    y = out.cpu().numpy()
    assert _lib.load().tpb200_device_error(0) == 0
    assert rel_err(y, ref) <= 2e-5, rel_err(y, ref)      # products of e2m1 x E4M3 are exact; only fp32 summation order
    assert (buf[0] == -777.0).all() and (buf[-1] == -777.0).all()
    yb = ops.nvfp4_gemm(a, a_sf, b, b_sf, M, N, K, alpha=0.125, activation=1, out_dtype=torch.bfloat16)
    refb = nvfp4.gelu_tanh(0.125 * (ad @ bd.T))
    assert rel_err(yb.float().cpu().numpy(), refb) <= 1e-2 and cosine(yb.float().cpu().numpy(), refb) >= 0.999


@pytest.mark.parametrize("M,K", [(712, 2048), (5, 16), (130, 4304), (512, 1152)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_activation_quantiser_bit_exact(cuda_device, M, K, dt):
    """Codes and scale bytes equal the reference recipe (quantize_to_nvfp4_sim without MSE search,
    block 16; scales rounded to E4M3) bit for bit, including zero blocks, ties and the +-2688 clamp."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(M * K)
    x = (rng.normal(size=(M, K)) * rng.choice([0.01, 1.0, 30.0], size=(M, 1))).astype(np.float32)
    x[0, :16] = 0.0
    x[min(1, M - 1), :16] = [6, 5, 3.5, 2.5, 1.75, 1.25, 0.75, 0.25, -6, -5, -3.5, -2.5, -1.75, -1.25, -0.75, -0.25]
    x[min(2, M - 1), 0] = 1e5
    xt = _dev(x, cuda_device, dt)
    xr = xt.float().cpu().numpy()
    packed, sf = ops.nvfp4_quantize_act(xt)
    lim = np.float32(2688.0)
    q, s = nvfp4.quantize_to_nvfp4_sim(np.clip(xr, -lim, lim), 16, use_mse_search=False)
    ref_packed = nvfp4.pack_nvfp4_data(q)
    assert np.array_equal(packed.cpu().numpy()[:, :K // 2], ref_packed)
    ref_sf = nvfp4.swizzle_scales_128x4(formats.e4m3_encode(s), 16)
    assert np.array_equal(sf.cpu().numpy(), ref_sf)


def test_quantise_then_gemm_matches_reference_simulation(cuda_device):
    """The full W4A4 path against NVFP4Linear._forward_simulation restated in the oracle."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(99)
    M, N, K = 300, 512, 2048
    w = (rng.normal(size=(N, K)) * 0.02).astype(np.float32)
    x = formats.round_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    wq, ws = nvfp4.quantize_to_nvfp4_sim(w, 16, use_mse_search=False)
    ws_b = formats.e4m3_encode(ws * np.float32(256.0))          # keep small weight scales inside E4M3's range
    b = _dev(_pack_padded(nvfp4.pack_nvfp4_data(wq), ops.packed_pitch(K)), cuda_device)
    b_sf = _dev(nvfp4.swizzle_scales_128x4(ws_b, 16), cuda_device)
    a, a_sf = ops.nvfp4_quantize_act(_dev(x, cuda_device, torch.bfloat16))
    y = ops.nvfp4_gemm(a, a_sf, b, b_sf, M, N, K, alpha=1.0 / 256.0, out_dtype=torch.float32)
    lim = np.float32(2688.0)
    xq, xs = nvfp4.quantize_to_nvfp4_sim(np.clip(x, -lim, lim), 16, use_mse_search=False)
    xd = nvfp4.dequantize_nvfp4_sim(xq, xs, 16, use_fp8_scales=True).astype(np.float64)
    wd = (wq.reshape(N, -1, 16) * (formats.e4m3_decode(ws_b) / np.float32(256.0))[:, :, None]).reshape(N, K)
    ref = xd @ wd.astype(np.float64).T
    assert rel_err(y.cpu().numpy(), ref) <= 1e-4


@torch.no_grad()
def test_nvfp4_linear_module_matches_reference_golden(cuda_device, golden):
    """NVFP4Linear (block 32, MSE-searched weight scales, E4M3-rounded scales on both sides) against the
    output of the reference's own simulation forward on its own quantised tensors."""
    from turbopi_b200 import nvfp4_linear
    g = golden("nvfp4_sim")
    lin = torch.nn.Linear(128, 48, bias=False)
    lin.weight.copy_(torch.from_numpy(g["weight"]))
    # quantise on the CPU (where the golden vectors were made), then move the packed layer to the GPU
    layer = nvfp4_linear.NVFP4Linear.from_linear(lin, block_size=32, keep_sim_weights=True).to(cuda_device)
    assert np.array_equal(layer.weight_q.cpu().numpy(), g["wq_mse"])
    assert np.array_equal(layer.weight_scales.cpu().numpy(), g["ws_mse"])
    assert np.array_equal(layer.weight_packed.cpu().numpy()[:, :64], g["w_packed"])
    # activations: the reference example quantises x per 32; the kernel's native block is 16, so compare
    # against the oracle's simulation at block 16 for x and the golden block-32 weights
    x = torch.from_numpy(g["x"]).to(cuda_device)
    y = layer(x).float().cpu().numpy()
    xq, xs = nvfp4.quantize_to_nvfp4_sim(g["x"], 16, use_mse_search=False)
    xd = nvfp4.dequantize_nvfp4_sim(xq, xs, 16, use_fp8_scales=True).astype(np.float64)
    ref = xd @ g["w_dequant_fp8"].astype(np.float64).T
    assert rel_err(y, ref) <= 1e-4
    # and it stays close to the reference's block-32 activation result
    assert cosine(y, g["y"]) >= 0.99


@pytest.mark.parametrize("pieces,tol", [(1, 0.2), (2, 2.5e-2), (3, 4e-3), (4, 3e-3)])
def test_weight_only_semantics_through_residual_pieces(cuda_device, pieces, tol):
    """bf16 activations x NVFP4 weights on the tensor cores: the error against the dequantise-then-matmul
    reference falls with the number of residual pieces; three pieces are inside the 1e-2 bound."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(5)
    M, N, K = 200, 384, 2048
    w = (rng.normal(size=(N, K)) * 0.02).astype(np.float32)
    packed, sbytes, g = nvfp4.quantize_two_level(w, 16)
    x = formats.round_to_bf16((rng.normal(size=(M, K)) * rng.choice([0.05, 1.0, 20.0], size=(M, 1))).astype(np.float32))
    x[3] = 0.0
    b = _dev(_pack_padded(packed, ops.packed_pitch(K)), cuda_device)
    b_sf = _dev(nvfp4.swizzle_scales_128x4(sbytes, 16), cuda_device)
    y = ops.nvfp4_gemm_w4a16(_dev(x, cuda_device, torch.bfloat16), b, b_sf, N, alpha=float(g), pieces=pieces,
                             out_dtype=torch.float32).cpu().numpy()
    ref = nvfp4.gemv_dequant_matmul(x, packed, sbytes, None, 0, 16, float(g), True)
    assert np.isfinite(y).all() and (y[3] == 0).all()
    # every row against its own scale: rows differ by 400x in magnitude
    err = np.abs(y - ref).max(axis=1) / np.maximum(np.abs(ref).max(axis=1), 1e-30)
    assert err.max() <= tol, err.max()


def test_fused_qkv_rope_kv_append_prefix(cuda_device):
    """Benchmark configuration 3: hidden 2048, 8 query heads, 1 KV head, head_dim 256, 712 prefix tokens,
    positions 0..711, bf16 cache [18, 2, 1024, 256] pre-filled with a sentinel."""
    from oracle import kv_fuse
    from turbopi_b200 import _lib, ops
    rng = np.random.default_rng(12)
    S, H, QD = 712, 2048, 2048
    layer, pos0 = 7, 0
    x = formats.round_to_bf16(rng.normal(size=(S, H)).astype(np.float32))
    w = (rng.normal(size=(QD + 512, H)) * 0.02).astype(np.float32)
    packed, sbytes, g = nvfp4.quantize_two_level(w, 16)
    wd = nvfp4.dequantize(packed, sbytes, 16, float(g), True)
    perm = ops.qkv_tile_permutation(QD).numpy()
    b = _dev(_pack_padded(packed[perm], ops.packed_pitch(H)), cuda_device)
    b_sf = _dev(nvfp4.swizzle_scales_128x4(sbytes[perm], 16), cuda_device)
    cache = torch.full((18, 2, 1024, 256), -3.0, dtype=torch.bfloat16, device=cuda_device)
    positions = torch.arange(S, dtype=torch.int32, device=cuda_device)
    cos, sin = ops.rope_tables(1024, device=cuda_device)
    q = ops.fused_qkv_rope_append(_dev(x, cuda_device, torch.bfloat16), b, b_sf, QD, cache[layer, 0, pos0:],
                                  cache[layer, 1, pos0:], positions, cos, sin, alpha=float(g))
    assert _lib.load().tpb200_device_error(0) == 0
    ref_cache = np.full((18, 2, 1024, 256), -3.0, dtype=np.float32)
    # the rotary tables follow the model's recipe; cos/sin of the fp32 angle may differ from the oracle's
    # float64 evaluation in the last bf16 bit for a handful of entries
    oc, os_ = kv_fuse.rope_cos_sin(np.arange(1024), 256, 10000.0)
    tc_, ts_ = cos.float().cpu().numpy(), sin.float().cpu().numpy()
    assert (tc_ == oc[:, :128]).mean() > 0.995 and np.abs(tc_ - oc[:, :128]).max() <= 2 ** -7
    assert (ts_ == os_[:, :128]).mean() > 0.995 and np.abs(ts_ - os_[:, :128]).max() <= 2 ** -7
    full = (np.concatenate([tc_, tc_], axis=1)[:S], np.concatenate([ts_, ts_], axis=1)[:S])
    q_ref, _ = kv_fuse.fused_qkv_rope_append(x, wd[:QD], wd[QD:QD + 256], wd[QD + 256:], ref_cache, layer,
                                             np.arange(S), pos0, cos_sin=full)
    got = cache.float().cpu().numpy()
    # cache index writes: exactly rows pos0..pos0+S-1 of `layer` changed, nothing else
    touched = np.zeros((18, 2, 1024), dtype=bool)
    touched[layer, :, pos0:pos0 + S] = True
    assert (got[~touched] == -3.0).all()
    assert (got[touched] != -3.0).any(axis=-1).all()
    for name, y, r in (("q", q.float().cpu().numpy(), q_ref), ("k", got[layer, 0, :S], ref_cache[layer, 0, :S]),
                       ("v", got[layer, 1, :S], ref_cache[layer, 1, :S])):
        assert rel_err(y, r) <= 1e-2, (name, rel_err(y, r))
        assert cosine(y, r) >= 0.999, (name, cosine(y, r))


@pytest.mark.parametrize("M,N,K,act", [(50, 1024, 2048, 0), (50, 2048, 4096, 1), (300, 1152, 4608, 2), (17, 136, 2048, 0),
                                       (129, 520, 8192, 0)])
def test_split_k_through_workspace_matches_unsplit_and_oracle(cuda_device, M, N, K, act):
    """Few-tile shapes split their K range over several CTAs when a workspace is given: same result as
    the unsplit launch (up to fp32 summation order), twice in a row on one workspace (the kernel leaves
    its counters at zero), bias and activation applied once by the reducing CTA."""
    from turbopi_b200 import _lib, ops
    rng = np.random.default_rng(31)
    w = (rng.normal(size=(N, K)) * 0.02).astype(np.float32)
    packed, sbytes, g = nvfp4.quantize_two_level(w, 16)
    x = formats.round_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    bias = rng.normal(size=(N,)).astype(np.float32)
    b = _dev(_pack_padded(packed, ops.packed_pitch(K)), cuda_device)
    b_sf = _dev(nvfp4.swizzle_scales_128x4(sbytes, 16), cuda_device)
    xd, bd = _dev(x, cuda_device, torch.bfloat16), _dev(bias, cuda_device)
    need = ops.nvfp4_gemm_workspace_size(M, N, K, 3)
    assert need > 0, "shape expected to split"
    ws = ops.gemm_workspace(cuda_device, need)
    base = ops.nvfp4_gemm_w4a16(xd, b, b_sf, N, alpha=float(g), bias=bd, activation=act, out_dtype=torch.float32)
    y1 = ops.nvfp4_gemm_w4a16(xd, b, b_sf, N, alpha=float(g), bias=bd, activation=act, out_dtype=torch.float32,
                              workspace=ws)
    y2 = ops.nvfp4_gemm_w4a16(xd, b, b_sf, N, alpha=float(g), bias=bd, activation=act, out_dtype=torch.float32,
                              workspace=ws)
    assert _lib.load().tpb200_device_error(0) == 0
    assert torch.equal(y1, y2)
    assert (ws[:16384].view(torch.int32) == 0).all()
    scale = base.abs().max().item()
    assert (y1 - base).abs().max().item() <= 2e-5 * scale
    pre = nvfp4.gemv_dequant_matmul(x, packed, sbytes, None, 0, 16, float(g), True) + bias
    if act == 1:
        ref = 0.5 * pre * (1 + np.tanh(0.7978845608028654 * (pre + 0.044715 * pre ** 3)))
    elif act == 2:
        ref = pre / (1 + np.exp(-pre))
    else:
        ref = pre
    assert rel_err(y1.cpu().numpy(), ref) <= 1e-2


def test_fused_qkv_split_k_matches_unsplit(cuda_device):
    """The action expert's per-step shape (50 tokens): fused QKV + RoPE + cache rows with the K range
    split over CTAs gives the same bf16 values as the unsplit launch."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(13)
    S, H, QD = 50, 2048, 2048
    x = _dev(formats.round_to_bf16(rng.normal(size=(S, H)).astype(np.float32)), cuda_device, torch.bfloat16)
    w = (rng.normal(size=(QD + 512, H)) * 0.02).astype(np.float32)
    packed, sbytes, g = nvfp4.quantize_two_level(w, 16)
    perm = ops.qkv_tile_permutation(QD).numpy()
    b = _dev(_pack_padded(packed[perm], ops.packed_pitch(H)), cuda_device)
    b_sf = _dev(nvfp4.swizzle_scales_128x4(sbytes[perm], 16), cuda_device)
    positions = torch.arange(712, 712 + S, dtype=torch.int32, device=cuda_device)
    cos, sin = ops.rope_tables(1024, device=cuda_device)
    outs = []
    for ws in (None, ops.gemm_workspace(cuda_device)):
        cache = torch.full((2, 1024, 256), -3.0, dtype=torch.bfloat16, device=cuda_device)
        q = ops.fused_qkv_rope_append(x, b, b_sf, QD, cache[0, 712:], cache[1, 712:], positions, cos, sin,
                                      alpha=float(g), workspace=ws)
        outs.append((q.float(), cache.float()))
    assert ops.nvfp4_gemm_workspace_size(S, QD + 512, H, 3) > 0
    for a, c in zip(outs[0], outs[1]):
        # fp32 summation order differs, so a bf16 rounding may flip for a few elements
        assert (a == c).float().mean().item() > 0.99
        assert (a - c).abs().max().item() <= 2 ** -7 * a.abs().max().item()
    assert (outs[1][1][:, :712] == -3.0).all() and (outs[1][1][:, 762:] == -3.0).all()


# ---------------------------------------------------------------------------- tiled operand images
@pytest.mark.parametrize("M,N,K,act,split", [(128, 256, 256, 0, False), (200, 384, 2048, 1, False),
                                             (712, 2048, 2048, 0, False), (50, 1024, 4096, 2, True),
                                             (300, 1152, 4304, 0, True), (300, 1152, 1152, 0, False), (5, 8, 16, 0, False),
                                             (130, 4304, 1152, 1, False), (712, 2048, 16384, 0, True)])
def test_tiled_operands_match_oracle_and_rowmajor(cuda_device, M, N, K, act, split):
    """The fast path (pre-tiled operand images, 128 x 256 output tiles, bulk-copy producer) against the
    dequantise-then-matmul oracle and against the row-major form of the same kernel."""
    from turbopi_b200 import _lib, ops
    rng = np.random.default_rng(41)
    w = (rng.normal(size=(N, K)) * 0.02).astype(np.float32)
    packed, sbytes, g = nvfp4.quantize_two_level(w, 16)
    x = formats.round_to_bf16((rng.normal(size=(M, K)) * rng.choice([0.05, 1.0, 20.0], size=(M, 1))).astype(np.float32))
    bias = rng.normal(size=(N,)).astype(np.float32)
    b = _dev(_pack_padded(packed, ops.packed_pitch(K)), cuda_device)
    b_sf = _dev(nvfp4.swizzle_scales_128x4(sbytes, 16), cuda_device)
    image = ops.tile_weights(b, b_sf, N, K)
    xd, bd = _dev(x, cuda_device, torch.bfloat16), _dev(bias, cuda_device)
    ws = ops.gemm_workspace(cuda_device) if split else None
    if split:
        assert ops.nvfp4_gemm_workspace_size(M, N, K, 3, ops.OPERANDS_TILED) > 0
    y = ops.nvfp4_gemm_w4a16_tiled(xd, image, N, alpha=float(g), bias=bd, activation=act, out_dtype=torch.float32,
                                   workspace=ws)
    y2 = ops.nvfp4_gemm_w4a16_tiled(xd, image, N, alpha=float(g), bias=bd, activation=act, out_dtype=torch.float32,
                                    workspace=ws)
    base = ops.nvfp4_gemm_w4a16(xd, b, b_sf, N, alpha=float(g), bias=bd, activation=act, out_dtype=torch.float32)
    assert _lib.load().tpb200_device_error(0) == 0
    assert torch.equal(y, y2)
    assert (y - base).abs().max().item() <= 2e-5 * base.abs().max().item()
    pre = nvfp4.gemv_dequant_matmul(x, packed, sbytes, None, 0, 16, float(g), True) + bias
    if act == 1:
        ref = 0.5 * pre * (1 + np.tanh(0.7978845608028654 * (pre + 0.044715 * pre ** 3)))
    elif act == 2:
        ref = pre / (1 + np.exp(-pre))
    else:
        ref = pre
    got = y.cpu().numpy()
    err = np.abs(got - ref).max(axis=1) / np.maximum(np.abs(ref).max(axis=1), 1e-30)
    assert err.max() <= 5e-3, err.max()


def test_tiled_bf16_output_leaves_neighbours_untouched(cuda_device):
    """bf16 output into a view of a larger buffer: only the [M, N] window changes (tile stores are clipped
    by the tensor map at ragged edges: M = 130 rows, N = 328 columns)."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(43)
    M, N, K = 130, 328, 512
    w = (rng.normal(size=(N, K)) * 0.02).astype(np.float32)
    packed, sbytes, g = nvfp4.quantize_two_level(w, 16)
    x = formats.round_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    image = ops.tile_weights(_dev(_pack_padded(packed, ops.packed_pitch(K)), cuda_device),
                             _dev(nvfp4.swizzle_scales_128x4(sbytes, 16), cuda_device), N, K)
    canvas = torch.full((M + 3, 512), 7.0, dtype=torch.bfloat16, device=cuda_device)
    out = canvas[2:M + 2, 8:8 + N]
    ops.nvfp4_gemm_w4a16_tiled(_dev(x, cuda_device, torch.bfloat16), image, N, alpha=float(g), out=out)
    ref = nvfp4.gemv_dequant_matmul(x, packed, sbytes, None, 0, 16, float(g), True)
    assert rel_err(out.float().cpu().numpy(), ref) <= 1e-2
    mask = torch.ones_like(canvas, dtype=torch.bool)
    mask[2:M + 2, 8:8 + N] = False
    assert (canvas[mask] == 7.0).all()


def test_fused_qkv_tiled_matches_rowmajor(cuda_device):
    """Fused QKV + RoPE + cache rows through the tiled images: same bf16 results as the row-major form
    (prefix shape, 712 tokens; and the expert's 50-token shape with split K)."""
    from turbopi_b200 import ops
    rng = np.random.default_rng(17)
    QD = 2048
    for S, H, pos0, ws in ((712, 2048, 0, None), (50, 1024, 712, "ws")):
        x = _dev(formats.round_to_bf16(rng.normal(size=(S, H)).astype(np.float32)), cuda_device, torch.bfloat16)
        w = (rng.normal(size=(QD + 512, H)) * 0.02).astype(np.float32)
        packed, sbytes, g = nvfp4.quantize_two_level(w, 16)
        perm = ops.qkv_tile_permutation(QD).numpy()
        b = _dev(_pack_padded(packed[perm], ops.packed_pitch(H)), cuda_device)
        b_sf = _dev(nvfp4.swizzle_scales_128x4(sbytes[perm], 16), cuda_device)
        image = ops.tile_weights(b, b_sf, QD + 512, H)
        positions = torch.arange(pos0, pos0 + S, dtype=torch.int32, device=cuda_device)
        cos, sin = ops.rope_tables(1024, device=cuda_device)
        outs = []
        for tiled in (False, True):
            cache = torch.full((2, 1024, 256), -3.0, dtype=torch.bfloat16, device=cuda_device)
            q = ops.fused_qkv_rope_append(x, image if tiled else b, None if tiled else b_sf, QD, cache[0, pos0:],
                                          cache[1, pos0:], positions, cos, sin, alpha=float(g),
                                          workspace=ops.gemm_workspace(cuda_device) if (ws and tiled) else None)
            outs.append((q.float(), cache.float()))
        for a, c in zip(outs[0], outs[1]):
            assert (a == c).float().mean().item() > 0.99
            assert (a - c).abs().max().item() <= 2 ** -7 * a.abs().max().item()
        assert (outs[1][1][:, :pos0] == -3.0).all() and (outs[1][1][:, pos0 + S:] == -3.0).all()


@pytest.mark.parametrize("M,inter,K,split", [(712, 1024, 2048, False), (50, 512, 1024, True), (130, 384, 512, False)])
def test_gated_gelu_epilogue_matches_module_arithmetic(cuda_device, M, inter, K, split):
    """gate_up projection with GELU(gate) * up in the epilogue (tiled operands, 128 gate rows + 128 up rows
    per weight block): out = bf16(bf16(gelu_tanh(bf16(x Wg^T))) * bf16(x Wu^T)), N / 2 columns."""
    from turbopi_b200 import _lib, ops
    rng = np.random.default_rng(51)
    w = (rng.normal(size=(2 * inter, K)) * 0.03).astype(np.float32)
    packed, sbytes, g = nvfp4.quantize_two_level(w, 16)
    x = formats.round_to_bf16(rng.normal(size=(M, K)).astype(np.float32))
    perm = ops.geglu_row_permutation(inter).numpy()
    image = ops.tile_weights(_dev(_pack_padded(packed[perm], ops.packed_pitch(K)), cuda_device),
                             _dev(nvfp4.swizzle_scales_128x4(sbytes[perm], 16), cuda_device), 2 * inter, K)
    ws = ops.gemm_workspace(cuda_device) if split else None
    if split:
        assert ops.nvfp4_gemm_workspace_size(M, 2 * inter, K, 3, ops.OPERANDS_TILED) > 0
    canvas = torch.full((M + 2, inter + 16), 7.0, dtype=torch.bfloat16, device=cuda_device)
    out = canvas[1:M + 1, 8:8 + inter]
    ops.nvfp4_gemm_w4a16_tiled(_dev(x, cuda_device, torch.bfloat16), image, 2 * inter, alpha=float(g),
                               activation=_lib.ACT_GEGLU, out=out, workspace=ws)
    assert _lib.load().tpb200_device_error(0) == 0
    pre = nvfp4.gemv_dequant_matmul(x, packed, sbytes, None, 0, 16, float(g), True)
    gate, up = formats.round_to_bf16(pre[:, :inter].astype(np.float32)), formats.round_to_bf16(pre[:, inter:].astype(np.float32))
    act = formats.round_to_bf16((0.5 * gate * (1 + np.tanh(0.7978845608028654 * (gate + 0.044715 * gate ** 3)))).astype(np.float32))
    ref = formats.round_to_bf16(act * up)
    got = out.float().cpu().numpy()
    assert rel_err(got, ref) <= 1e-2 and cosine(got, ref) >= 0.999
    mask = torch.ones_like(canvas, dtype=torch.bool)
    mask[1:M + 1, 8:8 + inter] = False
    assert (canvas[mask] == 7.0).all()


@pytest.mark.gpu
@pytest.mark.parametrize("rowmajor", [True, False])
def test_split_k_launches_on_two_streams(cuda_device, rowmajor):
    """Two split-K launches (each with a workspace of its own) issued on two streams over and over: the CTAs of a
    tile wait for each other, so each launch is a cooperative launch and the other stream's launch cannot keep
    partners off the SMs.  Results equal the launches run one after the other; no device error."""
    from turbopi_b200 import _lib, ops
    from turbopi_b200.pi05 import TcLinear
    M, N, K = 50, 1024, 4096                       # 8 or 4 output tiles: the planner cuts K
    g = torch.Generator().manual_seed(3)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(cuda_device)
    lins, qs, outs, streams = [], [], [], []
    for i in range(2):
        lin = TcLinear.from_weight((torch.randn(N, K, generator=g) * 0.02).to(cuda_device), rowmajor=rowmajor)
        lin.ws = ops.gemm_workspace(cuda_device)
        q = ops.QuantBuf(M, K, 3, cuda_device, tiled=not rowmajor)
        ops.rowop(_lib.ROW_NONE, x, K, q)
        lins.append(lin)
        qs.append(q)
        outs.append(torch.empty((M, N), dtype=torch.bfloat16, device=cuda_device))
        streams.append(torch.cuda.Stream(device=cuda_device))
    assert ops.nvfp4_gemm_workspace_size(M, N, K, 3, 0 if rowmajor else 1) > 0      # i.e. these launches do split
    torch.cuda.synchronize()
    ref = [lins[i](qs[i], torch.empty_like(outs[i])) for i in range(2)]
    torch.cuda.synchronize()
    for _ in range(300):
        for i in range(2):
            with torch.cuda.stream(streams[i]):
                lins[i](qs[i], outs[i])
    torch.cuda.synchronize()
    assert _lib.load().tpb200_device_error(0) == 0
    for i in range(2):
        assert torch.equal(outs[i], ref[i])
