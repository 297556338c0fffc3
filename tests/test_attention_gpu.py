"""The tensor-core attention kernel against the pinned model oracle's attention (oracle/pi05.py::attention,
which follows the reference's scaled_dot_product_attention calls, pi0_pytorch.py:476-501,608-627) on the
Pi0.5 shapes: Gemma prefix (712 tokens x 8 heads on one KV head), action expert (50 x 8 rows on 762
keys), padded prompts / a missing camera through the additive key bias, and SigLIP's 2 x 16 heads of 72."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from conftest import cosine, rel_err
from oracle import pi05 as opi

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _gemma_case(cuda_device, L, S, valid, seed, heads=8, D=256):
    from turbopi_b200 import _lib, ops
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(L, heads * D, generator=g) * 2.0).to(BF)
    k = torch.randn(S, D, generator=g).to(BF)
    v = torch.randn(S, D, generator=g).to(BF)
    bias = None
    if valid is not None:
        bias = torch.where(valid, 0.0, opi.MASKED).to(BF).to(cuda_device)
    out = torch.full((L, heads * D), 7.0, dtype=BF, device=cuda_device)
    qd = q.to(cuda_device)
    ops.attention(qd.view(L * heads, D), k.to(cuda_device), v.to(cuda_device), out.view(L * heads, D), D ** -0.5, bias)
    torch.cuda.synchronize()
    assert _lib.load().tpb200_device_error(0) == 0
    ref = opi.attention(q.float(), k.float(), v.float(), heads, valid)
    return out.float().cpu().numpy(), ref.numpy()


@pytest.mark.parametrize("L,S", [(712, 712), (50, 762), (5, 3), (128, 128), (129, 129), (1, 300), (300, 1), (40, 256),
                                 (40, 257), (200, 384), (17, 385), (130, 1030)])
def test_gemma_attention_matches_oracle(cuda_device, L, S):
    got, ref = _gemma_case(cuda_device, L, S, None, L * 1000 + S)
    assert rel_err(got, ref) <= 1e-2
    assert cosine(got, ref) >= 0.9999


@pytest.mark.parametrize("L,S", [(712, 712), (50, 762)])
def test_gemma_attention_with_padded_keys(cuda_device, L, S):
    """Padded prompt tail and a whole missing camera (two full key tiles masked)."""
    valid = torch.ones(S, dtype=torch.bool)
    valid[256:512] = False
    valid[690:712] = False
    got, ref = _gemma_case(cuda_device, L, S, valid, 17)
    assert rel_err(got, ref) <= 1e-2
    assert cosine(got, ref) >= 0.9999
    # masked keys carry no weight at all: changing their values changes nothing
    from turbopi_b200 import ops
    g = torch.Generator().manual_seed(17)
    q = (torch.randn(L, 2048, generator=g) * 2.0).to(BF).to(cuda_device)
    k = torch.randn(S, 256, generator=g).to(BF).to(cuda_device)
    v = torch.randn(S, 256, generator=g).to(BF).to(cuda_device)
    bias = torch.where(valid, 0.0, opi.MASKED).to(BF).to(cuda_device)
    o1 = torch.empty((L * 8, 256), dtype=BF, device=cuda_device)
    o2 = torch.empty_like(o1)
    ops.attention(q.view(L * 8, 256), k, v, o1, 1 / 16, bias)
    k2, v2 = k.clone(), v.clone()
    k2[~valid.to(cuda_device)] = 55.0
    v2[~valid.to(cuda_device)] = -99.0
    ops.attention(q.view(L * 8, 256), k2, v2, o2, 1 / 16, bias)
    assert torch.equal(o1, o2)


def test_siglip_attention_matches_torch(cuda_device):
    """2 images x 16 heads x 256 tokens, head_dim 72, q / k / v as strided views of the fused projection
    [tokens, 3 * 1152] and the output as a view of [tokens, 1152] (modeling_siglip.py:371-417)."""
    from turbopi_b200 import _lib, ops
    g = torch.Generator().manual_seed(3)
    NI, T, H, D = 2, 256, 16, 72
    qkv = torch.randn(NI * T, 3 * H * D, generator=g).to(BF)
    qkv_d = qkv.to(cuda_device)
    out = torch.full((NI * T, H * D), 3.0, dtype=BF, device=cuda_device)
    view = qkv_d.view(NI, T, 3, H, D).permute(2, 0, 3, 1, 4)            # [3, NI, H, T, D]
    ops.attention(view[0], view[1], view[2], out.view(NI, T, H, D).permute(0, 2, 1, 3), D ** -0.5)
    torch.cuda.synchronize()
    assert _lib.load().tpb200_device_error(0) == 0
    r = qkv.float().view(NI, T, 3, H, D).permute(2, 0, 3, 1, 4)
    ref = F.scaled_dot_product_attention(r[0], r[1], r[2]).transpose(1, 2).reshape(NI * T, H * D)
    got = out.float().cpu()
    assert rel_err(got.numpy(), ref.numpy()) <= 1e-2
    assert cosine(got.numpy(), ref.numpy()) >= 0.9999


@pytest.mark.parametrize("D", [8, 64, 72, 128, 136, 200])
@pytest.mark.parametrize("S", [100, 300])
def test_other_head_dims_and_shared_keys(cuda_device, D, S):
    """Head dims that fill the 64-column blocks partly, and 3 x 2 groups of queries that all read the SAME keys
    and values (group strides 0)."""
    from turbopi_b200 import _lib, ops
    g = torch.Generator().manual_seed(D * 7 + S)
    A, B, R = 3, 2, 70
    q = torch.randn(A, B, R, D, generator=g).to(BF)
    k = torch.randn(S, D, generator=g).to(BF)
    v = torch.randn(S, D, generator=g).to(BF)
    out = torch.full((A, B, R, D), 5.0, dtype=BF, device=cuda_device)
    kd, vd = k.to(cuda_device), v.to(cuda_device)
    ops.attention(q.to(cuda_device), kd.expand(A, B, S, D), vd.expand(A, B, S, D), out, D ** -0.5)
    torch.cuda.synchronize()
    assert _lib.load().tpb200_device_error(0) == 0
    ref = F.scaled_dot_product_attention(q.float(), k.float().expand(A, B, S, D), v.float().expand(A, B, S, D))
    got = out.float().cpu()
    assert rel_err(got.numpy(), ref.numpy()) <= 1e-2
    assert cosine(got.numpy(), ref.numpy()) >= 0.9999


@pytest.mark.parametrize("tiled", [True, False])
@pytest.mark.parametrize("L,S,heads", [(50, 762, 8), (712, 712, 8), (130, 200, 8), (9, 300, 2)])
def test_fused_operand_output_equals_attention_then_row_kernel(cuda_device, L, S, heads, tiled):
    """attention(..., quant=) writes the next GEMM's operand itself, in either operand form: the codes, scales and
    row multipliers are byte for byte what attention followed by the row kernel's plain mode produces."""
    from turbopi_b200 import _lib, ops
    g = torch.Generator().manual_seed(L + S)
    D = 256
    q = (torch.randn(L, heads * D, generator=g) * 2.0).to(BF).to(cuda_device)
    k = torch.randn(S, D, generator=g).to(BF).to(cuda_device)
    v = torch.randn(S, D, generator=g).to(BF).to(cuda_device)
    valid = torch.ones(S, dtype=torch.bool)
    valid[S // 3: S // 3 + 20] = False
    bias = torch.where(valid, 0.0, opi.MASKED).to(BF).to(cuda_device)
    out = torch.empty_like(q)
    ops.attention(q.view(L * heads, D), k, v, out.view(L * heads, D), D ** -0.5, bias)
    two_step = ops.QuantBuf(L, heads * D, 3, cuda_device, tiled=tiled)
    ops.rowop(_lib.ROW_NONE, out, heads * D, two_step)
    fused = ops.QuantBuf(L, heads * D, 3, cuda_device, tiled=tiled)
    out2 = torch.empty_like(q)
    ops.attention(q.view(L * heads, D), k, v, out2.view(L * heads, D), D ** -0.5, bias, quant=fused, rows_per_token=heads)
    only = ops.QuantBuf(L, heads * D, 3, cuda_device, tiled=tiled)
    ops.attention(q.view(L * heads, D), k, v, None, D ** -0.5, bias, quant=only, rows_per_token=heads)
    torch.cuda.synchronize()
    assert _lib.load().tpb200_device_error(0) == 0
    assert torch.equal(out, out2)
    for got in (fused, only):
        assert torch.equal(got.packed, two_step.packed)
        assert tiled or torch.equal(got.sf, two_step.sf)
        assert torch.equal(got.row_scale, two_step.row_scale)


def test_attention_refuses_bad_arguments(cuda_device):
    from turbopi_b200 import ops
    from turbopi_b200._lib import TurboPiError
    q = torch.zeros((16, 256), dtype=BF, device=cuda_device)
    with pytest.raises(TurboPiError):
        ops.attention(q.float(), q, q, q, 1.0)                        # not bf16
    with pytest.raises(TurboPiError):
        ops.attention(q, q[:, :128], q, q, 1.0)                       # head_dim mismatch
    wide = torch.zeros((16, 264), dtype=BF, device=cuda_device)
    with pytest.raises(TurboPiError):
        ops.attention(wide, wide, wide, wide, 1.0)                    # head_dim > 256
    with pytest.raises(TurboPiError):
        ops.attention(q[:, :12], q[:, :12], q[:, :12], q[:, :12], 1.0)   # head_dim not a multiple of 8
