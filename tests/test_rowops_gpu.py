"""Row kernel (norms, gated residual, GELU * up, activation-piece quantiser) against a torch fp32
restatement of the PyTorch modules it replaces
(openpi/src/openpi/models_pytorch/transformers_replace/models/gemma/modeling_gemma.py:49-129, 212-230):
bf16 results equal up to a last-place flip where the fp32 reduction order differs; the e2m1 pieces of
the tiled operand image add up to the bf16 row within 5e-3 of the row maximum (each piece leaves at
most 1/6 of its block maximum, plus the round-up of its scale)."""
import numpy as np
import pytest
import torch

from oracle import formats

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _detile(image, M, K, P):
    """Tiled A image -> (codes [P, M, K] uint8, scales [P, M, K/16] float32)."""
    img = image.cpu().numpy()
    KS = (K + 255) // 256
    m = np.arange(M)[:, None]
    kb = np.arange(K // 16)[None, :]
    r, j = m % 128, kb % 16
    blk = ((m // 128) * KS + kb // 16).astype(np.int64) * (P * 18432)
    codes = np.zeros((P, M, K), dtype=np.uint8)
    scales = np.zeros((P, M, K // 16), dtype=np.float32)
    for p in range(P):
        c0 = blk + p * 16384 + r * 128 + (((j >> 1) ^ (r & 7)) << 4) + (j & 1) * 8
        by = img[c0[..., None] + np.arange(8)]                       # [M, K/16, 8] bytes = 16 codes
        lo, hi = by & 0xF, by >> 4
        codes[p] = np.stack([lo, hi], axis=-1).reshape(M, K)
        s0 = blk + P * 16384 + p * 2048 + (j >> 2) * 512 + (r % 32) * 16 + (r // 32) * 4 + (j & 3)
        scales[p] = formats.e4m3_decode(img[s0])
    return codes, scales


def _reconstruct(q, M, K):
    codes, scales = _detile(q.packed, M, K, q.pieces)
    x = (formats.E2M1_LUT[codes] * np.repeat(scales, 16, axis=2)).sum(axis=0)
    return x * q.row_scale.cpu().numpy()[:, None]


def _close_bf16(got, ref, min_equal=0.995, ulps=1, offset=None):
    """Equal except for last-place flips; `offset` is an addend of the result (a shift / bias) whose
    magnitude bounds the rounding step when the sum cancels."""
    got, ref = got.float(), ref.float()
    assert (got == ref).float().mean().item() >= min_equal
    scale = ref.abs() if offset is None else ref.abs() + offset.float().abs()
    tol = scale * 2.0 ** -7 * ulps + 1e-30        # results below ~1e-30 may be flushed to zero
    assert ((got - ref).abs() <= tol).all()


def _gelu_tanh(x):
    return 0.5 * x * (1 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


@pytest.mark.parametrize("M,K", [(50, 1024), (712, 2048), (300, 1152), (5, 16), (130, 4304), (64, 16384)])
@pytest.mark.parametrize("mode", ["none", "rms", "ada", "layernorm", "gelu_mul", "rms_residual_gate"])
def test_row_kernel_matches_module_arithmetic(cuda_device, M, K, mode):
    from turbopi_b200 import _lib, ops
    g = torch.Generator().manual_seed(M * 7 + K)
    x = (torch.randn(M, K, generator=g) * torch.rand(M, 1, generator=g) * 4).to(BF)
    w0 = (torch.randn(K, generator=g) * 0.2).to(BF)
    w1 = (torch.randn(K, generator=g) * 0.2).to(BF)
    res = torch.randn(M, K, generator=g).to(BF)
    gate = torch.randn(K, generator=g).to(BF)
    d = lambda t: t.to(cuda_device)
    q = ops.QuantBuf(M, K, 3, cuda_device)
    y = torch.empty((M, K), dtype=BF, device=cuda_device)
    eps = 1e-6
    xf = x.float()
    h_out = None
    if mode == "none":
        ops.rowop(_lib.ROW_NONE, d(x), K, q, y_out=y)
        ref = x
    elif mode == "rms":
        ops.rowop(_lib.ROW_RMSNORM, d(x), K, q, w0=d(w0), eps=eps, y_out=y)
        ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1 + w0.float())).to(BF)
    elif mode == "ada":
        ops.rowop(_lib.ROW_ADARMS, d(x), K, q, w0=d(w0), w1=d(w1), eps=eps, y_out=y)
        ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1 + w0.float()) + w1.float()).to(BF)
    elif mode == "layernorm":
        ops.rowop(_lib.ROW_LAYERNORM, d(x), K, q, w0=d(w0), w1=d(w1), eps=eps, y_out=y)
        mu = xf.mean(-1, keepdim=True)
        var = (xf - mu).pow(2).mean(-1, keepdim=True)
        ref = ((xf - mu) * torch.rsqrt(var + eps) * w0.float() + w1.float()).to(BF)
    elif mode == "gelu_mul":
        gu = torch.cat([x, res], dim=1).contiguous()
        ops.rowop(_lib.ROW_GELU_MUL, d(gu), K, q, y_out=y)
        # float64 evaluation of the tanh GELU in its cancellation-free form: torch's own fp32 evaluation of 0.5 x (1 + tanh z) loses
        # relative accuracy in the negative tail (1 + tanh z cancels) and differs from this in ~4 % of the
        # bf16 results there, by amounts far below one bf16 step of the row's significant values
        xd = xf.double()
        exact = xd / (1 + torch.exp(-1.5957691216057308 * (xd + 0.044715 * xd ** 3)))   # == 0.5 x (1 + tanh z)
        ref = (exact.float().to(BF).float() * res.float()).to(BF)
    else:
        h_out = torch.empty((M, K), dtype=BF, device=cuda_device)
        ops.rowop(_lib.ROW_RMSNORM, d(x), K, q, res_in=d(res), gate=d(gate), h_out=h_out, w0=d(w0), eps=eps, y_out=y)
        h = (res.float() + (xf * gate.float()).to(BF).float()).to(BF)
        assert torch.equal(h_out.cpu(), h)
        hf = h.float()
        ref = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * (1 + w0.float())).to(BF)
    assert _lib.load().tpb200_device_error(0) == 0
    if mode == "none":
        assert torch.equal(y.cpu(), ref)
    elif mode == "gelu_mul":
        _close_bf16(y.cpu(), ref, min_equal=0.98, ulps=2)     # hardware exp, then two bf16 roundings
        torch_ref = (torch.nn.functional.gelu(x, approximate="tanh").float() * res.float()).to(BF)
        assert (y.cpu().float() - torch_ref.float()).abs().max().item() <= 2.0 ** -7 * torch_ref.float().abs().max().item()
    else:
        _close_bf16(y.cpu(), ref, offset=w1[None, :] if mode in ("ada", "layernorm") else None)
    # the quantised operand carries the row the kernel wrote
    yk = y.float().cpu().numpy()
    rec = _reconstruct(q, M, K)
    err = np.abs(rec - yk).max(axis=1) / np.maximum(np.abs(yk).max(axis=1), 1e-30)
    assert err.max() <= 5e-3, err.max()


def test_row_kernel_rowmajor_operand_equals_tiled(cuda_device):
    """The same codes and scales land in the row-major operand and in the tiled image."""
    from turbopi_b200 import _lib, ops
    M, K, P = 200, 1152, 3
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(3)).to(BF).to(cuda_device)
    qt = ops.QuantBuf(M, K, P, cuda_device, tiled=True)
    qr = ops.QuantBuf(M, K, P, cuda_device, tiled=False)
    ops.rowop(_lib.ROW_NONE, x, K, qt)
    ops.rowop(_lib.ROW_NONE, x, K, qr)
    codes, scales = _detile(qt.packed, M, K, P)
    rm = qr.packed.cpu().numpy().reshape(P, qr.piece_rows, qr.pitch)[:, :M, :K // 2]
    rm_codes = np.stack([rm & 0xF, rm >> 4], axis=-1).reshape(P, M, K)
    assert (codes == rm_codes).all()
    assert torch.equal(qt.row_scale, qr.row_scale)
    packed2, sf2, rs2, _ = ops.nvfp4_quantize_act_pieces(x, P)
    assert torch.equal(packed2.reshape(P, -1, qr.pitch)[:, :M], qr.packed.reshape(P, -1, qr.pitch)[:, :M])
    assert torch.equal(rs2, qr.row_scale)


def _rowops_golden():
    from pathlib import Path
    return dict(np.load(Path(__file__).resolve().parent / "golden" / "pi05_rowops.npz"))


@pytest.mark.parametrize("K", [1024, 2048])
def test_row_kernel_matches_reference_modules(cuda_device, K):
    """The row kernel against outputs of the reference's own GemmaRMSNorm (plain and adaptive),
    _gated_residual and nn.LayerNorm run in bf16 (tests/golden/pi05_rowops.npz, made by
    tests/golden/make_golden_model.py from transformers_replace/models/gemma/modeling_gemma.py:49-129,212-230)."""
    from turbopi_b200 import _lib, ops
    g = _rowops_golden()
    t = lambda k: torch.from_numpy(g[k]).to(BF).to(cuda_device)
    x, res = t(f"rms{K}.x"), t(f"rms{K}.res")
    M = x.shape[0]
    q = ops.QuantBuf(M, K, 3, cuda_device)
    y = torch.empty((M, K), dtype=BF, device=cuda_device)
    h = torch.empty((M, K), dtype=BF, device=cuda_device)
    # plain RMSNorm after an ungated residual
    ops.rowop(_lib.ROW_RMSNORM, x, K, q, res_in=res, h_out=h, w0=t(f"rms{K}.w"), eps=1e-6, y_out=y)
    assert torch.equal(h.cpu(), t(f"rms{K}.h").cpu())
    _close_bf16(y.cpu(), t(f"rms{K}.y").cpu())
    # adaptive RMSNorm after a gated residual; scale / shift / gate are the chunks of dense(cond)
    mod = t(f"ada{K}.mod")
    scale, shift, gate = mod[:K].contiguous(), mod[K:2 * K].contiguous(), mod[2 * K:].contiguous()
    assert torch.equal(gate.cpu(), t(f"ada{K}.gate").cpu())
    ops.rowop(_lib.ROW_ADARMS, x, K, q, res_in=res, gate=t(f"ada{K}.gate_prev"), h_out=h, w0=scale, w1=shift, eps=1e-6, y_out=y)
    assert torch.equal(h.cpu(), t(f"ada{K}.h").cpu())
    _close_bf16(y.cpu(), t(f"ada{K}.y").cpu(), offset=shift.cpu()[None, :])
    # LayerNorm (SigLIP) on the same residual sum
    ops.rowop(_lib.ROW_LAYERNORM, x, K, q, res_in=res, h_out=h, w0=t(f"ln{K}.w"), w1=t(f"ln{K}.b"), eps=1e-6, y_out=y)
    _close_bf16(y.cpu(), t(f"ln{K}.y").cpu(), min_equal=0.99, ulps=2, offset=t(f"ln{K}.b").cpu()[None, :])
    assert _lib.load().tpb200_device_error(0) == 0


def test_gelu_mul_matches_reference_mlp(cuda_device):
    """GELU(gate) * up of the reference's GemmaMLP (captured at the input of its down projection) and the
    MLP output through the weight-only GEMMs."""
    from turbopi_b200 import _lib, ops
    g = _rowops_golden()
    gu = torch.from_numpy(g["mlp.gate_up"]).to(BF).to(cuda_device)
    I = gu.shape[1] // 2
    M = gu.shape[0]
    q = ops.QuantBuf(M, I, 3, cuda_device)
    y = torch.empty((M, I), dtype=BF, device=cuda_device)
    ops.rowop(_lib.ROW_GELU_MUL, gu, I, q, y_out=y)
    ref = torch.from_numpy(g["mlp.act"]).to(BF)
    # torch's fp32 tanh form loses accuracy in the negative tail; bound by one bf16 step of the row maximum
    assert (y.cpu().float() - ref.float()).abs().max().item() <= 2.0 ** -7 * ref.float().abs().max().item()
    assert (y.cpu() == ref).float().mean().item() >= 0.95
    assert _lib.load().tpb200_device_error(0) == 0
