"""The reference's module surfaces (NVFP4PackedLinear / NVFP4PackedMLP / replace_mlp_with_nvfp4_packed,
openpi/nvfp4_packed_plugin/python/nvfp4_packed.py:166-450) reach the tensor-core kernels: results against
dequantise-then-matmul of the stored weights for decode- and prefix-sized inputs, and the launch count."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from conftest import cosine, rel_err
from oracle import nvfp4 as onv

pytestmark = pytest.mark.gpu


def _kernel_names(fn):
    """Names of the CUDA kernels `fn` launches (None if the profiler is not usable here)."""
    try:
        from torch.profiler import ProfilerActivity, profile
        fn()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            fn()
            torch.cuda.synchronize()
        names = [e.name for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "Memcpy" not in e.name
                 and "Memset" not in e.name]
        return names or None
    except Exception:
        return None


def _dequant(layer):
    return onv.dequantize(layer.weight_packed.cpu().numpy(), layer.weight_scales.cpu().numpy(), 16,
                          float(layer.global_scale), scale_is_e4m3=True)


@torch.no_grad()
@pytest.mark.parametrize("T", [1, 4, 5, 16, 50, 712])
@pytest.mark.parametrize("act", ["none", "gelu"])
def test_nvfp4_packed_linear_dispatches_to_tensor_cores(cuda_device, T, act):
    from turbopi_b200 import _lib
    from turbopi_b200.nvfp4_packed import NVFP4PackedLinear
    g = torch.Generator().manual_seed(T)
    lin = nn.Linear(1024, 768, bias=True)
    lin.weight.data = torch.randn(768, 1024, generator=g) * 0.02
    lin.bias.data = torch.randn(768, generator=g) * 0.1
    layer = NVFP4PackedLinear.from_linear(lin.to(cuda_device), activation=act, fmt="nvfp4")
    assert layer.tensor_core_ready()
    x = torch.randn(T, 1024, generator=g).to(torch.bfloat16)
    y = layer(x.to(cuda_device))
    assert y.shape == (T, 768) and y.dtype == torch.bfloat16
    assert _lib.load().tpb200_device_error(0) == 0
    ref = onv.gemv_dequant_matmul(x.float().numpy(), layer.weight_packed.cpu().numpy(), layer.weight_scales.cpu().numpy(),
                                  lin.bias.data.cpu().numpy(), 1 if act == "gelu" else 0, 16, float(layer.global_scale), True)
    assert rel_err(y.float().cpu().numpy(), ref) <= 1e-2
    assert cosine(y.float().cpu().numpy(), ref) >= 0.999
    names = _kernel_names(lambda: layer(x.to(cuda_device)))
    if names is not None:
        gemm = [n for n in names if "nvfp4_gemm_kernel" in n]
        gemv = [n for n in names if "nvfp4_gemv_tc_kernel" in n]
        cuda_core = [n for n in names if "gemv_rowmajor" in n]
        assert len(gemm) + len(gemv) + len(cuda_core) == 1, names     # ONE weight pass, whatever the token count
        assert (len(cuda_core) == 1) == (T <= 4)                      # a few tokens: the packed rows as stored
        assert (len(gemv) == 1) == (4 < T <= 16)
    # leading dimensions are kept
    y3 = layer(x.to(cuda_device).reshape(1, T, 1024))
    assert y3.shape == (1, T, 768) and torch.equal(y3[0], y)


class _GemmaMLP(nn.Module):
    def __init__(self, hidden, inter):
        super().__init__()
        self.gate_proj = nn.Linear(hidden, inter, bias=False)
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)


def _mlp_reference(mlp, x, act):
    """fp32 MLP over the dequantised stored weights with the bf16 roundings of the bf16 module."""
    r = lambda t: t.to(torch.bfloat16).float()
    wg, wu, wd = (torch.from_numpy(_dequant(l)) for l in (mlp.gate_proj, mlp.up_proj, mlp.down_proj))
    xf = x.float()
    gate, up = r(xf @ wg.t()), r(xf @ wu.t())
    a = torch.nn.functional.gelu(gate, approximate="tanh") if act == "gelu" else torch.nn.functional.silu(gate)
    return r(r(r(a) * up) @ wd.t())


@torch.no_grad()
@pytest.mark.parametrize("T", [1, 16, 712])
@pytest.mark.parametrize("act", ["gelu", "silu"])
def test_nvfp4_packed_mlp_runs_gate_and_up_as_one_launch(cuda_device, T, act):
    from turbopi_b200 import _lib
    from turbopi_b200.nvfp4_packed import NVFP4PackedMLP
    torch.manual_seed(5)
    src = _GemmaMLP(512, 2048)
    for p in src.parameters():
        p.data.normal_(0, 0.03)
    mlp = NVFP4PackedMLP.from_gemma_mlp(src.to(cuda_device), gate_activation=act, fmt="nvfp4")
    assert mlp.gate_proj.global_scale == mlp.up_proj.global_scale
    x = torch.randn(T, 512).to(torch.bfloat16)
    y = mlp(x.to(cuda_device))
    assert _lib.load().tpb200_device_error(0) == 0
    ref = _mlp_reference(mlp, x, act)
    assert rel_err(y.float().cpu().numpy(), ref.numpy()) <= 1.5e-2
    assert cosine(y.float().cpu().numpy(), ref.numpy()) >= 0.999
    names = _kernel_names(lambda: mlp(x.to(cuda_device)))
    if names is not None:
        weight_passes = [n for n in names if "nvfp4_gemm_kernel" in n or "nvfp4_gemv_tc_kernel" in n or "gemv_rowmajor" in n]
        assert len(weight_passes) == 2, names                         # gate+up together, then down


@torch.no_grad()
def test_replace_mlp_with_nvfp4_packed_on_a_gemma_shaped_model(cuda_device):
    """The drop-in call of the reference: every layer's MLP replaced, outputs close to the fp32 module."""
    from turbopi_b200.nvfp4_packed import NVFP4PackedMLP, replace_mlp_with_nvfp4_packed

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.mlp = _GemmaMLP(256, 1024)

    class Holder(nn.Module):
        pass

    torch.manual_seed(9)
    model = Holder()
    lm = Holder()
    lm.layers = nn.ModuleList([Layer() for _ in range(3)])
    model.paligemma_with_expert = Holder()
    model.paligemma_with_expert.paligemma = Holder()
    model.paligemma_with_expert.paligemma.language_model = lm
    for p in lm.parameters():
        p.data.normal_(0, 0.03)
    model.to(cuda_device)
    x = torch.randn(40, 256, device=cuda_device).to(torch.bfloat16)
    want = []
    for layer in lm.layers:
        m = layer.mlp
        h = torch.nn.functional.gelu(x.float() @ m.gate_proj.weight.t(), approximate="tanh") * (x.float() @ m.up_proj.weight.t())
        want.append(h @ m.down_proj.weight.t())
    assert replace_mlp_with_nvfp4_packed(model, gate_activation="gelu", target_layers=[0, 2]) == 2
    assert isinstance(lm.layers[0].mlp, NVFP4PackedMLP) and not isinstance(lm.layers[1].mlp, NVFP4PackedMLP)
    for i in (0, 2):
        y = lm.layers[i].mlp(x)
        # 4-bit weights against the unquantised module: a few per cent
        assert cosine(y.float().cpu().numpy(), want[i].cpu().numpy()) >= 0.98
