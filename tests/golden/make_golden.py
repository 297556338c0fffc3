#!/usr/bin/env python3
"""Regenerate tests/golden/*.npz by running the reference's own Python code.

Runs only where the reference checkout is present (pass its root as argv[1],
default: the directory named by $TURBOPI_REFERENCE).  The fixtures are small
seeded cases; the tests compare the CPU oracle (and through it the CUDA path)
with them.  Nothing else in the repository needs the reference at run time.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py <reference-root>
"""
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, str(path))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    ref = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["TURBOPI_REFERENCE"])
    src = ref / "openpi" / "src"
    sys.path.insert(0, str(src))
    torch.set_grad_enabled(False)
    torch.set_num_threads(1)

    # ---------------- INT4 packers (openpi/src/openpi/utils/w4a16_packer.py) ----------
    pk = _load("ref_w4a16_packer", src / "openpi" / "utils" / "w4a16_packer.py")
    g = torch.Generator().manual_seed(1234)
    w = torch.randn(24, 128, generator=g)
    w[3, 32:64] = 0.0                       # an all-zero block
    w[5, 0] = 7.0; w[5, 1] = 3.5            # exact .5 tie after scaling by max/7 = 1
    w[5, 2] = -2.5; w[5, 3:32] *= 0.1
    fast = pk.W4A16PackerFast().pack(w)
    basic = pk.W4A16Packer().pack(w)
    np.savez_compressed(
        OUT / "int4_packers.npz",
        weight=w.numpy(),
        fast_packed=fast.weight_packed.numpy().astype(np.int64).astype(np.uint32).view(np.int32)
        if fast.weight_packed.dtype != torch.int32 else fast.weight_packed.numpy(),
        fast_scales=fast.scales.numpy(),
        basic_packed=basic.weight_packed.numpy(),
        basic_scales=basic.scales.numpy(),
        basic_unpacked=pk.W4A16Packer().unpack(basic).numpy(),
    )

    # ---------------- nvfp4_packed_plugin python ---------------------------------------
    npk = _load("ref_nvfp4_packed", ref / "openpi" / "nvfp4_packed_plugin" / "python" / "nvfp4_packed.py")
    g = torch.Generator().manual_seed(4321)
    w = torch.randn(40, 128, generator=g) * 0.02
    w[7, 32:64] = 0.0
    w[9, 0:32] = torch.tensor([6.0, 5.0, 3.5, 2.5, 1.75, 1.25, 0.75, 0.25] * 4) * 0.01   # every tie point
    w[9, 16:32] *= -1
    q, s = npk.quantize_to_nvfp4(w, 32)
    packed = npk.pack_nvfp4(q)
    layer = npk.NVFP4PackedLinear.__new__(npk.NVFP4PackedLinear)
    torch.nn.Module.__init__(layer)
    layer.in_features, layer.out_features, layer.block_size = 128, 40, 32
    layer.weight_packed, layer.weight_scales = packed, s
    layer.bias = torch.nn.Parameter(torch.randn(40, generator=g) * 0.1)
    x = torch.randn(5, 128, generator=g)
    outs = {f"out_act{a}": layer._forward_dequant_gemm(x, a).detach().numpy() for a in (0, 1, 2)}
    np.savez_compressed(
        OUT / "nvfp4_packed.npz", weight=w.numpy(), quantized=q.numpy(), scales=s.numpy(),
        packed=packed.numpy(), unpacked=npk.unpack_nvfp4(packed, 40, 128).numpy(),
        x=x.numpy(), bias=layer.bias.detach().numpy(), **outs)

    # ---------------- kv_fuse_plugin python --------------------------------------------
    kvf = _load("ref_kv_fuse", ref / "openpi" / "kv_fuse_plugin" / "python" / "kv_fuse.py")
    g = torch.Generator().manual_seed(99)
    H, NH, NKV, D = 64, 2, 1, 32
    Wq = torch.randn(NH * D, H, generator=g) * 0.05
    Wk = torch.randn(NKV * D, H, generator=g) * 0.05
    Wv = torch.randn(NKV * D, H, generator=g) * 0.05
    Wk[0, :8] = torch.tensor([-1e-9, 1e-9, -0.0, 0.0, -1e-4, 1e-4, -0.3, 0.3])  # tiny negatives -> code 8
    mod = kvf.FusedQKVProjection.__new__(kvf.FusedQKVProjection)
    torch.nn.Module.__init__(mod)
    mod.hidden_size, mod.num_heads, mod.num_kv_heads, mod.head_dim = H, NH, NKV, D
    mod.block_size, mod.q_dim, mod.kv_dim = 32, NH * D, NKV * D
    (mod.Wq_packed, mod.scale_Wq) = kvf.quantize_to_fp4(Wq, 32)
    (mod.Wk_packed, mod.scale_Wk) = kvf.quantize_to_fp4(Wk, 32)
    (mod.Wv_packed, mod.scale_Wv) = kvf.quantize_to_fp4(Wv, 32)
    x = torch.randn(3, H, generator=g)
    Kc = torch.full((3, 6, NKV, D), -7.0)
    Vc = torch.full((3, 6, NKV, D), -7.0)
    Q, Kc, Vc = mod._forward_fallback(x, Kc, Vc, 4)
    np.savez_compressed(
        OUT / "kv_fuse.npz", Wq=Wq.numpy(), Wk=Wk.numpy(), Wv=Wv.numpy(), x=x.numpy(),
        Wq_packed=mod.Wq_packed.numpy(), scale_Wq=mod.scale_Wq.numpy(),
        Wk_packed=mod.Wk_packed.numpy(), scale_Wk=mod.scale_Wk.numpy(),
        Wv_packed=mod.Wv_packed.numpy(), scale_Wv=mod.scale_Wv.numpy(),
        Wk_dequant=mod._dequantize(mod.Wk_packed, mod.scale_Wk, NKV * D, H).numpy(),
        Q=Q.numpy(), K_cache=Kc.numpy(), V_cache=Vc.numpy(), cache_pos=np.int64(4))

    # ---------------- nvfp4_mlp.py simulation path --------------------------------------
    sim = _load("ref_nvfp4_mlp", src / "openpi" / "models_pytorch" / "nvfp4_mlp.py")
    g = torch.Generator().manual_seed(777)
    w = torch.randn(48, 128, generator=g) * 0.02
    w[0, 5] = 0.3                                            # an outlier, so the MSE search moves a scale
    x = torch.randn(9, 128, generator=g)
    wq_mse, ws_mse = sim.quantize_to_nvfp4_sim(w, 32, use_mse_search=True, use_triton=False)
    wq_mm, ws_mm = sim.quantize_to_nvfp4_sim(w, 32, use_mse_search=False, use_triton=False)
    wd = sim.dequantize_nvfp4_sim(wq_mse, ws_mse, 32, use_fp8_scales=True, use_triton=False)
    xq, xs = sim.quantize_to_nvfp4_sim(x, 32, use_mse_search=False, use_triton=False)
    xd = sim.dequantize_nvfp4_sim(xq, xs, 32, use_fp8_scales=True, use_triton=False)
    y = torch.nn.functional.linear(xd.float(), wd.float())
    sw = sim.swizzle_scales_for_cutlass(ws_mse, 48, 4)
    np.savez_compressed(
        OUT / "nvfp4_sim.npz", weight=w.numpy(), x=x.numpy(),
        wq_mse=wq_mse.numpy(), ws_mse=ws_mse.numpy(), wq_minmax=wq_mm.numpy(), ws_minmax=ws_mm.numpy(),
        w_dequant_fp8=wd.numpy(), xq=xq.numpy(), xs=xs.numpy(), x_dequant_fp8=xd.numpy(), y=y.numpy(),
        w_packed=sim.pack_nvfp4_data(wq_mse, 32).numpy(),
        ws_fp8_bytes=sim.convert_scales_to_fp8(ws_mse).numpy(),
        ws_swizzled=sw.numpy(),
        linspace=torch.linspace(0.7, 1.0, 10).numpy())

    # ---------------- RoPE restatement (openpi/src/openpi/inference/w4a16_tvm_kv_cache.py) ----
    # The module's import list pulls TensorRT/TVM helpers lazily; the RoPE classes
    # themselves only need torch, so run exactly those definitions.
    text = (src / "openpi" / "inference" / "w4a16_tvm_kv_cache.py").read_text().splitlines()
    start = next(i for i, l in enumerate(text) if l.startswith("class RotaryEmbedding"))
    end = next(i for i, l in enumerate(text) if l.startswith("class W4A16TVMMLP"))
    ns = {"torch": torch, "nn": torch.nn, "Tuple": tuple, "ROPE_THETA": 10000.0}
    exec("from typing import Tuple\n" + "\n".join(text[start:end]), ns)
    g = torch.Generator().manual_seed(5)
    S, NH, D = 13, 2, 256
    q = torch.randn(1, NH, S, D, generator=g).to(torch.bfloat16)
    k = torch.randn(1, 1, S, D, generator=g).to(torch.bfloat16)
    pos = torch.tensor([[0, 1, 2, 3, 7, 50, 199, 200, 511, 512, 700, 711, 1023]])
    rope = ns["RotaryEmbedding"](D, dtype=torch.bfloat16)
    cos, sin = rope(q, pos)
    qe, ke = ns["apply_rotary_pos_emb"](q, k, cos, sin)
    np.savez_compressed(
        OUT / "rope.npz", positions=pos[0].numpy(), q=q.float().numpy(), k=k.float().numpy(),
        cos=cos.float().numpy(), sin=sin.float().numpy(),
        q_embed=qe.float().numpy(), k_embed=ke.float().numpy(),
        inv_freq=rope.inv_freq.float().numpy())
    print("wrote", sorted(p.name for p in OUT.glob("*.npz")))


if __name__ == "__main__":
    main()
