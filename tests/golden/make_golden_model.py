#!/usr/bin/env python3
"""Regenerate tests/golden/pi05_model.npz, pi05_rowops.npz and policy.npz by running the reference's own code.

The reference model cannot be constructed here (its constructor wants a patched `transformers`
4.53.2 install and a checkpoint), but the classes and methods that define the arithmetic depend on
`torch` only.  This script executes exactly those definitions out of the reference's files:

  transformers_replace/models/gemma/modeling_gemma.py    GemmaRMSNorm (plain + adaptive), GemmaMLP,
        GemmaRotaryEmbedding, rotate_half, apply_rotary_pos_emb, _gated_residual, GemmaAttention,
        GemmaDecoderLayer
  transformers_replace/models/siglip/modeling_siglip.py  SiglipVisionEmbeddings, SiglipAttention,
        SiglipMLP, SiglipEncoderLayer, SiglipEncoder, SiglipVisionTransformer
  models_pytorch/pi0_pytorch.py                          create_sinusoidal_pos_embedding,
        make_att_2d_masks and the PI0Pytorch methods embed_prefix, compute_prefix_kv_cache,
        precompute_graph_tensors, denoise_step_graphed, denoise_step_with_cache

on a small randomly initialised model (names the files import from `transformers` are replaced by the
few plain-torch stand-ins below: the default RoPE frequencies, the tanh-GELU entry of ACT2FN, output
containers).  Runs only where the reference checkout is present:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_model.py <reference-root>
"""
import math
import os
import sys
import types
from pathlib import Path
from types import SimpleNamespace as NS

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn

OUT = Path(__file__).resolve().parent
FUTURE = "from __future__ import annotations\n"


def _between(lines, start, end):
    i = next(k for k, l in enumerate(lines) if l.startswith(start))
    j = next(k for k, l in enumerate(lines) if k > i and l.startswith(end)) if end else len(lines)
    return "\n".join(lines[i:j]) + "\n"


class _Output:
    """Stand-in for transformers' ModelOutput containers: attribute bag."""

    def __init__(self, **kw):
        self.__dict__.update(kw)


def _default_rope(config, device=None):
    # transformers 4.53.2 `_compute_default_rope_parameters`: 1 / base^(2i/d), attention scaling 1
    dim = config.head_dim
    inv = 1.0 / (config.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    return inv, 1.0


def load_reference(ref):
    mp = ref / "openpi" / "src" / "openpi" / "models_pytorch"
    from typing import Any, Callable, Optional, Union
    common = dict(torch=torch, nn=nn, F=F, math=math, Optional=Optional, Callable=Callable, Union=Union, Any=Any,
                  ACT2FN={"gelu_pytorch_tanh": lambda x: F.gelu(x, approximate="tanh")},
                  GradientCheckpointingLayer=nn.Module, ALL_ATTENTION_FUNCTIONS={},
                  can_return_tuple=lambda f: f, auto_docstring=lambda f: f,
                  BaseModelOutput=_Output, BaseModelOutputWithPooling=_Output)

    gl = (mp / "transformers_replace" / "models" / "gemma" / "modeling_gemma.py").read_text().splitlines()
    gemma = dict(common, ROPE_INIT_FUNCTIONS={"default": _default_rope}, dynamic_rope_update=lambda f: f)
    exec(FUTURE + _between(gl, "class GemmaRMSNorm", "@auto_docstring"), gemma)

    sl = (mp / "transformers_replace" / "models" / "siglip" / "modeling_siglip.py").read_text().splitlines()
    siglip = dict(common)
    exec(FUTURE + _between(sl, "class SiglipVisionEmbeddings", "class SiglipTextEmbeddings"), siglip)
    exec(FUTURE + _between(sl, "def eager_attention_forward", "@auto_docstring"), siglip)
    exec(FUTURE + _between(sl, "class SiglipEncoder(", "class SiglipTextTransformer"), siglip)
    exec(FUTURE + _between(sl, "class SiglipVisionTransformer", "class SiglipMultiheadAttentionPoolingHead"), siglip)

    pl = (mp / "pi0_pytorch.py").read_text().splitlines()
    import logging
    pi0 = dict(common, Tensor=torch.Tensor, logging=logging)
    exec(FUTURE + _between(pl, "def get_safe_dtype", None), pi0)

    # the PI0Pytorch methods do `from transformers.models.gemma import modeling_gemma` for
    # apply_rotary_pos_emb and _gated_residual: hand them the definitions executed above
    fake = types.ModuleType("reference_modeling_gemma")
    fake.__dict__.update(gemma)
    import transformers.models.gemma as tg
    tg.modeling_gemma = fake
    sys.modules["transformers.models.gemma.modeling_gemma"] = fake
    return NS(**{k: v for k, v in gemma.items() if isinstance(k, str) and not k.startswith("__")}), \
        NS(**{k: v for k, v in siglip.items() if isinstance(k, str) and not k.startswith("__")}), \
        NS(**{k: v for k, v in pi0.items() if isinstance(k, str) and not k.startswith("__")})


def randomize(module, gen, std=0.05):
    for p in module.parameters():
        p.data = (torch.randn(p.shape, generator=gen) * std).to(p.dtype)


def build_model(G, S, P, cfg, gen):
    """A PI0Pytorch instance assembled from the reference's own layer classes, small and random."""
    def gemma_cfg(width, mlp, layers, adarms):
        return NS(hidden_size=width, intermediate_size=mlp, hidden_act="gelu_pytorch_tanh", head_dim=cfg["head_dim"],
                  num_attention_heads=cfg["heads"], num_key_value_heads=1, attention_bias=False, attention_dropout=0.0,
                  rms_norm_eps=1e-6, use_adarms=adarms, adarms_cond_dim=width if adarms else None,
                  max_position_embeddings=8192, rope_theta=10000.0, rope_scaling=None, _attn_implementation="eager",
                  num_hidden_layers=layers)

    pc = gemma_cfg(cfg["width"], cfg["mlp"], cfg["prefix_layers"], False)
    ec = gemma_cfg(cfg["expert_width"], cfg["expert_mlp"], cfg["expert_layers"], True)
    vc = NS(hidden_size=cfg["vision_width"], image_size=cfg["image_size"], patch_size=cfg["patch"], num_channels=3,
            num_attention_heads=cfg["vision_heads"], attention_dropout=0.0, hidden_act="gelu_pytorch_tanh",
            intermediate_size=cfg["vision_mlp"], layer_norm_eps=1e-6, num_hidden_layers=cfg["vision_layers"],
            _attn_implementation="eager", output_attentions=False, output_hidden_states=False, vision_use_head=False)

    lm = nn.Module()
    lm.layers = nn.ModuleList([G.GemmaDecoderLayer(pc, i) for i in range(pc.num_hidden_layers)])
    lm.embed_tokens = nn.Embedding(cfg["vocab"], cfg["width"])
    lm.rotary_emb = G.GemmaRotaryEmbedding(pc)
    lm.config = pc
    ex = nn.Module()
    ex.layers = nn.ModuleList([G.GemmaDecoderLayer(ec, i) for i in range(ec.num_hidden_layers)])
    ex.norm = G.GemmaRMSNorm(ec.hidden_size, eps=1e-6, cond_dim=ec.hidden_size)
    ex.config = ec
    vt = S.SiglipVisionTransformer(vc)
    proj = nn.Linear(cfg["vision_width"], cfg["width"], bias=True)     # PaliGemmaMultiModalProjector.linear

    m = P.PI0Pytorch.__new__(P.PI0Pytorch)
    nn.Module.__init__(m)
    m.config = NS(action_horizon=cfg["action_horizon"], action_dim=cfg["action_dim"])
    m.pi05 = True
    m.gradient_checkpointing_enabled = False
    m.lm, m.ex, m.vt, m.proj = lm, ex, vt, proj
    m.action_in_proj = nn.Linear(cfg["action_dim"], ec.hidden_size)
    m.action_out_proj = nn.Linear(ec.hidden_size, cfg["action_dim"])
    m.time_mlp_in = nn.Linear(ec.hidden_size, ec.hidden_size)
    m.time_mlp_out = nn.Linear(ec.hidden_size, ec.hidden_size)
    randomize(m, gen)

    def embed_image(img):
        # PaliGemmaModel.get_image_features (transformers_replace/models/paligemma/modeling_paligemma.py:232-245)
        return proj(vt(img).last_hidden_state)

    m.paligemma_with_expert = NS(
        paligemma=NS(language_model=lm), gemma_expert=NS(model=ex), embed_image=embed_image,
        embed_language_tokens=lambda t: lm.embed_tokens(t))
    m.eval()
    return m


def export_weights(m, out):
    """Flat float32 copies of every parameter, in the naming the oracle's weight dict is built from."""
    f = lambda t: t.detach().float().numpy()
    vt = m.vt
    out["v.patch_w"] = f(vt.embeddings.patch_embedding.weight).reshape(vt.embeddings.embed_dim, -1)   # (c, i, j) order
    out["v.patch_b"] = f(vt.embeddings.patch_embedding.bias)
    out["v.pos_emb"] = f(vt.embeddings.position_embedding.weight)
    for i, L in enumerate(vt.encoder.layers):
        a = L.self_attn
        out[f"v.{i}.ln1_w"], out[f"v.{i}.ln1_b"] = f(L.layer_norm1.weight), f(L.layer_norm1.bias)
        out[f"v.{i}.ln2_w"], out[f"v.{i}.ln2_b"] = f(L.layer_norm2.weight), f(L.layer_norm2.bias)
        out[f"v.{i}.qkv"] = np.concatenate([f(a.q_proj.weight), f(a.k_proj.weight), f(a.v_proj.weight)], 0)
        out[f"v.{i}.qkv_b"] = np.concatenate([f(a.q_proj.bias), f(a.k_proj.bias), f(a.v_proj.bias)], 0)
        out[f"v.{i}.out"], out[f"v.{i}.out_b"] = f(a.out_proj.weight), f(a.out_proj.bias)
        out[f"v.{i}.fc1"], out[f"v.{i}.fc1_b"] = f(L.mlp.fc1.weight), f(L.mlp.fc1.bias)
        out[f"v.{i}.fc2"], out[f"v.{i}.fc2_b"] = f(L.mlp.fc2.weight), f(L.mlp.fc2.bias)
    out["v.post_ln_w"], out["v.post_ln_b"] = f(vt.post_layernorm.weight), f(vt.post_layernorm.bias)
    out["projector"], out["projector_b"] = f(m.proj.weight), f(m.proj.bias)
    out["embed_tokens"] = f(m.lm.embed_tokens.weight)

    def dec(prefix, L, adaptive):
        a = L.self_attn
        out[f"{prefix}.qkv"] = np.concatenate([f(a.q_proj.weight), f(a.k_proj.weight), f(a.v_proj.weight)], 0)
        out[f"{prefix}.o"] = f(a.o_proj.weight)
        out[f"{prefix}.gate_up"] = np.concatenate([f(L.mlp.gate_proj.weight), f(L.mlp.up_proj.weight)], 0)
        out[f"{prefix}.down"] = f(L.mlp.down_proj.weight)
        if adaptive:
            out[f"{prefix}.in_dense"], out[f"{prefix}.in_dense_b"] = f(L.input_layernorm.dense.weight), f(L.input_layernorm.dense.bias)
            out[f"{prefix}.post_dense"] = f(L.post_attention_layernorm.dense.weight)
            out[f"{prefix}.post_dense_b"] = f(L.post_attention_layernorm.dense.bias)
        else:
            out[f"{prefix}.in_norm"] = f(L.input_layernorm.weight)
            out[f"{prefix}.post_norm"] = f(L.post_attention_layernorm.weight)

    for i, L in enumerate(m.lm.layers):
        dec(f"p.{i}", L, False)
    for i, L in enumerate(m.ex.layers):
        dec(f"e.{i}", L, True)
    out["e.norm_dense"], out["e.norm_dense_b"] = f(m.ex.norm.dense.weight), f(m.ex.norm.dense.bias)
    for k in ("action_in_proj", "action_out_proj", "time_mlp_in", "time_mlp_out"):
        out[k], out[k + "_b"] = f(getattr(m, k).weight), f(getattr(m, k).bias)


CFG = dict(image_size=56, patch=14, vision_layers=2, vision_width=64, vision_mlp=112, vision_heads=4,
           prefix_layers=2, width=96, mlp=160, heads=4, head_dim=32, text_len=10, vocab=50,
           expert_layers=2, expert_width=64, expert_mlp=96, action_horizon=6, action_dim=32)


def model_fixture(G, S, P):
    gen = torch.Generator().manual_seed(2024)
    cfg = CFG
    m = build_model(G, S, P, cfg, gen)
    out = {"cfg_keys": np.array(sorted(cfg)), "cfg_vals": np.array([cfg[k] for k in sorted(cfg)])}
    export_weights(m, out)

    images_u8 = torch.randint(0, 256, (2, cfg["image_size"], cfg["image_size"], 3), generator=gen, dtype=torch.uint8)
    tokens = torch.randint(0, cfg["vocab"], (cfg["text_len"],), generator=gen)
    noise = torch.randn(cfg["action_horizon"], cfg["action_dim"], generator=gen)
    out.update(images_u8=images_u8.numpy(), tokens=tokens.numpy(), noise=noise.numpy())
    # the reference's image convention after preprocessing: float [-1, 1], [B, C, H, W], one entry per camera
    imgs = [(images_u8[i].float() / 127.5 - 1.0).permute(2, 0, 1)[None] for i in range(2)]

    # case A: everything valid.  case B: the last 3 prompt tokens are padding.  case C: second camera missing too.
    cases = {
        "A": (torch.ones(cfg["text_len"], dtype=torch.bool), [True, True]),
        "B": (torch.arange(cfg["text_len"]) < cfg["text_len"] - 3, [True, True]),
        "C": (torch.arange(cfg["text_len"]) < cfg["text_len"] - 3, [True, False]),
    }
    steps = 3
    for name, (lang_mask, img_valid) in cases.items():
        img_masks = [torch.tensor([v]) for v in img_valid]
        embs, pad, att = m.embed_prefix(imgs, img_masks, tokens[None], lang_mask[None])
        kv = m.compute_prefix_kv_cache(embs, pad, att)
        gt = m.precompute_graph_tensors(1, pad.shape[1], steps, torch.device("cpu"), pad)
        x_t = noise[None].clone()
        v0 = None
        mask = gt["attention_mask"].float()     # the reference builds it in bf16 for its bf16 model; this one is fp32
        for i in range(steps):
            v = m.denoise_step_graphed(x_t, gt["suffix_position_ids"], gt["adarms_conds"][i], kv, mask)
            v0 = v if v0 is None else v0
            x_t = x_t + gt["dt"] * v                                   # Euler update of sample_actions (:928-929)
        out[f"{name}.pad_mask"] = pad[0].numpy()
        out[f"{name}.prefix_embs"] = embs[0].detach().numpy()
        out[f"{name}.position_ids"] = (torch.cumsum(pad, dim=1) - 1)[0].numpy()
        out[f"{name}.suffix_position_ids"] = gt["suffix_position_ids"][0].numpy()
        out[f"{name}.attention_mask_is_zero"] = (gt["attention_mask"][0, 0].float() == 0).numpy()
        out[f"{name}.adarms_conds"] = torch.stack([c[0] for c in gt["adarms_conds"]]).detach().numpy()
        for l, (k, v) in enumerate(kv):
            out[f"{name}.k{l}"], out[f"{name}.v{l}"] = k[0, 0].detach().numpy(), v[0, 0].detach().numpy()
        out[f"{name}.v_step0"] = v0[0].detach().numpy()
        out[f"{name}.actions"] = x_t[0].detach().numpy()
        if name == "A":
            # the unmasked cached step agrees with the graphed one when nothing is padded
            vc = m.denoise_step_with_cache(None, kv, pad, noise[None], torch.tensor([1.0]))
            out["A.v_step0_with_cache"] = vc[0].detach().numpy()
    # sinusoid at the real width, the ten timesteps of a 10-step schedule
    ts = torch.tensor([1.0 + i * (-1.0 / 10) for i in range(10)], dtype=torch.float32)
    out["sinusoid_t"] = ts.numpy()
    out["sinusoid_1024"] = P.create_sinusoidal_pos_embedding(ts, 1024, 4e-3, 4.0, torch.device("cpu")).numpy()
    m2d = P.make_att_2d_masks(torch.tensor([[1, 1, 0, 1, 0]], dtype=torch.bool), torch.tensor([[0, 0, 0, 1, 0]]))
    out["att2d_example"] = m2d[0].numpy()
    np.savez_compressed(OUT / "pi05_model.npz", **out)


def rowops_fixture(G):
    """bf16 inputs / outputs of the reference's norm, gated-residual and MLP-activation arithmetic at the
    kernel's row widths (values stored as float32; all of them are bf16-representable)."""
    gen = torch.Generator().manual_seed(77)
    bf = torch.bfloat16
    out = {}
    for K in (1024, 2048):
        M = 6
        x = (torch.randn(M, K, generator=gen) * 1.5).to(bf)
        res = torch.randn(M, K, generator=gen).to(bf)
        w = (torch.randn(K, generator=gen) * 0.1).to(bf)
        plain = G.GemmaRMSNorm(K, eps=1e-6)
        plain.weight.data = w
        h = G._gated_residual(res, x, None)
        y, g_none = plain(h)
        assert g_none is None
        out[f"rms{K}.x"], out[f"rms{K}.res"], out[f"rms{K}.w"] = x.float().numpy(), res.float().numpy(), w.float().numpy()
        out[f"rms{K}.h"], out[f"rms{K}.y"] = h.float().numpy(), y.float().numpy()

        ada = G.GemmaRMSNorm(K, eps=1e-6, cond_dim=64).to(bf)
        randomize(ada, gen, 0.1)
        cond = torch.randn(1, 64, generator=gen).to(bf)
        gate_prev = (torch.randn(1, 1, K, generator=gen) * 0.5).to(bf)
        h3 = G._gated_residual(res[None], x[None], gate_prev)           # [1, M, K] + [1, M, K] * [1, 1, K]
        y3, gate = ada(h3, cond)
        mod = ada.dense(cond)
        out[f"ada{K}.gate_prev"] = gate_prev[0, 0].float().numpy()
        out[f"ada{K}.h"], out[f"ada{K}.y"] = h3[0].float().numpy(), y3[0].float().numpy()
        out[f"ada{K}.mod"] = mod[0].float().numpy()                     # [3K]: scale | shift | gate
        out[f"ada{K}.gate"] = gate[0, 0].float().numpy()

        ln = nn.LayerNorm(K, eps=1e-6).to(bf)
        randomize(ln, gen, 0.3)
        yl = ln(h)
        out[f"ln{K}.w"], out[f"ln{K}.b"], out[f"ln{K}.y"] = ln.weight.float().detach().numpy(), ln.bias.float().detach().numpy(), yl.float().detach().numpy()
    # GemmaMLP: act_fn(gate_proj(x)) * up_proj(x) in bf16, captured from inside the reference module
    K, I = 256, 512
    mlp = G.GemmaMLP(NS(hidden_size=K, intermediate_size=I, hidden_act="gelu_pytorch_tanh")).to(bf)
    randomize(mlp, gen, 0.08)
    x = (torch.randn(5, K, generator=gen) * 2.0).to(bf)
    grabbed = {}
    hook = mlp.down_proj.register_forward_hook(lambda mod, inp, o: grabbed.update(act=inp[0]))
    y = mlp(x)
    hook.remove()
    out["mlp.x"] = x.float().numpy()
    out["mlp.gate_up_w"] = torch.cat([mlp.gate_proj.weight, mlp.up_proj.weight], 0).float().detach().numpy()
    out["mlp.down_w"] = mlp.down_proj.weight.float().detach().numpy()
    out["mlp.gate_up"] = torch.cat([mlp.gate_proj(x), mlp.up_proj(x)], 1).float().detach().numpy()
    out["mlp.act"] = grabbed["act"].float().detach().numpy()
    out["mlp.y"] = y.float().detach().numpy()
    np.savez_compressed(OUT / "pi05_rowops.npz", **out)


def policy_fixture(ref):
    """Pre / post-processing of `PyTorchBackend` (openpi/src/openpi/inference/unified_policy.py:179-296): its own
    _normalize_state, _unnormalize_actions and _preprocess, run with a stand-in tokenizer and norm statistics."""
    text = (ref / "openpi" / "src" / "openpi" / "inference" / "unified_policy.py").read_text().splitlines()
    import json, logging
    from abc import ABC, abstractmethod
    from dataclasses import dataclass
    from typing import Any, Dict, List, Optional
    ns = dict(torch=torch, np=np, json=json, logging=logging, ABC=ABC, abstractmethod=abstractmethod, dataclass=dataclass,
              Dict=Dict, List=List, Optional=Optional, Any=Any, Path=Path, logger=logging.getLogger("ref"))
    exec(FUTURE + _between(text, "@dataclass", "class PyTorchPipelinedBackend"), ns)
    # `_preprocess` imports the model's Observation container: give it an attribute bag under that module name
    fake = types.ModuleType("openpi.models_pytorch.pi0_pytorch")
    fake.Observation = lambda **kw: NS(**kw)
    for name in ("openpi", "openpi.models_pytorch"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["openpi.models_pytorch.pi0_pytorch"] = fake

    class Tok:                      # deterministic stand-in for the SentencePiece model: BOS = 2, one id per character
        def Encode(self, prompt, add_bos=True):
            return ([2] if add_bos else []) + [10 + (ord(ch) % 200) for ch in prompt]

    gen = np.random.default_rng(5)
    stats_q = {"state": {"q01": (gen.normal(size=8) - 2).tolist(), "q99": (gen.normal(size=8) + 2).tolist()},
               "actions": {"q01": (gen.normal(size=7) - 1).tolist(), "q99": (gen.normal(size=7) + 1).tolist()}}
    stats_z = {"state": {"mean": gen.normal(size=8).tolist(), "std": (np.abs(gen.normal(size=8)) + 0.1).tolist()},
               "actions": {"mean": gen.normal(size=7).tolist(), "std": (np.abs(gen.normal(size=7)) + 0.1).tolist()}}
    be = ns["PyTorchBackend"].__new__(ns["PyTorchBackend"])
    be.config = ns["PolicyConfig"](checkpoint_dir=".")
    be.device, be.dtype, be.tokenizer = torch.device("cpu"), torch.float32, Tok()
    state = gen.normal(size=8).astype(np.float32)
    actions = gen.normal(size=(50, 32)).astype(np.float32)
    img = gen.integers(0, 256, (224, 224, 3), dtype=np.uint8)
    out = {"state": state, "actions": actions, "image": img,
           "stats_q": np.frombuffer(json.dumps(stats_q).encode(), dtype=np.uint8),
           "stats_z": np.frombuffer(json.dumps(stats_z).encode(), dtype=np.uint8)}
    for tag, st in (("q", stats_q), ("z", stats_z), ("none", None)):
        be.norm_stats = st
        out[f"{tag}.state_norm"] = be._normalize_state(state)
        out[f"{tag}.actions_unnorm"] = be._unnormalize_actions(actions)
    be.norm_stats = stats_q
    long_prompt = "pick up the black bowl and place it on the plate " * 6       # longer than 200 tokens with BOS
    for tag, prompt, wrist in (("short", "pick up the black bowl", img[::-1].copy()), ("long", long_prompt, None)):
        obs = be._preprocess({"observation/image": img, "observation/wrist_image": wrist, "observation/state": state,
                              "prompt": prompt})
        out[f"{tag}.prompt"] = np.frombuffer(prompt.encode(), dtype=np.uint8)
        out[f"{tag}.tokens"] = obs.tokenized_prompt[0].numpy()
        out[f"{tag}.token_mask"] = obs.tokenized_prompt_mask[0].numpy()
        out[f"{tag}.state"] = obs.state[0].numpy()
        out[f"{tag}.base_image"] = obs.images["base_0_rgb"][0].numpy()[:, ::16, ::16].copy()          # subsampled
        out[f"{tag}.wrist_image"] = obs.images["left_wrist_0_rgb"][0].numpy()[:, ::16, ::16].copy()
        out[f"{tag}.image_masks"] = np.array([bool(obs.image_masks[k][0]) for k in ("base_0_rgb", "left_wrist_0_rgb", "right_wrist_0_rgb")])
    np.savez_compressed(OUT / "policy.npz", **out)


def main():
    ref = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["TURBOPI_REFERENCE"])
    torch.set_grad_enabled(False)
    torch.set_num_threads(1)
    G, S, P = load_reference(ref)
    model_fixture(G, S, P)
    rowops_fixture(G)
    policy_fixture(ref)
    for n in ("pi05_model.npz", "pi05_rowops.npz", "policy.npz"):
        print(n, (OUT / n).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
