"""End-to-end parity of the Pi0.5-shaped pipeline with the CPU oracle on a reduced model
(full head geometry, fewer / narrower layers so the fp32 CPU oracle finishes in seconds)."""
import numpy as np
import pytest
import torch

from conftest import cosine, rel_err
from oracle import nvfp4 as onv
from oracle import pi05 as opi

pytestmark = pytest.mark.gpu


def _deq(lin):
    packed, scales, g = lin.raw
    w = onv.dequantize(packed.cpu().numpy(), scales.cpu().numpy(), 16, float(g), scale_is_e4m3=True)
    return torch.from_numpy(w), (None if lin.bias is None else lin.bias.float().cpu())


def _extract(model):
    """Plain float32 weights of the quantised model, in the oracle's naming."""
    f = lambda t: t.float().cpu()
    w = {}
    w["patch_embed"], w["patch_embed_b"] = _deq(model.patch_embed)
    w["pos_emb"] = f(model.pos_emb)
    w["vision"] = []
    for L in model.vision:
        d = {k: f(L[k]) for k in ("ln1_w", "ln1_b", "ln2_w", "ln2_b")}
        for k in ("qkv", "out", "fc1", "fc2"):
            d[k], d[k + "_b"] = _deq(L[k])
        w["vision"].append(d)
    w["post_ln_w"], w["post_ln_b"] = f(model.post_ln_w), f(model.post_ln_b)
    w["projector"], w["projector_b"] = _deq(model.projector)
    w["embed_tokens"] = f(model.embed_tokens)
    w["prefix"] = [dict(in_norm=f(L["in_norm"]), post_norm=f(L["post_norm"]), qkv=_deq(L["qkv"])[0], o=_deq(L["o"])[0],
                        gate_up=_deq(L["gate_up"])[0], down=_deq(L["down"])[0]) for L in model.prefix]
    for k in ("action_in", "action_out", "time_mlp_in", "time_mlp_out", "ada_dense"):
        w[k], w[k + "_b"] = _deq(getattr(model, k))
    w["expert"] = [dict(qkv=_deq(L["qkv"])[0], o=_deq(L["o"])[0], gate_up=_deq(L["gate_up"])[0], down=_deq(L["down"])[0])
                   for L in model.expert]
    return w


@torch.no_grad()
@pytest.mark.parametrize("steps", [1, 3])
def test_reduced_pi05_matches_oracle(cuda_device, steps):
    from turbopi_b200 import _lib
    from turbopi_b200.pi05 import Pi05, Pi05Config
    cfg = Pi05Config(image_size=56, patch=14, vision_layers=2, vision_width=128, vision_mlp=272, vision_heads=2,
                     prefix_layers=2, width=256, mlp=512, text_len=24, vocab=1000, expert_layers=2, expert_width=128,
                     expert_mlp=256, action_horizon=50, action_dim=32, max_seq=256)
    model = Pi05(cfg, cuda_device, seed=1, keep_raw=True)
    g = torch.Generator().manual_seed(2)
    images = torch.randint(0, 256, (2, 56, 56, 3), generator=g, dtype=torch.uint8)
    tokens = torch.randint(0, 1000, (24,), generator=g)
    noise = torch.randn(50, 32, generator=g)
    eager = model.infer(images, tokens, noise, num_steps=steps, use_graph=False).cpu().clone()
    graphed = model.infer(images, tokens, noise, num_steps=steps, use_graph=True).cpu().clone()
    replay = model.infer(images, tokens, noise, num_steps=steps, use_graph=True).cpu().clone()
    assert _lib.load().tpb200_device_error(0) == 0
    assert torch.equal(graphed, replay)                       # a replay is deterministic
    assert (eager - graphed).abs().max() < 1e-3               # graph == eager up to atomics-free reordering (none)

    w = _extract(model)
    ocfg = dict(image_size=56, patch=14, vision_width=128, vision_heads=2, eps=cfg.eps, width=256, q_dim=cfg.q_dim,
                head_dim=256, heads=8, expert_width=128)
    cos, sin = model.cos.float().cpu(), model.sin.float().cpu()
    ref, kv = opi.sample_actions(w, images, tokens, noise, steps, ocfg, cos, sin)
    S = cfg.prefix_len
    cache = model.cache.float().cpu()
    for l in range(cfg.prefix_layers):
        assert rel_err(cache[l, 0, :S].numpy(), kv[l][0].numpy()) <= 2e-2, ("K", l)
        assert rel_err(cache[l, 1, :S].numpy(), kv[l][1].numpy()) <= 2e-2, ("V", l)
    assert (cache[:, :, S + 50:] == 0).all()                  # rows past prefix + suffix never written
    err = (graphed - ref).abs().max().item()
    assert err <= 2e-2, err                                   # end-to-end actions within 2e-2 absolute
    assert cosine(graphed.numpy(), ref.numpy()) >= 0.999
