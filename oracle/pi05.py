"""CPU oracle of the Pi0.5-shaped inference: torch fp32 arithmetic, optionally with the bf16 roundings of
the reference's bf16 model.  Test infrastructure; see oracle/__init__.py.

Follows `PI0Pytorch.sample_actions` (openpi/src/openpi/models_pytorch/pi0_pytorch.py:876-937):
embed_prefix (:215-264), compute_prefix_kv_cache (:406-522), the graph-safe denoise step
denoise_step_graphed (:656-768) with the tensors of precompute_graph_tensors (:770-874), embed_suffix
(:266-345), make_att_2d_masks (:80-108); GemmaRMSNorm / adaptive RMSNorm / _gated_residual / GemmaMLP
(transformers_replace/models/gemma/modeling_gemma.py:49-129,212-230); RoPE (:132-197);
SigLIP embeddings / encoder layer (transformers_replace/models/siglip/modeling_siglip.py:212-283,348-482).

Pinned: tests/test_oracle_golden.py runs this file in exact-fp32 mode on the weights of
tests/golden/pi05_model.npz, which tests/golden/make_golden_model.py produced by executing those reference
classes and methods themselves (padded prompt and missing-camera cases included).

Padding.  `valid` marks the prefix tokens that exist (image tokens of a present camera, prompt tokens
before the padding).  As in the reference, position ids are `cumsum(valid) - 1`, the action tokens
continue at `sum(valid)`, and nobody attends to an invalid key.  Rows of invalid QUERY tokens are
computed like any other (they differ from the reference's, which softmaxes a fully masked row; no valid
token ever reads them).  `PI0Pytorch.denoise_step_with_cache` (:619-621) drops the mask altogether and
lets action tokens attend to padded keys; the oracle follows the masked `denoise_step_graphed`.

Weights are plain float32 matrices (already dequantised) in a dict; see tests/test_pi05_gpu.py.
Every tensor follows the device of the weights, so the full-depth comparison can execute this same code
with fp32 torch kernels on the GPU (checked against its CPU execution at reduced depth).
"""
import contextlib
import math

import torch
import torch.nn.functional as F

_ROUND = True
MASKED = -2.3819763e38            # the reference's additive mask value (pi0_pytorch.py:185-188)


@contextlib.contextmanager
def exact_fp32():
    """Inside this context no bf16 rounding is applied: the oracle then computes what the reference's
    modules compute when they hold fp32 weights."""
    global _ROUND
    prev, _ROUND = _ROUND, False
    try:
        yield
    finally:
        _ROUND = prev


def r(x):
    """round to bf16, keep float32 storage"""
    return x.to(torch.bfloat16).float() if _ROUND else x


def linear(x, w, b=None, act=None, out_fp32=False):
    y = r(x) @ w.t()
    if b is not None:
        y = y + b
    if act == "gelu":
        y = F.gelu(y, approximate="tanh")
    elif act == "silu":
        y = F.silu(y)
    return y if out_fp32 else r(y)


def rms(x, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rope(x, cos, sin):
    """x [L, H, D]; cos, sin [L, D/2] (bf16 values); bf16 product-by-product as torch does."""
    h = x.shape[-1] // 2
    c = torch.cat([cos, cos], -1)[:, None, :]
    s = torch.cat([sin, sin], -1)[:, None, :]
    rot = torch.cat([-x[..., h:], x[..., :h]], -1)
    return r(r(x * c) + r(rot * s))


def rope_tables(positions, head_dim, theta=10000.0, bf16=True):
    """cos / sin [len(positions), head_dim / 2] (GemmaRotaryEmbedding.forward; the bf16 model holds
    inv_freq in bf16, openpi/src/openpi/inference/w4a16_tvm_kv_cache.py:144-146)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    if bf16:
        inv = inv.to(torch.bfloat16).float()
    f = positions.float()[:, None] * inv[None, :]
    c, s = f.cos(), f.sin()
    return (c.to(torch.bfloat16).float(), s.to(torch.bfloat16).float()) if bf16 else (c, s)


def attention(q, k, v, heads, key_valid=None):
    """q [L, H*D], k/v [S, D] (one KV head); keys with key_valid False are masked out."""
    L, D = q.shape[0], k.shape[1]
    qh = q.view(L, heads, D).transpose(0, 1)
    mask = None
    if key_valid is not None:
        mask = torch.where(key_valid.to(q.device), 0.0, MASKED)[None, None, None, :].to(q.dtype)
    o = F.scaled_dot_product_attention(qh[None], k[None, None].expand(1, heads, -1, -1),
                                       v[None, None].expand(1, heads, -1, -1), attn_mask=mask)
    return r(o[0].transpose(0, 1).reshape(L, heads * D))


def vision_tower(w, images_u8, cfg):
    n = cfg["image_size"] // cfg["patch"]
    NI, vw = images_u8.shape[0], cfg["vision_width"]
    img = images_u8.float() / 127.5 - 1.0
    pt = img.view(NI, n, cfg["patch"], n, cfg["patch"], 3).permute(0, 1, 3, 5, 2, 4).reshape(NI * n * n, -1)
    pk = pt.shape[1]
    h = linear(pt, w["patch_embed"][:, :pk], w["patch_embed_b"])
    h = r(h.view(NI, n * n, vw) + w["pos_emb"]).view(-1, vw)
    heads = cfg["vision_heads"]
    hd = vw // heads
    for L in w["vision"]:
        x = r(F.layer_norm(h, (vw,), L["ln1_w"], L["ln1_b"], cfg["eps"]))
        qkv = linear(x, L["qkv"], L["qkv_b"]).view(NI, n * n, 3, heads, hd).permute(2, 0, 3, 1, 4)
        o = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])
        o = r(o.transpose(1, 2).reshape(-1, vw))
        h = r(h + linear(o, L["out"], L["out_b"]))
        x = r(F.layer_norm(h, (vw,), L["ln2_w"], L["ln2_b"], cfg["eps"]))
        h = r(h + linear(linear(x, L["fc1"], L["fc1_b"], "gelu"), L["fc2"], L["fc2_b"]))
    x = r(F.layer_norm(h, (vw,), w["post_ln_w"], w["post_ln_b"], cfg["eps"]))
    return linear(x, w["projector"], w["projector_b"])


def prefix_positions(valid):
    """position ids of the prefix tokens and the first position of the action tokens
    (pi0_pytorch.py:442 and :791-796)."""
    pos = torch.cumsum(valid.long(), 0) - 1
    return pos.clamp_min(0), int(valid.long().sum())


def prefix_pass(w, img_tokens, tokens, cfg, cos, sin, valid=None):
    """Returns the per-layer (K post-RoPE, V) rows, each [S, head_dim].  cos / sin are tables indexed by
    POSITION; token i uses row `cumsum(valid)[i] - 1`."""
    width, qd, hd = cfg["width"], cfg["q_dim"], cfg["head_dim"]
    h = torch.cat([img_tokens, r(w["embed_tokens"][tokens] * math.sqrt(width))], 0)
    S = h.shape[0]
    if valid is None:
        valid = torch.ones(S, dtype=torch.bool)
    valid = valid.to(h.device)
    pos, _ = prefix_positions(valid)
    pc, ps = cos[pos], sin[pos]
    kv = []
    for L in w["prefix"]:
        x = r(rms(h, cfg["eps"]) * (1.0 + L["in_norm"]))
        qkv = linear(x, L["qkv"])
        q = rope(qkv[:, :qd].view(S, -1, hd), pc, ps).reshape(S, qd)
        k = rope(qkv[:, qd:qd + hd].view(S, 1, hd), pc, ps).reshape(S, hd)
        v = qkv[:, qd + hd:]
        kv.append((k, v))
        h = r(h + linear(attention(q, k, v, cfg["heads"], valid), L["o"]))
        x = r(rms(h, cfg["eps"]) * (1.0 + L["post_norm"]))
        gu = linear(x, L["gate_up"])
        I = gu.shape[1] // 2
        act = r(r(F.gelu(gu[:, :I], approximate="tanh")) * gu[:, I:])
        h = r(h + linear(act, L["down"]))
    return kv


def sinusoidal(t, dim, min_period=4e-3, max_period=4.0):
    frac = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float64)
    period = min_period * (max_period / min_period) ** frac
    ang = (1.0 / period * 2 * math.pi)[None, :] * t.to(torch.float64)[:, None]
    return torch.cat([torch.sin(ang), torch.cos(ang)], 1)


def adarms_cond(w, t, ew):
    """silu(time_mlp_out(silu(time_mlp_in(sincos(t))))) (pi0_pytorch.py:817-839)."""
    emb = r(sinusoidal(t.cpu(), ew).float()).to(w["time_mlp_in"].device)
    return linear(linear(emb, w["time_mlp_in"], w["time_mlp_in_b"], "silu"), w["time_mlp_out"], w["time_mlp_out_b"], "silu")


def denoise_velocity(w, kv, x_t, cond, cfg, cos, sin, valid=None):
    """One evaluation of the action expert: v_t [A, action_dim] (fp32)."""
    ew, qd, hd, A = cfg["expert_width"], cfg["q_dim"], cfg["head_dim"], x_t.shape[0]
    S = kv[0][0].shape[0]
    if valid is None:
        valid = torch.ones(S, dtype=torch.bool)
    valid = valid.to(x_t.device)
    _, first = prefix_positions(valid)
    pos_c, pos_s = cos[first:first + A], sin[first:first + A]
    key_valid = torch.cat([valid, torch.ones(A, dtype=torch.bool, device=valid.device)])
    mod = linear(cond, w["ada_dense"], w["ada_dense_b"]).view(-1, 3, ew)       # [n_norms, (scale, shift, gate), ew]
    h = linear(r(x_t), w["action_in"], w["action_in_b"])
    for l, L in enumerate(w["expert"]):
        m_in, m_post = mod[2 * l], mod[2 * l + 1]
        x = r(rms(h, cfg["eps"]) * (1.0 + m_in[0]) + m_in[1])
        qkv = linear(x, L["qkv"])
        q = rope(qkv[:, :qd].view(A, -1, hd), pos_c, pos_s).reshape(A, qd)
        k = rope(qkv[:, qd:qd + hd].view(A, 1, hd), pos_c, pos_s).reshape(A, hd)
        v = qkv[:, qd + hd:]
        kf, vf = torch.cat([kv[l][0], k], 0), torch.cat([kv[l][1], v], 0)
        o = linear(attention(q, kf, vf, cfg["heads"], key_valid), L["o"])
        h = r(h + r(o * m_in[2]))
        x = r(rms(h, cfg["eps"]) * (1.0 + m_post[0]) + m_post[1])
        gu = linear(x, L["gate_up"])
        I = gu.shape[1] // 2
        act = r(r(F.gelu(gu[:, :I], approximate="tanh")) * gu[:, I:])
        h = r(h + r(linear(act, L["down"]) * m_post[2]))
    m_f = mod[2 * len(w["expert"])]
    x = r(rms(h, cfg["eps"]) * (1.0 + m_f[0]) + m_f[1])
    return linear(x, w["action_out"], w["action_out_b"], out_fp32=True)


def denoise(w, kv, noise, num_steps, cfg, cos, sin, valid=None):
    ew = cfg["expert_width"]
    dt = -1.0 / num_steps
    x_t = noise.clone().float()
    for i in range(num_steps):
        t = torch.tensor([1.0 + i * dt], dtype=torch.float32)
        v_t = denoise_velocity(w, kv, x_t, adarms_cond(w, t, ew), cfg, cos, sin, valid)
        x_t = x_t + dt * v_t
    return x_t


def prefix_valid(cfg, image_valid=None, prompt_len=None):
    """bool [S]: image tokens of the present cameras, then the first `prompt_len` prompt tokens."""
    n = (cfg["image_size"] // cfg["patch"]) ** 2
    NI = cfg.get("num_images", 2)
    image_valid = [True] * NI if image_valid is None else list(image_valid)
    text_len = cfg["text_len"]
    prompt_len = text_len if prompt_len is None else int(prompt_len)
    parts = [torch.full((n,), bool(v)) for v in image_valid] + [torch.arange(text_len) < prompt_len]
    return torch.cat(parts)


def sample_actions(w, images_u8, tokens, noise, num_steps, cfg, cos, sin, valid=None):
    img_tokens = vision_tower(w, images_u8, cfg)
    kv = prefix_pass(w, img_tokens, tokens, cfg, cos, sin, valid)
    return denoise(w, kv, noise, num_steps, cfg, cos, sin, valid), kv
