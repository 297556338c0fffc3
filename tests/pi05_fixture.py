"""Helpers shared by the CPU and GPU tests: the reference-generated model fixture
(tests/golden/pi05_model.npz, see tests/golden/make_golden_model.py) as the oracle's weight dict."""
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_model_fixture():
    g = dict(np.load(GOLDEN / "pi05_model.npz"))
    cfg = {str(k): int(v) for k, v in zip(g["cfg_keys"], g["cfg_vals"])}
    return g, cfg


def oracle_weights(g, cfg):
    """Weight dict in the naming of oracle/pi05.py from the flat arrays of the fixture."""
    t = lambda k: torch.from_numpy(np.asarray(g[k], dtype=np.float32))
    w = {"patch_embed": t("v.patch_w"), "patch_embed_b": t("v.patch_b"), "pos_emb": t("v.pos_emb"), "vision": []}
    for i in range(cfg["vision_layers"]):
        w["vision"].append({k: t(f"v.{i}.{k}") for k in ("ln1_w", "ln1_b", "ln2_w", "ln2_b", "qkv", "qkv_b", "out", "out_b",
                                                        "fc1", "fc1_b", "fc2", "fc2_b")})
    w["post_ln_w"], w["post_ln_b"] = t("v.post_ln_w"), t("v.post_ln_b")
    w["projector"], w["projector_b"] = t("projector"), t("projector_b")
    w["embed_tokens"] = t("embed_tokens")
    w["prefix"] = [{k: t(f"p.{i}.{k}") for k in ("in_norm", "post_norm", "qkv", "o", "gate_up", "down")}
                   for i in range(cfg["prefix_layers"])]
    w["expert"] = [{k: t(f"e.{i}.{k}") for k in ("qkv", "o", "gate_up", "down")} for i in range(cfg["expert_layers"])]
    dense, dense_b = [], []
    for i in range(cfg["expert_layers"]):            # every adaptive norm's dense(cond), stacked in model order
        dense += [t(f"e.{i}.in_dense"), t(f"e.{i}.post_dense")]
        dense_b += [t(f"e.{i}.in_dense_b"), t(f"e.{i}.post_dense_b")]
    w["ada_dense"] = torch.cat(dense + [t("e.norm_dense")], 0)
    w["ada_dense_b"] = torch.cat(dense_b + [t("e.norm_dense_b")], 0)
    for ours, theirs in (("action_in", "action_in_proj"), ("action_out", "action_out_proj"),
                         ("time_mlp_in", "time_mlp_in"), ("time_mlp_out", "time_mlp_out")):
        w[ours], w[ours + "_b"] = t(theirs), t(theirs + "_b")
    return w


def oracle_cfg(cfg):
    return dict(image_size=cfg["image_size"], patch=cfg["patch"], vision_width=cfg["vision_width"],
                vision_heads=cfg["vision_heads"], eps=1e-6, width=cfg["width"], q_dim=cfg["heads"] * cfg["head_dim"],
                head_dim=cfg["head_dim"], heads=cfg["heads"], expert_width=cfg["expert_width"], text_len=cfg["text_len"],
                num_images=2)
