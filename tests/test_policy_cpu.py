"""Host pre / post-processing (turbopi_b200/policy.py) against what the reference's own `PyTorchBackend`
methods produced (tests/golden/policy.npz, made by tests/golden/make_golden_model.py from
openpi/src/openpi/inference/unified_policy.py:179-296)."""
import json

import numpy as np
import pytest
import torch

from turbopi_b200 import policy
from turbopi_b200.pi05 import Pi05, Pi05Config


class Tok:                      # the stand-in tokenizer of the fixture: BOS = 2, one id per character
    def Encode(self, prompt, add_bos=True):
        return ([2] if add_bos else []) + [10 + (ord(ch) % 200) for ch in prompt]


@pytest.fixture(scope="module")
def g(golden):
    return golden("policy")


def _stats(g, tag):
    return None if tag == "none" else json.loads(bytes(g[f"stats_{tag}"]).decode())


@pytest.mark.parametrize("tag", ["q", "z", "none"])
def test_state_and_action_normalisation_match_reference(g, tag):
    st = _stats(g, tag)
    assert np.array_equal(policy.normalize_state(g["state"], st), g[f"{tag}.state_norm"])
    assert np.array_equal(policy.unnormalize_actions(g["actions"], st), g[f"{tag}.actions_unnorm"])


@pytest.mark.parametrize("tag", ["short", "long"])
def test_prompt_padding_state_padding_and_masks_match_reference(g, tag):
    prompt = bytes(g[f"{tag}.prompt"]).decode()
    ids, n = policy.tokenize_prompt(prompt, Tok(), 200)
    assert np.array_equal(ids, g[f"{tag}.tokens"])
    assert np.array_equal(np.arange(200) < n, g[f"{tag}.token_mask"])
    assert (n == 200) == (tag == "long")
    state = policy.pad_state(policy.normalize_state(g["state"], _stats(g, "q")), 32)
    assert np.array_equal(state, g[f"{tag}.state"])
    # the two real cameras count as present even when the wrist image is missing (all -1), the third never does
    assert g[f"{tag}.image_masks"].tolist() == [True, True, False]
    assert np.array_equal(ids, policy.tokenize_prompt(ids[:n].tolist(), None, 200)[0])   # ids pass through


def test_policy_stages_an_observation_like_the_reference(g):
    """Pi05Policy.preprocess on a (CPU-resident, never launched) pipeline: staged uint8 images scale to the
    reference's float images, a missing wrist camera becomes the reference's all -1 image."""
    cfg = Pi05Config(vision_layers=1, vision_width=64, vision_mlp=112, vision_heads=2, prefix_layers=1, width=128, mlp=256,
                     vocab=256, expert_layers=1, expert_width=64, expert_mlp=128)
    pol = policy.Pi05Policy(Pi05(cfg, "cpu", seed=0), _stats(g, "q"), Tok())
    for tag, wrist in (("short", g["image"][::-1].copy()), ("long", None)):
        pre = pol.preprocess({"observation/image": g["image"], "observation/wrist_image": wrist,
                              "observation/state": g["state"], "prompt": bytes(g[f"{tag}.prompt"]).decode()})
        assert pre["prompt_len"] == int(g[f"{tag}.token_mask"].sum())
        assert np.array_equal(pre["state"], g[f"{tag}.state"])
        assert np.array_equal(pol.h_tokens.numpy(), g[f"{tag}.tokens"])
        scaled = pol.h_images.float() / 127.5 - 1.0                   # what the pipeline does on the device
        for i, key in enumerate(("base_image", "wrist_image")):
            ours = scaled[i].permute(2, 0, 1)[:, ::16, ::16].numpy()
            assert np.allclose(ours, g[f"{tag}.{key}"], atol=1e-6)
    with pytest.raises(policy.TurboPiError):
        pol.preprocess({"observation/image": g["image"][:100], "prompt": [2, 3]})
    with pytest.raises(policy.TurboPiError):
        policy.Pi05Policy(Pi05(cfg, "cpu", seed=0)).preprocess({"observation/image": g["image"], "prompt": "text, no tokenizer"})
