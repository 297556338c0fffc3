"""Host boundary of the Pi0.5 pipeline: observation dict in, unnormalised actions out.

Mirrors `PyTorchBackend` of the reference (openpi/src/openpi/inference/unified_policy.py:179-324):
quantile (or z-score) normalisation of the robot state and its padding to 32, image handling (uint8
H x W x 3; a missing camera becomes an all -1 image that still counts as present, as there), prompt
tokenisation with BOS, truncation / zero padding to 200 tokens and the padding mask, and the quantile
un-normalisation of the predicted actions.  The observation keys and the result dict are the reference's.

What is B200-specific: the inputs are staged in pinned host buffers allocated once and copied
asynchronously; images stay uint8 until they are on the device (the scaling to [-1, 1] runs there); the
prompt's padding only changes small device buffers (position ids, additive key bias), so every prompt
length replays the same captured graph; nothing is allocated per call.

The reference's third camera (`right_wrist_0_rgb`) is always masked out (unified_policy.py:262-266): its
tokens carry no weight and do not advance the position ids, so the pipeline does not compute it at all.
Pi0.5 does not feed the state to the action expert (`embed_suffix`, pi0_pytorch.py:273-296, pi05 branch);
it is normalised and returned for callers that log it.
"""
import json
from pathlib import Path
from typing import Any, Dict, Optional

import numpy as np
import torch

from ._lib import TurboPiError


def load_norm_stats(checkpoint_dir) -> Optional[dict]:
    """norm_stats.json of a checkpoint (unified_policy.py:157-177), or None (identity) if there is none."""
    root = Path(checkpoint_dir)
    for path in (root / "assets" / "physical-intelligence" / "libero" / "norm_stats.json", root / "norm_stats.json"):
        if path.exists():
            data = json.loads(path.read_text())
            return data.get("norm_stats", data)
    return None


def normalize_state(state: np.ndarray, norm_stats: Optional[dict]) -> np.ndarray:
    """[q01, q99] -> [-1, 1], or z-score when the quantiles are missing (unified_policy.py:179-201)."""
    if norm_stats is None:
        return state
    stats = norm_stats.get("state", {})
    q01, q99 = stats.get("q01"), stats.get("q99")
    if q01 is not None and q99 is not None:
        q01 = np.array(q01, dtype=np.float32)[:len(state)]
        q99 = np.array(q99, dtype=np.float32)[:len(state)]
        return (state - q01) / (q99 - q01 + 1e-6) * 2.0 - 1.0
    mean = np.array(stats.get("mean", [0.0] * len(state)), dtype=np.float32)[:len(state)]
    std = np.clip(np.array(stats.get("std", [1.0] * len(state)), dtype=np.float32)[:len(state)], 1e-6, None)
    return (state - mean) / std


def unnormalize_actions(actions: np.ndarray, norm_stats: Optional[dict]) -> np.ndarray:
    """[-1, 1] -> [q01, q99] on the first len(q01) action dimensions (unified_policy.py:203-232)."""
    if norm_stats is None:
        return actions
    stats = norm_stats.get("actions", {})
    q01, q99 = stats.get("q01"), stats.get("q99")
    out = actions.copy()
    if q01 is not None and q99 is not None:
        q01 = np.array(q01, dtype=np.float32)
        q99 = np.array(q99, dtype=np.float32)
        d = min(actions.shape[-1], len(q01))
        out[..., :d] = (actions[..., :d] + 1.0) / 2.0 * (q99[:d] - q01[:d] + 1e-6) + q01[:d]
        return out
    mean = np.array(stats.get("mean", [0.0] * 7), dtype=np.float32)
    std = np.array(stats.get("std", [1.0] * 7), dtype=np.float32)
    d = min(actions.shape[-1], len(mean))
    out[..., :d] = actions[..., :d] * std[:d] + mean[:d]
    return out


def pad_state(state: np.ndarray, max_state_dim: int = 32) -> np.ndarray:
    out = np.zeros(max_state_dim, dtype=np.float32)
    n = min(len(state), max_state_dim)
    out[:n] = state[:n]
    return out


def tokenize_prompt(prompt, tokenizer, max_token_len: int = 200):
    """(ids [max_token_len] int64 zero-padded, number of real tokens): BOS + pieces, truncated
    (unified_policy.py:284-293).  `prompt` may already be a sequence of ids."""
    if isinstance(prompt, str):
        if tokenizer is None:
            raise TurboPiError("a text prompt needs a tokenizer (a SentencePiece model); pass token ids otherwise")
        ids = list(tokenizer.Encode(prompt, add_bos=True))
    else:
        ids = [int(t) for t in prompt]
    ids = ids[:max_token_len]
    out = np.zeros(max_token_len, dtype=np.int64)
    out[:len(ids)] = ids
    return out, len(ids)


class Pi05Policy:
    """`infer(observation) -> {"actions": [horizon, action_dim] float32}` over a `Pi05` pipeline."""

    def __init__(self, model, norm_stats: Optional[dict] = None, tokenizer=None, num_denoising_steps: int = 3,
                 max_state_dim: int = 32, seed: int = 0):
        self.model, self.cfg = model, model.cfg
        self.norm_stats, self.tokenizer = norm_stats, tokenizer
        self.num_denoising_steps = num_denoising_steps
        self.max_state_dim = max_state_dim
        c = self.cfg
        cuda = torch.device(model.device).type == "cuda"
        pin = (lambda t: t.pin_memory()) if cuda else (lambda t: t)
        self.h_images = pin(torch.zeros((c.num_images, c.image_size, c.image_size, 3), dtype=torch.uint8))
        self.h_tokens = pin(torch.zeros((c.text_len,), dtype=torch.long))
        self.h_noise = pin(torch.zeros((c.action_horizon, c.action_dim), dtype=torch.float32))
        self.h_actions = pin(torch.zeros((c.action_horizon, c.action_dim), dtype=torch.float32))
        self.gen = torch.Generator().manual_seed(seed)

    @classmethod
    def from_checkpoint(cls, checkpoint_dir, device, tokenizer_path=None, **kw):
        """Model weights (`model.tpb` prepared container, else `model.safetensors`), norm stats and the
        SentencePiece tokenizer of a checkpoint directory (unified_policy.py:96-177)."""
        from . import weights
        from .pi05 import Pi05, Pi05Config
        root = Path(checkpoint_dir)
        if (root / "model.tpb").exists():
            model = Pi05.from_file(root / "model.tpb", device)
        else:
            model = Pi05.from_state_dict(weights.load_checkpoint(root / "model.safetensors"), Pi05Config(), device)
        tokenizer = None
        for path in ([Path(tokenizer_path)] if tokenizer_path else []) + [root / "paligemma_tokenizer.model"]:
            if path.exists():
                import sentencepiece as spm
                tokenizer = spm.SentencePieceProcessor()
                tokenizer.Load(str(path))
                break
        return cls(model, load_norm_stats(root), tokenizer, **kw)

    def preprocess(self, observation: Dict[str, Any]) -> Dict[str, Any]:
        """Fills the pinned staging buffers; returns the prompt length and the normalised, padded state."""
        c = self.cfg
        keys = ("observation/image", "observation/wrist_image")
        for i in range(c.num_images):
            img = observation.get(keys[i]) if i < len(keys) else None
            if img is None:
                self.h_images[i].zero_()            # uint8 0 -> -1.0 after scaling: the reference's blank image
            else:
                img = np.asarray(img)
                if img.dtype != np.uint8 or img.shape != (c.image_size, c.image_size, 3):
                    raise TurboPiError(f"{keys[i]}: expected uint8 [{c.image_size}, {c.image_size}, 3], got {img.dtype} {img.shape}")
                self.h_images[i].copy_(torch.from_numpy(img))
        state = observation.get("observation/state")
        if state is not None:
            state = pad_state(normalize_state(np.asarray(state, dtype=np.float32), self.norm_stats), self.max_state_dim)
        else:
            state = np.zeros(self.max_state_dim, dtype=np.float32)
        ids, n = tokenize_prompt(observation.get("prompt", ""), self.tokenizer, c.text_len)
        self.h_tokens.copy_(torch.from_numpy(ids))
        noise = observation.get("noise")
        if noise is None:
            self.h_noise.normal_(generator=self.gen)
        else:
            self.h_noise.copy_(torch.as_tensor(noise, dtype=torch.float32))
        return {"prompt_len": n, "state": state}

    @torch.no_grad()
    def infer(self, observation: Dict[str, Any], num_steps: Optional[int] = None) -> Dict[str, np.ndarray]:
        steps = self.num_denoising_steps if num_steps is None else num_steps
        pre = self.preprocess(observation)
        # both cameras count as present even when blank, as in the reference (unified_policy.py:262-266)
        actions = self.model.infer(self.h_images, self.h_tokens, self.h_noise, num_steps=steps,
                                   image_valid=[True] * self.cfg.num_images, prompt_len=max(pre["prompt_len"], 1))
        self.h_actions.copy_(actions, non_blocking=True)
        if actions.is_cuda:
            torch.cuda.current_stream(actions.device).synchronize()
        return {"actions": unnormalize_actions(self.h_actions.numpy().copy(), self.norm_stats), "state": pre["state"]}

    def warmup(self, num_iterations: int = 5):
        c = self.cfg
        rng = np.random.default_rng(0)
        obs = {"observation/image": rng.integers(0, 255, (c.image_size, c.image_size, 3), dtype=np.uint8),
               "observation/wrist_image": rng.integers(0, 255, (c.image_size, c.image_size, 3), dtype=np.uint8),
               "observation/state": np.zeros(8, dtype=np.float32), "prompt": [2, 5, 7]}
        for _ in range(num_iterations):
            self.infer(obs)
