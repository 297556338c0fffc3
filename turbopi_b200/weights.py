"""Offline weight pipeline: checkpoint tensors -> packed 4-bit weights -> files -> device buffers.

Two layers:

1. The reference's interchange formats, same function names and file layouts as
   openpi/nvfp4_packed_plugin/scripts/prepare_weights.py:134-296 (`prepare_linear_weights`,
   `process_model_weights`, `save_packed_weights` with formats npz / safetensors / bin, plus the
   matching `load_packed_weights`): packed e2m1 codes [N, K/2] + fp32 block-32 scales, one entry per
   2-D `weight` of a state dict.  Files written here load in the reference and vice versa.

2. The B200 container (`save_container` / `load_container`): named blobs behind a versioned header,
   each blob 256-byte aligned so it can be copied straight into a device buffer.  `Pi05.save()` /
   `Pi05.from_file()` store the prepared model in it: per linear the tiled 36 KB-block operand image
   that the tensor-core GEMM and the decode GEMV stream (codes + UE4M3 scales, standard NVFP4 with an
   fp32 global scale), bf16 norm / embedding tables, fp32 biases.

`tile_weights_host` builds that tiled image with plain tensor indexing, so a checkpoint can be prepared
on a machine without a GPU; it is byte-identical to the CUDA tiler (tested).  `reference_state_dict_names`
lists the tensors a Pi0.5 checkpoint holds under the reference's module names.
"""
import json
import struct
from pathlib import Path
from typing import Dict, Optional

import numpy as np
import torch

from .nvfp4_packed import BLOCK_SIZE, pack_nvfp4, quantize_nvfp4_two_level, quantize_to_nvfp4, unpack_nvfp4

# ------------------------------------------------------------------------------------------------
# 1. reference interchange formats
# ------------------------------------------------------------------------------------------------


def prepare_linear_weights(weight: torch.Tensor, block_size: int = BLOCK_SIZE, verify: bool = True) -> Dict:
    """[N, K] -> {'weight_packed' [N, K/2] uint8, 'weight_scales' [N, K/block] fp32, 'out_features',
    'in_features'}; K is zero-padded to a multiple of the block (prepare_weights.py:134-183)."""
    N, K = weight.shape
    if K % block_size != 0:
        weight = torch.nn.functional.pad(weight, (0, block_size - K % block_size))
        K = weight.shape[1]
    quantized, scales = quantize_to_nvfp4(weight, block_size)
    packed = pack_nvfp4(quantized)
    if verify:
        diff = (quantized - unpack_nvfp4(packed, N, K)).abs().max().item()
        if diff >= 1e-6:
            raise ValueError(f"pack/unpack mismatch: {diff}")
    return {"weight_packed": packed.cpu(), "weight_scales": scales.cpu().float(), "out_features": N, "in_features": K}


def process_model_weights(state_dict: Dict[str, torch.Tensor], layer_patterns: Optional[list] = None,
                          block_size: int = BLOCK_SIZE, device: str = "cpu") -> Dict[str, Dict]:
    """Every 2-D tensor whose name contains 'weight' (and one of `layer_patterns`, when given) is
    quantised and packed (prepare_weights.py:186-231).  Unlike the reference, a failing layer raises."""
    processed = {}
    for name, param in state_dict.items():
        if "weight" not in name or param.dim() != 2:
            continue
        if layer_patterns and not any(p in name for p in layer_patterns):
            continue
        processed[name] = prepare_linear_weights(param.to(device), block_size)
    return processed


def save_packed_weights(processed: Dict[str, Dict], output_path, format: str = "npz") -> Path:
    """npz: `<name with . -> _>_packed / _scales / _shape`; safetensors: `_packed / _scales`; bin:
    u32 count, then per layer u32 name length, name, u32 N, u32 K, u32 bytes, codes, u32 bytes, scales
    (prepare_weights.py:234-296)."""
    output_path = Path(output_path)
    output_path.parent.mkdir(parents=True, exist_ok=True)
    if format == "npz":
        arrays = {}
        for name, d in processed.items():
            safe = name.replace(".", "_")
            arrays[f"{safe}_packed"] = d["weight_packed"].numpy()
            arrays[f"{safe}_scales"] = d["weight_scales"].numpy()
            arrays[f"{safe}_shape"] = np.array([d["out_features"], d["in_features"]])
        np.savez_compressed(output_path, **arrays)
    elif format == "safetensors":
        from safetensors.torch import save_file
        tensors = {}
        for name, d in processed.items():
            safe = name.replace(".", "_")
            tensors[f"{safe}_packed"] = d["weight_packed"].contiguous()
            tensors[f"{safe}_scales"] = d["weight_scales"].contiguous()
        save_file(tensors, str(output_path))
    elif format == "bin":
        with open(output_path, "wb") as f:
            f.write(struct.pack("I", len(processed)))
            for name, d in processed.items():
                nb = name.encode("utf-8")
                f.write(struct.pack("I", len(nb)))
                f.write(nb)
                f.write(struct.pack("II", d["out_features"], d["in_features"]))
                for t in (d["weight_packed"], d["weight_scales"]):
                    raw = t.contiguous().numpy().tobytes()
                    f.write(struct.pack("I", len(raw)))
                    f.write(raw)
    else:
        raise ValueError(f"unknown format {format!r}")
    return output_path


def load_packed_weights(path, format: Optional[str] = None) -> Dict[str, Dict]:
    """Inverse of save_packed_weights.  npz / safetensors entries come back under their flattened names
    (dots are not recoverable from those two formats); safetensors files carry no shape entry, so the
    shape is taken from the code tensor."""
    path = Path(path)
    format = format or path.suffix.lstrip(".")
    out: Dict[str, Dict] = {}
    if format == "npz":
        z = np.load(path)
        for key in z.files:
            if key.endswith("_packed"):
                base = key[:-len("_packed")]
                N, K = (int(v) for v in z[base + "_shape"])
                out[base] = {"weight_packed": torch.from_numpy(z[key]), "weight_scales": torch.from_numpy(z[base + "_scales"]),
                             "out_features": N, "in_features": K}
    elif format == "safetensors":
        from safetensors.torch import load_file
        t = load_file(str(path))
        for key, packed in t.items():
            if key.endswith("_packed"):
                base = key[:-len("_packed")]
                out[base] = {"weight_packed": packed, "weight_scales": t[base + "_scales"],
                             "out_features": packed.shape[0], "in_features": packed.shape[1] * 2}
    elif format == "bin":
        raw = path.read_bytes()
        pos = 0

        def u32():
            nonlocal pos
            v = struct.unpack_from("I", raw, pos)[0]
            pos += 4
            return v

        for _ in range(u32()):
            n = u32()
            name = raw[pos:pos + n].decode("utf-8")
            pos += n
            N, K = u32(), u32()
            nb = u32()
            packed = np.frombuffer(raw, dtype=np.uint8, count=nb, offset=pos).reshape(N, K // 2).copy()
            pos += nb
            nb = u32()
            scales = np.frombuffer(raw, dtype=np.float32, count=nb // 4, offset=pos).reshape(N, -1).copy()
            pos += nb
            out[name] = {"weight_packed": torch.from_numpy(packed), "weight_scales": torch.from_numpy(scales),
                         "out_features": N, "in_features": K}
    else:
        raise ValueError(f"unknown format {format!r}")
    return out


# ------------------------------------------------------------------------------------------------
# 2. tiled operand images and the container
# ------------------------------------------------------------------------------------------------
K_STAGE = 256                  # K elements per block
BLOCK_ROWS = 256
CODE_BYTES = BLOCK_ROWS * 128  # 32 KB of codes
SLAB_BYTES = 2048              # scales of 128 rows x 16 K-blocks
BLOCK_BYTES = CODE_BYTES + 2 * SLAB_BYTES


def swizzle_scales_host(sf_bytes: torch.Tensor) -> torch.Tensor:
    """UE4M3 scale bytes [rows, K/16] -> 512-byte atoms of 128 rows x 4 K-blocks, ordered [row tile][K atom],
    byte (r % 32) * 16 + (r // 32) * 4 + kb inside an atom; rows padded to 128, K-blocks to 16."""
    R, KB = sf_bytes.shape
    Rp, Kp = (R + 127) // 128 * 128, (KB + 15) // 16 * 16
    pad = torch.zeros((Rp, Kp), dtype=torch.uint8, device=sf_bytes.device)
    pad[:R, :KB] = sf_bytes
    return pad.reshape(Rp // 128, 4, 32, Kp // 4, 4).permute(0, 3, 2, 1, 4).contiguous().reshape(-1)


def tile_weights_host(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """codes [N, K/2] uint8 + UE4M3 scale bytes [N, K/16] -> the tiled B image (flat uint8):
    blocks [ceil(N/256)][ceil(K/256)] of 36 KB = 256 rows x 128 B of codes with the 16-byte chunk c of
    row r stored at c ^ (r & 7), then the 2 KB scale slabs of rows [0,128) and [128,256).  Padding rows
    and padding K are zero codes with zero scales."""
    N, Kh = packed.shape
    nb, ks = (N + BLOCK_ROWS - 1) // BLOCK_ROWS, (Kh * 2 + K_STAGE - 1) // K_STAGE
    dev = packed.device
    codes = torch.zeros((nb * BLOCK_ROWS, ks * 128), dtype=torch.uint8, device=dev)
    codes[:N, :Kh] = packed
    codes = codes.reshape(nb, BLOCK_ROWS, ks, 8, 16).permute(0, 2, 1, 3, 4)         # [nb, ks, r, chunk, 16]
    r = torch.arange(BLOCK_ROWS, device=dev)[:, None]
    slot = torch.arange(8, device=dev)[None, :]
    src = (slot ^ (r & 7))[None, None, :, :, None].expand(nb, ks, BLOCK_ROWS, 8, 16)
    codes = torch.gather(codes, 3, src).reshape(nb, ks, CODE_BYTES)
    sf = swizzle_scales_host(scales.reshape(N, -1))
    row_tiles = sf.numel() // (ks * SLAB_BYTES)
    slabs = torch.zeros((2 * nb, ks, SLAB_BYTES), dtype=torch.uint8, device=dev)
    slabs[:row_tiles] = sf.reshape(row_tiles, ks, SLAB_BYTES)
    slabs = slabs.reshape(nb, 2, ks, SLAB_BYTES).permute(0, 2, 1, 3).reshape(nb, ks, 2 * SLAB_BYTES)
    return torch.cat([codes, slabs], dim=2).contiguous().reshape(-1)


def prepare_tiled_linear(weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                         row_perm: Optional[torch.Tensor] = None) -> Dict:
    """[N, K] float weight -> standard NVFP4 (E4M3 scale per 16 + fp32 global scale) in the tiled image.
    Runs on whatever device `weight` lives on (CPU included)."""
    N, K = weight.shape
    if K % 16:
        raise ValueError("K must be a multiple of 16")
    packed, scales, g = quantize_nvfp4_two_level(weight, 16)
    if row_perm is not None:
        packed, scales = packed[row_perm], scales[row_perm]
    return {"image": tile_weights_host(packed, scales), "global_scale": float(g), "N": N, "K": K,
            "bias": None if bias is None else bias.detach().float().contiguous()}


MAGIC = b"TPB200W\0"
CONTAINER_VERSION = 1
_NP = {"uint8": np.uint8, "float32": np.float32, "int32": np.int32, "int64": np.int64, "bfloat16": np.uint16,
       "float16": np.float16}


def save_container(path, tensors: Dict[str, torch.Tensor], meta: Optional[dict] = None) -> Path:
    """magic(8) | u32 version | u32 reserved | u64 header bytes | JSON header | blobs.
    JSON: {"meta": ..., "tensors": {name: {"dtype", "shape", "offset", "nbytes"}}}; every blob starts on a
    256-byte boundary of the file."""
    path = Path(path)
    index, offset = {}, 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        dt = str(t.dtype).replace("torch.", "")
        if dt not in _NP:
            raise ValueError(f"{name}: dtype {dt} is not storable")
        raw = (t.view(torch.uint16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        index[name] = {"dtype": dt, "shape": list(t.shape), "offset": offset, "nbytes": len(raw)}
        blobs.append(raw)
        offset += (len(raw) + 255) // 256 * 256
    header = json.dumps({"meta": meta or {}, "tensors": index}).encode("utf-8")
    base = (24 + len(header) + 255) // 256 * 256
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<IIQ", CONTAINER_VERSION, 0, len(header)))
        f.write(header)
        f.write(b"\0" * (base - 24 - len(header)))
        for raw in blobs:
            f.write(raw)
            f.write(b"\0" * ((-len(raw)) % 256))
    return path


def load_container(path, device="cpu"):
    """-> (tensors, meta).  The file is memory-mapped; each blob is copied once, to `device`."""
    path = Path(path)
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    if bytes(mm[:8]) != MAGIC:
        raise ValueError(f"{path}: not a turbopi_b200 weight container")
    version, _, hlen = struct.unpack("<IIQ", bytes(mm[8:24]))
    if version != CONTAINER_VERSION:
        raise ValueError(f"{path}: container version {version}, this build reads {CONTAINER_VERSION}")
    header = json.loads(bytes(mm[24:24 + hlen]).decode("utf-8"))
    base = (24 + hlen + 255) // 256 * 256
    out = {}
    for name, e in header["tensors"].items():
        raw = mm[base + e["offset"]: base + e["offset"] + e["nbytes"]]
        arr = np.frombuffer(raw, dtype=_NP[e["dtype"]]).reshape(e["shape"])
        t = torch.from_numpy(arr.copy())
        if e["dtype"] == "bfloat16":
            t = t.view(torch.bfloat16)
        out[name] = t.to(device)
    return out, header["meta"]


# ------------------------------------------------------------------------------------------------
# reference checkpoint naming
# ------------------------------------------------------------------------------------------------
_PG = "paligemma_with_expert.paligemma.model."
_EX = "paligemma_with_expert.gemma_expert.model."


def reference_state_dict_names(cfg) -> Dict[str, tuple]:
    """name -> shape of every tensor the Pi0.5 pipeline reads from a `PI0Pytorch.state_dict()`
    (module tree: openpi/src/openpi/models_pytorch/pi0_pytorch.py:112-140, gemma_pytorch.py:17-68 over the
    PaliGemma / Gemma / SigLIP modules of transformers 4.53.2)."""
    c = cfg
    vw, hd = c.vision_width, c.head_dim
    names = {}
    v = _PG + "vision_tower.vision_model."
    names[v + "embeddings.patch_embedding.weight"] = (vw, 3, c.patch, c.patch)
    names[v + "embeddings.patch_embedding.bias"] = (vw,)
    names[v + "embeddings.position_embedding.weight"] = (c.image_tokens, vw)
    for i in range(c.vision_layers):
        L = f"{v}encoder.layers.{i}."
        for ln in ("layer_norm1", "layer_norm2"):
            names[L + ln + ".weight"] = (vw,)
            names[L + ln + ".bias"] = (vw,)
        for p in ("q_proj", "k_proj", "v_proj", "out_proj"):
            names[L + f"self_attn.{p}.weight"] = (vw, vw)
            names[L + f"self_attn.{p}.bias"] = (vw,)
        names[L + "mlp.fc1.weight"], names[L + "mlp.fc1.bias"] = (c.vision_mlp, vw), (c.vision_mlp,)
        names[L + "mlp.fc2.weight"], names[L + "mlp.fc2.bias"] = (vw, c.vision_mlp), (vw,)
    names[v + "post_layernorm.weight"], names[v + "post_layernorm.bias"] = (vw,), (vw,)
    names[_PG + "multi_modal_projector.linear.weight"] = (c.width, vw)
    names[_PG + "multi_modal_projector.linear.bias"] = (c.width,)
    names[_PG + "language_model.embed_tokens.weight"] = (c.vocab, c.width)

    def decoder(prefix, width, mlp, adaptive):
        for p, n in (("q_proj", c.q_dim), ("k_proj", hd), ("v_proj", hd)):
            names[prefix + f"self_attn.{p}.weight"] = (n, width)
        names[prefix + "self_attn.o_proj.weight"] = (width, c.q_dim)
        names[prefix + "mlp.gate_proj.weight"] = (mlp, width)
        names[prefix + "mlp.up_proj.weight"] = (mlp, width)
        names[prefix + "mlp.down_proj.weight"] = (width, mlp)
        for ln in ("input_layernorm", "post_attention_layernorm"):
            if adaptive:
                names[prefix + ln + ".dense.weight"] = (3 * width, width)
                names[prefix + ln + ".dense.bias"] = (3 * width,)
            else:
                names[prefix + ln + ".weight"] = (width,)

    for i in range(c.prefix_layers):
        decoder(f"{_PG}language_model.layers.{i}.", c.width, c.mlp, False)
    for i in range(c.expert_layers):
        decoder(f"{_EX}layers.{i}.", c.expert_width, c.expert_mlp, True)
    ew = c.expert_width
    names[_EX + "norm.dense.weight"], names[_EX + "norm.dense.bias"] = (3 * ew, ew), (3 * ew,)
    names["action_in_proj.weight"], names["action_in_proj.bias"] = (ew, c.action_dim), (ew,)
    names["action_out_proj.weight"], names["action_out_proj.bias"] = (c.action_dim, ew), (c.action_dim,)
    for k in ("time_mlp_in", "time_mlp_out"):
        names[k + ".weight"], names[k + ".bias"] = (ew, ew), (ew,)
    return names


def random_state_dict(cfg, seed=0, device="cpu", std=0.02) -> Dict[str, torch.Tensor]:
    """A seeded stand-in for a checkpoint, under the reference's tensor names (small configs only: the full
    model is 3.3 G parameters)."""
    g = torch.Generator(device=device).manual_seed(seed)
    sd = {}
    for name, shape in reference_state_dict_names(cfg).items():
        norm = len(shape) == 1 and ("layernorm" in name or "layer_norm" in name)
        t = torch.randn(shape, generator=g, device=device) * (0.1 if norm else std)
        if "layer_norm" in name and name.endswith("weight") or "post_layernorm.weight" in name:
            t = t + 1.0                       # nn.LayerNorm scales sit around one; GemmaRMSNorm stores (scale - 1)
        sd[name] = t
    return sd


def load_checkpoint(path) -> Dict[str, torch.Tensor]:
    """A `.safetensors` checkpoint (what the reference ships) or a torch-saved state dict, on the host."""
    path = Path(path)
    if path.suffix == ".safetensors":
        from safetensors.torch import load_file
        return load_file(str(path))
    sd = torch.load(path, map_location="cpu", weights_only=True)
    return sd.get("state_dict", sd) if isinstance(sd, dict) else sd
