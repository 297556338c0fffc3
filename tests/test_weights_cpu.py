"""Offline weight pipeline on the host: reference interchange formats, the tiled-image container,
state-dict naming (turbopi_b200/weights.py; reference: openpi/nvfp4_packed_plugin/scripts/prepare_weights.py:134-296)."""
import numpy as np
import pytest
import torch

from turbopi_b200 import weights
from turbopi_b200.pi05 import Pi05, Pi05Config, TcLinear

SMALL = dict(image_size=28, patch=14, vision_layers=1, vision_width=64, vision_mlp=112, vision_heads=2,
             prefix_layers=1, width=128, mlp=256, text_len=8, vocab=64, expert_layers=1, expert_width=64,
             expert_mlp=128, action_horizon=50, action_dim=32, max_seq=128)


def test_prepare_linear_weights_matches_reference_golden(golden):
    """Same codes and scales as the reference's quantise + pack on its own golden weight."""
    g = golden("nvfp4_packed")
    d = weights.prepare_linear_weights(torch.from_numpy(g["weight"]), 32)
    assert np.array_equal(d["weight_packed"].numpy(), g["packed"])
    assert np.array_equal(d["weight_scales"].numpy(), g["scales"])
    assert (d["out_features"], d["in_features"]) == g["weight"].shape


@pytest.mark.parametrize("fmt", ["npz", "safetensors", "bin"])
def test_reference_formats_round_trip(tmp_path, fmt):
    gen = torch.Generator().manual_seed(0)
    sd = {"layers.0.mlp.gate_proj.weight": torch.randn(24, 64, generator=gen) * 0.02,
          "layers.0.mlp.down_proj.weight": torch.randn(16, 40, generator=gen) * 0.02,      # K padded to 64
          "layers.0.input_layernorm.weight": torch.randn(64, generator=gen),               # 1-D: skipped
          "layers.0.mlp.gate_proj.bias": torch.randn(24, generator=gen)}
    processed = weights.process_model_weights(sd, layer_patterns=["mlp"])
    assert set(processed) == {"layers.0.mlp.gate_proj.weight", "layers.0.mlp.down_proj.weight"}
    assert processed["layers.0.mlp.down_proj.weight"]["in_features"] == 64
    path = weights.save_packed_weights(processed, tmp_path / f"w.{fmt}", fmt)
    back = weights.load_packed_weights(path)
    for name, d in processed.items():
        key = name if fmt == "bin" else name.replace(".", "_")
        assert torch.equal(back[key]["weight_packed"], d["weight_packed"])
        assert torch.equal(back[key]["weight_scales"], d["weight_scales"])
        assert back[key]["out_features"] == d["out_features"] and back[key]["in_features"] == d["in_features"]


def test_container_round_trip_and_alignment(tmp_path):
    gen = torch.Generator().manual_seed(1)
    tensors = {"a.image": torch.randint(0, 256, (36864 * 2 + 0,), generator=gen, dtype=torch.uint8),
               "b": torch.randn(5, 7, generator=gen).to(torch.bfloat16), "c": torch.randn(3, generator=gen),
               "d": torch.arange(10, dtype=torch.int32)}
    path = weights.save_container(tmp_path / "m.tpb", tensors, {"kind": "test", "x": 1})
    raw = path.read_bytes()
    assert raw[:8] == weights.MAGIC
    back, meta = weights.load_container(path)
    assert meta == {"kind": "test", "x": 1}
    for k, t in tensors.items():
        assert back[k].dtype == t.dtype and torch.equal(back[k], t)
    # blobs sit on 256-byte boundaries of the file
    import json, struct
    version, _, hlen = struct.unpack("<IIQ", raw[8:24])
    assert version == weights.CONTAINER_VERSION
    base = (24 + hlen + 255) // 256 * 256
    for e in json.loads(raw[24:24 + hlen])["tensors"].values():
        assert (base + e["offset"]) % 256 == 0
    bad = tmp_path / "bad.tpb"
    bad.write_bytes(b"NOTMAGIC" + raw[8:])
    with pytest.raises(ValueError):
        weights.load_container(bad)


def test_state_dict_to_file_to_model_is_byte_identical(tmp_path):
    """random reference-named state dict -> Pi05 (quantise, permute, tile) -> file -> Pi05: every prepared
    tensor identical to the in-process path; a second preparation of the same state dict too."""
    cfg = Pi05Config(**SMALL)
    sd = weights.random_state_dict(cfg, seed=3)
    assert set(sd) == set(weights.reference_state_dict_names(cfg))
    m1 = Pi05.from_state_dict(sd, cfg, "cpu")
    path = m1.save(tmp_path / "pi05.tpb")
    m2 = Pi05.from_file(path, "cpu")
    m3 = Pi05.from_state_dict(sd, cfg, "cpu")
    assert m2.cfg == cfg
    n = 0
    for (na, a), (nb, b), (_, c) in zip(m1._named_parts(), m2._named_parts(), m3._named_parts()):
        assert na == nb
        if isinstance(a, TcLinear):
            assert torch.equal(a.b, b.b) and torch.equal(a.b, c.b)
            assert a.rowmajor == b.rowmajor == c.rowmajor           # the operand form travels with the file
            assert not a.rowmajor or (torch.equal(a.sf, b.sf) and torch.equal(a.sf, c.sf))
            assert a.g == b.g and (a.N, a.K) == (b.N, b.K)
            assert (a.bias is None) == (b.bias is None) and (a.bias is None or torch.equal(a.bias, b.bias))
            n += 1
        else:
            assert a.dtype == b.dtype and torch.equal(a, b)
    assert n == 2 + 4 * cfg.vision_layers + 4 * cfg.prefix_layers + 4 * cfg.expert_layers + 5
    # fused tensors: q / k / v stacked and tile-permuted, gate / up stacked, adaptive norms stacked
    assert m1.prefix[0]["qkv"].N == cfg.q_dim + 2 * cfg.head_dim and m1.prefix[0]["gate_up"].N == 2 * cfg.mlp
    assert m1.ada_dense.N == m1.n_norms * 3 * cfg.expert_width
    # the large prefix MLP matrices are tiled images, the rest row-major
    assert not m1.prefix[0]["gate_up"].rowmajor and not m1.prefix[0]["down"].rowmajor
    assert m1.prefix[0]["qkv"].rowmajor and m1.prefix[0]["o"].rowmajor and m1.expert[0]["down"].rowmajor
    assert m1.expert[0]["o"].rowmajor and m1.vision[0]["fc1"].rowmajor


def test_state_dict_errors():
    cfg = Pi05Config(**SMALL)
    sd = weights.random_state_dict(cfg, seed=3)
    from turbopi_b200._lib import TurboPiError
    broken = dict(sd)
    broken.pop("time_mlp_in.weight")
    with pytest.raises(TurboPiError):
        Pi05.from_state_dict(broken, cfg, "cpu")
    broken = dict(sd)
    broken["time_mlp_in.weight"] = torch.zeros(3, 3)
    with pytest.raises(TurboPiError):
        Pi05.from_state_dict(broken, cfg, "cpu")
    with pytest.raises(TurboPiError):                         # prefix + horizon must fit the KV cache
        Pi05(Pi05Config(**{**SMALL, "max_seq": 32}), "cpu")


def test_valid_mask_buffers():
    """Position ids and key bias for a padded prompt and a missing camera (pi0_pytorch.py:442,791-796)."""
    cfg = Pi05Config(**SMALL)
    m = Pi05(cfg, "cpu", seed=0)
    T = cfg.image_tokens
    m.set_valid([True, False], prompt_len=5)
    S = cfg.prefix_len
    valid = torch.cat([torch.ones(T, dtype=torch.bool), torch.zeros(T, dtype=torch.bool), torch.arange(cfg.text_len) < 5])
    assert torch.equal(m.valid, valid)
    pos = m.b["pos_prefix"].long()
    assert torch.equal(pos[valid], torch.arange(T + 5))
    assert torch.equal(m.b["pos_suffix"].long(), torch.arange(T + 5, T + 5 + cfg.action_horizon))
    assert (m.key_bias[:S][~valid].float() < -1e38).all() and (m.key_bias[:S][valid] == 0).all()
    assert (m.key_bias[S:] == 0).all()
    m.set_valid()
    assert torch.equal(m.b["pos_prefix"].long(), torch.arange(S)) and (m.key_bias == 0).all()


def test_a_second_pipeline_shares_the_weights_and_nothing_else():
    """`Pi05.sharing_weights`: the same weight tensors (no copy), separate linear objects, buffers, KV cache and
    scratch: what two pipelines need to run side by side on one GPU."""
    cfg = Pi05Config(**SMALL)
    a = Pi05.from_state_dict(weights.random_state_dict(cfg, seed=5), cfg, "cpu")
    b = Pi05.sharing_weights(a)
    assert b.cfg == a.cfg and b.launch_flags == a.launch_flags
    for (na, x), (nb, y) in zip(a._named_parts(), b._named_parts()):
        assert na == nb
        if isinstance(x, TcLinear):
            assert x is not y and x.b.data_ptr() == y.b.data_ptr() and x.rowmajor == y.rowmajor
            assert (x.N, x.K, x.g) == (y.N, y.K, y.g)
            assert x.ws.data_ptr() != y.ws.data_ptr()            # split-K scratch per pipeline
        else:
            assert x.data_ptr() == y.data_ptr()
    assert a.cache.data_ptr() != b.cache.data_ptr() and a.attn_ws.data_ptr() != b.attn_ws.data_ptr()
    assert a.b["ph"].data_ptr() != b.b["ph"].data_ptr() and a.actions.data_ptr() != b.actions.data_ptr()
