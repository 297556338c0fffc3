"""Pin the CPU oracle: against the reference's deterministic packer test and
against golden vectors made by the reference's own Python code
(tests/golden/make_golden.py)."""
import numpy as np
import torch

from oracle import formats, int4, kv_fuse, nvfp4, w4a8


# ---------------------------------------------------------------- number formats
def test_e4m3_matches_torch_exhaustive_bytes():
    codes = np.arange(256, dtype=np.uint8)
    ours = formats.e4m3_decode(codes)
    theirs = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    ok = ~np.isnan(theirs)
    assert np.array_equal(ours[ok], theirs[ok])
    assert np.isnan(ours[~ok]).all()


def test_e4m3_encode_matches_torch():
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.normal(size=20000).astype(np.float32) * rng.choice([1e-3, 0.02, 1.0, 50.0], size=20000).astype(np.float32),
        np.linspace(-448, 448, 4001, dtype=np.float32),
        formats.e4m3_decode(np.arange(0, 127, dtype=np.uint8)),                       # exact values
        (formats.e4m3_decode(np.arange(0, 126, dtype=np.uint8)) +
         formats.e4m3_decode(np.arange(1, 127, dtype=np.uint8))) / 2,                # every midpoint (ties)
        np.array([0.0, -0.0, 2.0 ** -10, 2.0 ** -9, 1.5 * 2.0 ** -9, 448.0, 447.9], dtype=np.float32),
    ]).astype(np.float32)
    ours = formats.e4m3_encode(x)
    theirs = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(ours, theirs)
    # saturation (CUDA's satfinite; torch would give NaN there)
    assert formats.e4m3_encode(np.float32([1e6, -500.0])).tolist() == [0x7E, 0xFE]


def test_bf16_rounding_matches_torch():
    rng = np.random.default_rng(1)
    x = (rng.normal(size=50000) * 10.0 ** rng.integers(-6, 6, size=50000)).astype(np.float32)
    ours = formats.round_to_bf16(x)
    theirs = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(ours, theirs)
    assert np.array_equal(formats.bf16_from_bits(formats.bf16_bits(x)), ours)


# ---------------------------------------------------------------- INT4 packers
def test_debug_packer_known_answer():
    """openpi/src/openpi/tests/debug_packer.py:41-117: weight ((n*K+k) % 15) - 7,
    N=4, K=32; expected first word and scale are computed by hand there."""
    N, K = 4, 32
    w = np.array([[((n * K + k) % 15) - 7 for k in range(K)] for n in range(N)], dtype=np.float32)
    block = w[0]
    scale_manual = np.max(np.abs(block)) / 7
    qm = [max(0, min(15, int(np.round(block[i] / scale_manual) + 8))) for i in range(8)]
    expected = 0
    for i in range(8):
        expected |= qm[i] << (i * 4)
    for packer in (int4.pack_basic, int4.pack_fast):
        packed, scales = packer(w)
        assert packed.shape == (1, 4, 4) and scales.shape == (1, 4)
        assert int(packed.view(np.uint32)[0, 0, 0]) == expected
        assert float(scales[0, 0]) == float(np.float16(scale_manual))
        assert np.array_equal(int4.dequantize(packed, scales), w)    # integers round-trip exactly


def test_int4_packers_match_reference(golden):
    g = golden("int4_packers")
    packed, scales = int4.pack_fast(g["weight"])
    assert np.array_equal(packed, g["fast_packed"].astype(np.int32))
    assert np.array_equal(scales.view(np.uint16), g["fast_scales"].view(np.uint16))
    bpacked, bscales = int4.pack_basic(g["weight"])
    assert np.array_equal(bpacked, g["basic_packed"])
    assert np.array_equal(bscales.view(np.uint16), g["basic_scales"].view(np.uint16))
    assert np.array_equal(int4.dequantize(bpacked, bscales), g["basic_unpacked"].astype(np.float32))


def test_int4_rowmajor_layout_holds_the_same_codes():
    rng = np.random.default_rng(3)
    w = rng.normal(size=(16, 256)).astype(np.float32)
    pk, sk = int4.pack_fast(w, 32, "kblock")
    pr, sr = int4.pack_fast(w, 32, "rowmajor")
    assert np.array_equal(int4.unpack_codes(pk, "kblock"), int4.unpack_codes(pr, "rowmajor"))
    assert np.array_equal(sk.T, sr)
    x = rng.normal(size=(1, 256)).astype(np.float32)
    a = int4.gemv_reference_math(x, pk, sk, "kblock")
    b = int4.gemv_dequant_matmul(x.astype(np.float16), pk, sk, "kblock")
    assert np.abs(a - b).max() / np.abs(b).max() < 2e-3


def test_plugin_int4_quantiser_roundtrip():
    rng = np.random.default_rng(4)
    w = formats.round_to_bf16(rng.uniform(-1, 1, size=(8, 256)).astype(np.float32))
    packed, scales, zeros = int4.plugin_quantize_int4(w, 128)
    assert packed.shape == (8, 128) and scales.shape == (8, 2)
    d = int4.plugin_dequantize_int4(packed, scales, zeros, 128)
    assert np.abs(d - w).max() <= np.repeat(scales, 128, axis=1).max() * 0.5 + 1.5e-2   # half a step + bf16 rounding of scale and output


# ---------------------------------------------------------------- NVFP4 packed plugin
def test_nvfp4_packed_matches_reference(golden):
    g = golden("nvfp4_packed")
    q, s = nvfp4.quantize_to_nvfp4(g["weight"], 32)
    assert np.array_equal(q, g["quantized"])
    assert np.array_equal(s, g["scales"])
    packed = nvfp4.pack_nvfp4(q)
    assert np.array_equal(packed, g["packed"])
    assert not ((packed & 0xF) == 8).any() and not ((packed >> 4) == 8).any()   # code 8 never emitted
    assert np.array_equal(nvfp4.unpack_nvfp4(packed), g["unpacked"])
    for a in (0, 1, 2):
        y = nvfp4.gemv_dequant_matmul(g["x"], packed, s, g["bias"], a, 32)
        np.testing.assert_allclose(y, g[f"out_act{a}"], rtol=2e-5, atol=2e-6)


def test_kv_fuse_matches_reference(golden):
    g = golden("kv_fuse")
    for name in ("q", "k", "v"):
        packed, scales = nvfp4.kv_fuse_quantize_to_fp4(g[f"W{name}"], 32)
        assert np.array_equal(packed, g[f"W{name}_packed"])
        assert np.array_equal(scales, g[f"scale_W{name}"])
    assert ((g["Wk_packed"] & 0xF) == 8).any()          # sign taken from the input: code 8 appears
    assert np.array_equal(kv_fuse.kv_fuse_dequantize(g["Wk_packed"], g["scale_Wk"]), g["Wk_dequant"])
    kc = np.full_like(g["K_cache"], -7.0)
    vc = np.full_like(g["V_cache"], -7.0)
    Q = kv_fuse.fused_qkv_fallback(g["x"], g["Wq_packed"], g["scale_Wq"], g["Wk_packed"], g["scale_Wk"],
                                   g["Wv_packed"], g["scale_Wv"], kc, vc, int(g["cache_pos"]),
                                   num_kv_heads=1, head_dim=32)
    np.testing.assert_allclose(Q, g["Q"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(kc, g["K_cache"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(vc, g["V_cache"], rtol=1e-5, atol=1e-6)
    # rows other than cache_pos keep the sentinel, exactly
    other = [i for i in range(kc.shape[1]) if i != int(g["cache_pos"])]
    assert (kc[:, other] == -7.0).all() and (g["K_cache"][:, other] == -7.0).all()


# ---------------------------------------------------------------- NVFP4 simulation (prefix GEMM)
def test_nvfp4_sim_matches_reference(golden):
    g = golden("nvfp4_sim")
    assert np.array_equal(nvfp4._torch_linspace_f32(0.7, 1.0, 10), g["linspace"])
    q, s = nvfp4.quantize_to_nvfp4_sim(g["weight"], 32, use_mse_search=True)
    assert np.array_equal(s, g["ws_mse"])
    assert np.array_equal(q, g["wq_mse"])
    assert (g["ws_mse"] != g["ws_minmax"]).any()        # the search really moved a scale
    q2, s2 = nvfp4.quantize_to_nvfp4_sim(g["weight"], 32, use_mse_search=False)
    assert np.array_equal(q2, g["wq_minmax"]) and np.array_equal(s2, g["ws_minmax"])
    wd = nvfp4.dequantize_nvfp4_sim(q, s, 32, use_fp8_scales=True)
    assert np.array_equal(wd, g["w_dequant_fp8"])
    xq, xs = nvfp4.quantize_to_nvfp4_sim(g["x"], 32, use_mse_search=False)
    assert np.array_equal(xq, g["xq"]) and np.array_equal(xs, g["xs"])
    assert np.array_equal(nvfp4.dequantize_nvfp4_sim(xq, xs, 32, True), g["x_dequant_fp8"])
    assert np.array_equal(nvfp4.pack_nvfp4_data(q), g["w_packed"])
    assert np.array_equal(formats.e4m3_encode(s).reshape(-1), g["ws_fp8_bytes"].reshape(-1))
    y = nvfp4.linear_sim(g["x"], q, s, 32)
    np.testing.assert_allclose(y, g["y"], rtol=2e-5, atol=2e-6)


def test_scale_swizzle_matches_reference_python_layout(golden):
    """The reference's python description of the 128x4 scale atom
    (openpi/src/openpi/models_pytorch/nvfp4_mlp.py:224-288) orders bytes inside a
    tile as [row % 32][row // 32][k-block]; its tile order is k-tile outer.  Ours
    is row-tile outer (one 512-byte tile per MMA k-step is then contiguous per
    row-tile), so compare tile by tile."""
    g = golden("nvfp4_sim")
    ws = g["ws_mse"]                                      # (48, 4) fp32
    ref = g["ws_swizzled"].reshape(-1)                    # fp32 values in the reference's order
    ours = nvfp4.swizzle_scales_128x4(formats.e4m3_encode(ws))
    assert ours.size == 512
    # the reference groups [row//32][row%32][kb]; byte (r%32)*16 + (r//32)*4 + kb in ours
    r = np.arange(128)
    for kb in range(4):
        ref_vals = ref.reshape(4, 32, 4)[r // 32, r % 32, kb]
        our_vals = formats.e4m3_decode(ours[(r % 32) * 16 + (r // 32) * 4 + kb])
        assert np.array_equal(formats.round_to_e4m3(ref_vals), our_vals)


# ---------------------------------------------------------------- RoPE
def test_rope_matches_reference(golden):
    g = golden("rope")
    cos, sin = kv_fuse.rope_cos_sin(g["positions"], 256, 10000.0)
    assert np.array_equal(cos, g["cos"][0])
    assert np.array_equal(sin, g["sin"][0])
    q = np.transpose(g["q"][0], (1, 0, 2))              # (S, heads, d)
    k = np.transpose(g["k"][0], (1, 0, 2))
    qe = kv_fuse.apply_rope_bf16(q, cos, sin)
    ke = kv_fuse.apply_rope_bf16(k, cos, sin)
    assert np.array_equal(qe, np.transpose(g["q_embed"][0], (1, 0, 2)))
    assert np.array_equal(ke, np.transpose(g["k_embed"][0], (1, 0, 2)))


# ---------------------------------------------------------------- plugin CUDA quantisers (unpinned: self-consistency)
def test_plugin_nvfp4_weight_quantiser_properties():
    rng = np.random.default_rng(7)
    w = formats.round_to_bf16((rng.normal(size=(12, 64)) * 0.02).astype(np.float32))
    packed_t, scales_t = nvfp4.plugin_quantize_weight_nvfp4(w)
    assert packed_t.shape == (32, 12) and scales_t.shape == (4, 12)
    deq = nvfp4.dequantize(np.ascontiguousarray(packed_t.T), np.ascontiguousarray(scales_t.T), 16,
                           scale_is_e4m3=True)
    # e2m1 step is at most 1/3 of the value range; E4M3 rounding of the scale adds <= 6.25 %
    assert np.abs(deq - w).max() < np.abs(w).max() * 0.3


def test_fp8_activation_quantiser_properties():
    rng = np.random.default_rng(8)
    x = formats.round_to_bf16(rng.normal(size=(5, 1024)).astype(np.float32))   # 64 blocks per row: beyond 32
    v, s = w4a8.quantize_activation_fp8(x)
    assert v.shape == (5, 1024) and s.shape == (5, 64)
    deq = formats.e4m3_decode(v) * np.repeat(formats.e4m3_decode(s), 16, axis=1)
    # the stored scale is E4M3-rounded (subnormal range for N(0,1) inputs: steps of 2**-9) while the
    # values were divided by the unrounded one, so the round trip carries the scale's rounding error
    assert np.abs(deq - x).max() / np.abs(x).max() < 0.2
    assert (s[:, 32:] != 0).all()                       # every block is quantised, not only the first 32


# ---------------------------------------------------------------- model-level oracle (a12 / a13 / a14)
def _model_case(name):
    from oracle import pi05
    from pi05_fixture import load_model_fixture, oracle_cfg, oracle_weights
    g, cfg = load_model_fixture()
    w, ocfg = oracle_weights(g, cfg), oracle_cfg(cfg)
    valid = torch.from_numpy(g[f"{name}.pad_mask"])
    cos, sin = pi05.rope_tables(torch.arange(1024), cfg["head_dim"], bf16=False)
    return pi05, g, cfg, w, ocfg, valid, cos, sin


def test_model_oracle_masks_and_positions_match_reference():
    """prefix_valid / prefix_positions against the masks and position ids the reference's embed_prefix,
    compute_prefix_kv_cache and precompute_graph_tensors produced (padded prompt, missing camera)."""
    for name, image_valid, prompt_len in (("A", [True, True], 10), ("B", [True, True], 7), ("C", [True, False], 7)):
        pi05, g, cfg, w, ocfg, valid, cos, sin = _model_case(name)
        ours = pi05.prefix_valid(ocfg, image_valid, prompt_len)
        assert torch.equal(ours, valid)
        pos, first = pi05.prefix_positions(valid)
        ref_pos = torch.from_numpy(g[f"{name}.position_ids"])
        assert torch.equal(pos[valid], ref_pos[valid])
        A = cfg["action_horizon"]
        assert np.array_equal(np.arange(first, first + A), g[f"{name}.suffix_position_ids"])
        # the reference's additive mask: action tokens see valid prefix keys and every action token
        key_valid = torch.cat([valid, torch.ones(A, dtype=torch.bool)])
        assert np.array_equal(np.broadcast_to(key_valid.numpy(), (A, key_valid.numel())), g[f"{name}.attention_mask_is_zero"])


def test_model_oracle_sinusoid_and_conditioning_match_reference():
    pi05, g, cfg, w, ocfg, valid, cos, sin = _model_case("A")
    s = pi05.sinusoidal(torch.from_numpy(g["sinusoid_t"]), 1024)
    assert np.array_equal(s.numpy(), g["sinusoid_1024"])              # float64, bit-exact
    with pi05.exact_fp32():
        for i, t in enumerate([1.0, 1.0 - 1.0 / 3, 1.0 - 2.0 / 3]):
            c = pi05.adarms_cond(w, torch.tensor([t], dtype=torch.float32), cfg["expert_width"])
            assert np.allclose(c[0].numpy(), g["A.adarms_conds"][i], rtol=1e-5, atol=1e-6)


def test_model_oracle_matches_reference_model():
    """Vision tower + prefix pass + denoise steps of the oracle in exact-fp32 mode against what the
    reference's own classes / PI0Pytorch methods computed on the same weights."""
    for name in ("A", "B", "C"):
        pi05, g, cfg, w, ocfg, valid, cos, sin = _model_case(name)
        images = torch.from_numpy(g["images_u8"])
        tokens = torch.from_numpy(g["tokens"])
        noise = torch.from_numpy(g["noise"])
        T = 2 * (cfg["image_size"] // cfg["patch"]) ** 2
        with pi05.exact_fp32():
            img_tokens = pi05.vision_tower(w, images, ocfg)
            assert np.allclose(img_tokens.numpy(), g[f"{name}.prefix_embs"][:T], rtol=1e-4, atol=2e-5)
            kv = pi05.prefix_pass(w, img_tokens, tokens, ocfg, cos, sin, valid)
            v = valid.numpy()
            for l in range(cfg["prefix_layers"]):
                assert np.allclose(kv[l][0].numpy()[v], g[f"{name}.k{l}"][v], rtol=1e-4, atol=2e-5), (name, "K", l)
                assert np.allclose(kv[l][1].numpy()[v], g[f"{name}.v{l}"][v], rtol=1e-4, atol=2e-5), (name, "V", l)
            # the denoise steps read the REFERENCE's cache (invalid rows included: they are masked)
            kv_ref = [(torch.from_numpy(g[f"{name}.k{l}"]), torch.from_numpy(g[f"{name}.v{l}"]))
                      for l in range(cfg["prefix_layers"])]
            cond = pi05.adarms_cond(w, torch.tensor([1.0]), cfg["expert_width"])
            v0 = pi05.denoise_velocity(w, kv_ref, noise, cond, ocfg, cos, sin, valid)
            assert np.allclose(v0.numpy(), g[f"{name}.v_step0"], rtol=1e-4, atol=2e-5), name
            actions = pi05.denoise(w, kv, noise, 3, ocfg, cos, sin, valid)
            assert np.allclose(actions.numpy(), g[f"{name}.actions"], rtol=1e-4, atol=5e-5), name
    # with nothing padded the reference's unmasked cached step equals its graph-safe masked one
    assert np.allclose(g["A.v_step0_with_cache"], g["A.v_step0"], rtol=1e-5, atol=1e-6)


def test_model_oracle_bf16_mode_stays_close_to_fp32_reference():
    """The bf16-rounding mode (the one the GPU pipeline is compared with) differs from the fp32 reference
    only by bf16 noise."""
    pi05, g, cfg, w, ocfg, valid, cos, sin = _model_case("B")
    cos_b, sin_b = pi05.rope_tables(torch.arange(1024), cfg["head_dim"], bf16=True)
    actions, _ = pi05.sample_actions(w, torch.from_numpy(g["images_u8"]), torch.from_numpy(g["tokens"]),
                                     torch.from_numpy(g["noise"]), 3, ocfg, cos_b, sin_b, valid)
    assert np.abs(actions.numpy() - g["B.actions"]).max() < 2e-2


def test_att_2d_mask_example():
    """make_att_2d_masks on a hand-sized case (prefix-LM blocks + padding), as stored by the reference run."""
    from pi05_fixture import load_model_fixture
    g, _ = load_model_fixture()
    pad = np.array([1, 1, 0, 1, 0], dtype=bool)
    ar = np.cumsum([0, 0, 0, 1, 0])
    ours = (ar[None, :] <= ar[:, None]) & (pad[None, :] & pad[:, None])
    assert np.array_equal(ours, g["att2d_example"])
