"""End-to-end parity of the Pi0.5-shaped pipeline with the oracle (oracle/pi05.py, pinned to the
reference's own model code by tests/test_oracle_golden.py): a reduced model against the CPU oracle
(padded prompt / missing camera included), then the FULL widths and head geometry at growing depth, up
to the full 27 + 18 + 18 layers, where the same oracle code is executed in fp32 on the GPU (after a check
that its GPU execution agrees with its CPU execution)."""
import os
import numpy as np
import pytest
import torch

from conftest import cosine, rel_err
from oracle import nvfp4 as onv
from oracle import pi05 as opi

pytestmark = pytest.mark.gpu


_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def _deq_torch(lin, device):
    """NVFP4 dequantisation with torch ops (exact: code value x E4M3 scale x global scale in fp32), for
    matrices too large for the numpy oracle to be practical; checked against it in
    test_torch_dequant_equals_numpy_oracle."""
    packed, scales, g = lin.raw
    lut = _E2M1.to(packed.device)
    N, Kh = packed.shape
    vals = torch.stack([lut[(packed & 0xF).long()], lut[(packed >> 4).long()]], dim=2).reshape(N, Kh * 2)
    sc = scales.view(torch.float8_e4m3fn).float().repeat_interleave(16, dim=1)
    return (vals * sc * torch.tensor(g, dtype=torch.float32, device=vals.device)).to(device), (None if lin.bias is None else lin.bias.float().to(device))


def _deq(lin):
    packed, scales, g = lin.raw
    w = onv.dequantize(packed.cpu().numpy(), scales.cpu().numpy(), 16, float(g), scale_is_e4m3=True)
    return torch.from_numpy(w), (None if lin.bias is None else lin.bias.float().cpu())


def _extract(model, device="cpu", deq=None):
    """Plain float32 weights of the quantised model, in the oracle's naming."""
    f = lambda t: t.float().to(device)
    _deq = deq or globals()["_deq"]
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


def _ocfg(cfg):
    return dict(image_size=cfg.image_size, patch=cfg.patch, vision_width=cfg.vision_width, vision_heads=cfg.vision_heads,
                eps=cfg.eps, width=cfg.width, q_dim=cfg.q_dim, head_dim=cfg.head_dim, heads=cfg.heads,
                expert_width=cfg.expert_width, text_len=cfg.text_len, num_images=cfg.num_images)


@torch.no_grad()
def test_torch_dequant_equals_numpy_oracle(cuda_device):
    from turbopi_b200.pi05 import TcLinear
    w = torch.randn(96, 256, generator=torch.Generator().manual_seed(0)) * 0.02
    lin = TcLinear.from_weight(w.to(cuda_device), None, None, keep_raw=True)
    a, _ = _deq(lin)
    b, _ = _deq_torch(lin, "cpu")
    assert torch.equal(a, b)


@torch.no_grad()
@pytest.mark.parametrize("image_valid,prompt_len", [([True, True], 17), ([True, False], 9)])
def test_reduced_pi05_padded_prompt_matches_oracle(cuda_device, image_valid, prompt_len):
    """Padded prompt / missing camera: positions from the mask, invalid keys never attended to."""
    from turbopi_b200 import _lib
    from turbopi_b200.pi05 import Pi05, Pi05Config
    cfg = Pi05Config(image_size=56, patch=14, vision_layers=2, vision_width=128, vision_mlp=272, vision_heads=2,
                     prefix_layers=2, width=256, mlp=512, text_len=24, vocab=1000, expert_layers=2, expert_width=128,
                     expert_mlp=256, action_horizon=50, action_dim=32, max_seq=256)
    model = Pi05(cfg, cuda_device, seed=4, keep_raw=True)
    g = torch.Generator().manual_seed(5)
    images = torch.randint(0, 256, (2, 56, 56, 3), generator=g, dtype=torch.uint8)
    tokens = torch.randint(0, 1000, (24,), generator=g)
    noise = torch.randn(50, 32, generator=g)
    full = model.infer(images, tokens, noise, num_steps=2, use_graph=True).cpu().clone()
    got = model.infer(images, tokens, noise, num_steps=2, use_graph=True, image_valid=image_valid,
                      prompt_len=prompt_len).cpu().clone()            # same captured graph, new mask buffers
    eager = model.infer(images, tokens, noise, num_steps=2, use_graph=False, image_valid=image_valid,
                        prompt_len=prompt_len).cpu().clone()
    assert _lib.load().tpb200_device_error(0) == 0
    assert (got - eager).abs().max() < 1e-3
    assert (got - full).abs().max() > 1e-3                     # the mask matters
    w = _extract(model)
    ocfg = _ocfg(cfg)
    valid = opi.prefix_valid(ocfg, image_valid, prompt_len)
    cos, sin = model.cos.float().cpu(), model.sin.float().cpu()
    ref, kv = opi.sample_actions(w, images, tokens, noise, 2, ocfg, cos, sin, valid)
    cache = model.cache.float().cpu()
    v = valid.numpy()
    for l in range(cfg.prefix_layers):
        assert rel_err(cache[l, 0, :cfg.prefix_len].numpy()[v], kv[l][0].numpy()[v]) <= 2e-2, ("K", l)
        assert rel_err(cache[l, 1, :cfg.prefix_len].numpy()[v], kv[l][1].numpy()[v]) <= 2e-2, ("V", l)
    err = (got - ref).abs().max().item()
    assert err <= 2e-2, err
    back = model.infer(images, tokens, noise, num_steps=2, use_graph=True, image_valid=[True, True],
                       prompt_len=cfg.text_len).cpu()
    assert torch.equal(back, full)                             # and the mask can be lifted again


@torch.no_grad()
def test_pi05_from_file_equals_from_state_dict(cuda_device, tmp_path):
    """state dict (reference names) -> prepared container -> model: same actions as the in-process path;
    the host tiler's images equal the CUDA tiler's."""
    from turbopi_b200 import ops, weights
    from turbopi_b200.pi05 import Pi05, Pi05Config
    cfg = Pi05Config(image_size=56, patch=14, vision_layers=1, vision_width=128, vision_mlp=272, vision_heads=2,
                     prefix_layers=1, width=256, mlp=512, text_len=24, vocab=500, expert_layers=1, expert_width=128,
                     expert_mlp=256, action_horizon=50, action_dim=32, max_seq=256)
    sd = weights.random_state_dict(cfg, seed=11)
    m1 = Pi05.from_state_dict(sd, cfg, cuda_device, keep_raw=True)
    m2 = Pi05.from_file(m1.save(tmp_path / "m.tpb"), cuda_device)
    g = torch.Generator().manual_seed(6)
    images = torch.randint(0, 256, (2, 56, 56, 3), generator=g, dtype=torch.uint8)
    tokens = torch.randint(0, 500, (24,), generator=g)
    noise = torch.randn(50, 32, generator=g)
    a1 = m1.infer(images, tokens, noise, num_steps=2).cpu()
    a2 = m2.infer(images, tokens, noise, num_steps=2).cpu()
    assert torch.equal(a1, a2)
    lin = m1.prefix[0]["gate_up"]
    packed, scales, _ = lin.raw
    b = torch.zeros((lin.N, ops.packed_pitch(lin.K)), dtype=torch.uint8, device=cuda_device)
    b[:, :lin.K // 2] = packed
    assert torch.equal(ops.tile_weights(b, ops.swizzle_scales(scales.contiguous()), lin.N, lin.K), lin.b)


FULL = dict(vision_layers=27, prefix_layers=18, expert_layers=18)


@torch.no_grad()
@pytest.mark.parametrize("depth", [2, 4, 8, "full"])
def test_full_width_error_vs_depth(cuda_device, depth):
    """Full widths (1152 / 2048 / 1024), real head geometry, 712-token prefix, 10 denoise steps at 2, 4, 8
    layers per tower and at the full 27 + 18 + 18: end-to-end actions within 2e-2 absolute of the oracle.
    Depth 2 also checks that the oracle's GPU execution (fp32 torch kernels) equals its CPU execution."""
    from turbopi_b200 import _lib
    from turbopi_b200.pi05 import Pi05, Pi05Config
    layers = FULL if depth == "full" else dict(vision_layers=depth, prefix_layers=depth, expert_layers=depth)
    steps = 10
    cfg = Pi05Config(vocab=4096, **layers)
    model = Pi05(cfg, cuda_device, seed=7, keep_raw=True)
    g = torch.Generator().manual_seed(8)
    images = torch.randint(0, 256, (2, 224, 224, 3), generator=g, dtype=torch.uint8)
    tokens = torch.randint(0, 4096, (cfg.text_len,), generator=g)
    noise = torch.randn(cfg.action_horizon, cfg.action_dim, generator=g)
    got = model.infer(images, tokens, noise, num_steps=steps, use_graph=True, prompt_len=180).cpu().clone()
    assert _lib.load().tpb200_device_error(0) == 0
    ocfg = _ocfg(cfg)
    valid = opi.prefix_valid(ocfg, None, 180)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        w = _extract(model, cuda_device, lambda lin: _deq_torch(lin, cuda_device))
        ref, _ = opi.sample_actions(w, images.to(cuda_device), tokens.to(cuda_device), noise.to(cuda_device), steps, ocfg,
                                    model.cos.float(), model.sin.float(), valid)
        ref = ref.cpu()
        if depth == 2:
            wc = _extract(model, "cpu", lambda lin: _deq_torch(lin, "cpu"))
            ref_cpu, _ = opi.sample_actions(wc, images, tokens, noise, steps, ocfg, model.cos.float().cpu(),
                                            model.sin.float().cpu(), valid)
            # same code, other fp32 summation orders; a flipped bf16 rounding moves an action by a few 1e-3
            assert (ref - ref_cpu).abs().max().item() <= 1e-2
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    err = (got - ref).abs().max().item()
    print(f"full-width depth {depth}: max |actions - oracle| = {err:.3e}, cosine = {cosine(got.numpy(), ref.numpy()):.6f}, "
          f"max |actions| = {ref.abs().max().item():.3f}")
    assert err <= 2e-2, err
    assert cosine(got.numpy(), ref.numpy()) >= 0.999


def test_two_pipelines_over_one_set_of_weights_on_two_streams(cuda_device):
    """`Pi05.sharing_weights`: a second pipeline over the same weight tensors (no copy) with buffers and scratch of
    its own.  Both replay their graphs on two streams at the same time, over and over; each returns what it
    returns alone (their split-K launches are cooperative launches, their scratch is per pipeline)."""
    from turbopi_b200 import _lib
    from turbopi_b200.pi05 import Pi05, Pi05Config
    cfg = Pi05Config(image_size=56, patch=14, vision_layers=2, vision_width=128, vision_mlp=272, vision_heads=2,
                     prefix_layers=2, width=256, mlp=512, text_len=24, vocab=500, expert_layers=2, expert_width=128,
                     expert_mlp=256, action_horizon=50, action_dim=32, max_seq=256)
    a = Pi05(cfg, cuda_device, seed=4)
    b = Pi05.sharing_weights(a)
    assert b.prefix[0]["gate_up"].b.data_ptr() == a.prefix[0]["gate_up"].b.data_ptr()
    assert b.workspace.data_ptr() != a.workspace.data_ptr() and b.cache.data_ptr() != a.cache.data_ptr()
    g = torch.Generator().manual_seed(8)
    inputs = [(torch.randint(0, 256, (2, 56, 56, 3), generator=g, dtype=torch.uint8), torch.randint(0, 500, (24,), generator=g),
               torch.randn(50, 32, generator=g)) for _ in range(2)]
    alone = [a.infer(*inputs[0], num_steps=3).clone(), a.infer(*inputs[1], num_steps=3).clone()]
    b.infer(*inputs[1], num_steps=3)                      # captures b's graph
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(device=cuda_device) for _ in range(2)]
    for _ in range(20):
        for m, s, inp in ((a, streams[0], inputs[0]), (b, streams[1], inputs[1])):
            with torch.cuda.stream(s):
                m.infer(*inp, num_steps=3)
    torch.cuda.synchronize()
    assert _lib.load().tpb200_device_error(0) == 0
    assert torch.equal(a.actions, alone[0]) and torch.equal(b.actions, alone[1])


def test_dispatcher_with_two_pipelines_in_flight_returns_what_one_returns(cuda_device):
    """`RequestDispatcher` over two `Pi05Policy` pipelines that share their weights (one host thread and one stream
    each): every request's actions equal those of the same request served by a single pipeline."""
    import numpy as np
    from turbopi_b200 import _lib
    from turbopi_b200.pi05 import Pi05, Pi05Config
    from turbopi_b200.policy import Pi05Policy
    from turbopi_b200.replicas import ReplicaGroup, RequestDispatcher
    cfg = Pi05Config(image_size=56, patch=14, vision_layers=2, vision_width=128, vision_mlp=272, vision_heads=2,
                     prefix_layers=2, width=256, mlp=512, text_len=24, vocab=500, expert_layers=2, expert_width=128,
                     expert_mlp=256, action_horizon=50, action_dim=32, max_seq=256)
    first = Pi05(cfg, cuda_device, seed=9)
    policies = [Pi05Policy(first, None, None, num_denoising_steps=3),
                Pi05Policy(Pi05.sharing_weights(first), None, None, num_denoising_steps=3)]
    rng = np.random.default_rng(2)
    noise = rng.normal(size=(50, 32)).astype(np.float32)
    reqs = [{"observation/image": rng.integers(0, 256, (56, 56, 3), dtype=np.uint8),
             "observation/wrist_image": rng.integers(0, 256, (56, 56, 3), dtype=np.uint8),
             "observation/state": rng.normal(size=8).astype(np.float32),
             "prompt": [2] + rng.integers(3, 500, 5 + i % 7).tolist(), "noise": noise} for i in range(10)]
    for p in policies:
        p.warmup(1)
    alone = [policies[0].infer(r)["actions"] for r in reqs]
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    group = ReplicaGroup(0, 1, 0, cuda_device)
    disp = RequestDispatcher(group, [lambda r, p=p: p.infer(r)["actions"] for p in policies], timeout_s=60.0)
    results, stats = disp.serve(reqs)
    assert _lib.load().tpb200_device_error(0) == 0
    assert stats["done"] == 10 and stats["requeued"] == []
    for got, ref in zip(results, alone):
        assert np.array_equal(got, ref)
