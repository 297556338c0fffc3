"""Pi0.5-shaped inference pipeline on the turbopi_b200 kernels.

SigLIP-So400m/14 vision tower -> Gemma-2B prefix (image + text tokens, fills the KV cache) ->
Gemma-300M action expert running N flow-matching Euler steps over 50 action tokens against that
cache (`PI0Pytorch.sample_actions`, openpi/src/openpi/models_pytorch/pi0_pytorch.py:876-937;
cached denoise step :524-654; adaptive RMSNorm / gated residual / MLP,
transformers_replace/models/gemma/modeling_gemma.py:49-129,212-230).

Every linear layer runs as NVFP4 weights x bf16 activations on the tcgen05 GEMM (activations
carried as residual e2m1 pieces); norms, residuals and GELU*up are the fused row kernels that
write the next GEMM's operand directly; Q/K/V + RoPE + KV-cache append is the GEMM's fused
epilogue; attention is the tensor-core kernel of csrc/attention.cu (`ops.attention`).  All buffers are
allocated once, so the whole inference (or just the denoise loop) replays as ONE CUDA graph.

Weights come from a reference-named state dict (`Pi05.from_state_dict`, tensor names of
`PI0Pytorch.state_dict()`), from a prepared container file (`Pi05.save` / `Pi05.from_file`,
turbopi_b200/weights.py) or, for benchmarks, from a seeded random initialisation.

Padding follows the reference: prefix tokens that do not exist (a missing camera, the padded tail of the
prompt) are never attended to, position ids are `cumsum(valid) - 1`, and the action tokens continue at
`sum(valid)` (pi0_pytorch.py:80-108,442,571-579,791-866).  The valid mask only changes small device
buffers (positions, additive key bias), so one captured graph serves every mask.
"""
import ctypes
import math
from dataclasses import dataclass

import torch

from . import _lib, ops, weights
from ._lib import ACT_GELU, ACT_NONE, ACT_SILU, TurboPiError
from .nvfp4_packed import quantize_nvfp4_two_level


@dataclass
class Pi05Config:
    # SigLIP-So400m/14
    image_size: int = 224
    patch: int = 14
    vision_layers: int = 27
    vision_width: int = 1152
    vision_mlp: int = 4304
    vision_heads: int = 16
    num_images: int = 2
    # Gemma-2B prefix
    prefix_layers: int = 18
    width: int = 2048
    mlp: int = 16384
    heads: int = 8
    head_dim: int = 256
    text_len: int = 200
    vocab: int = 257152
    # Gemma-300M action expert
    expert_layers: int = 18
    expert_width: int = 1024
    expert_mlp: int = 4096
    action_horizon: int = 50
    action_dim: int = 32
    max_seq: int = 1024
    pieces: int = 3
    eps: float = 1e-6

    @property
    def image_tokens(self):
        return (self.image_size // self.patch) ** 2

    @property
    def prefix_len(self):
        return self.num_images * self.image_tokens + self.text_len

    @property
    def q_dim(self):
        return self.heads * self.head_dim


QuantBuf, rowop = ops.QuantBuf, ops.rowop


class TcLinear:
    """One NVFP4 weight matrix prepared for the tensor-core GEMM (standard NVFP4: E4M3 scale per 16 and
    an fp32 global scale), the global scale, an optional fp32 bias, in one of the GEMM's two operand forms:
    the tiled image (`sf is None`; 128 x 256 output tiles, one contiguous block per K stage: the form for the
    large prefix MLP matrices), or
    row-major codes [N, pitch] + swizzled scale atoms (128 x 128 tiles, a three-stage ring: ~2 us less per launch
    on the small, latency-bound linears of the vision tower and the action expert).  The activation operand
    (`QuantBuf`) must be in the same form.  `raw` keeps the reference-layout codes / scale bytes for
    dequantisation in tests."""

    def __init__(self, image, g, N, K, bias=None, raw=None, sf=None):
        self.b, self.sf, self.g, self.N, self.K = image, sf, float(g), int(N), int(K)
        self.bias = None if bias is None else bias.float().contiguous()
        if raw is not None:
            self.raw = raw
        self.ws = None            # split-K scratch, set by the owning pipeline

    @property
    def rowmajor(self):
        return self.sf is not None

    @classmethod
    def from_weight(cls, weight, bias=None, row_perm=None, keep_raw=False, rowmajor=False):
        N, K = weight.shape
        packed, scales, g = quantize_nvfp4_two_level(weight, 16)
        raw = (packed.clone(), scales.clone(), g) if keep_raw else None
        if row_perm is not None:
            packed, scales = packed[row_perm], scales[row_perm]
        if rowmajor:
            b = torch.zeros((N, ops.packed_pitch(K)), dtype=torch.uint8, device=packed.device)
            b[:, :K // 2] = packed
            return cls(b, g, N, K, bias, raw, sf=ops.swizzle_scales(scales.contiguous()))
        return cls(weights.tile_weights_host(packed, scales), g, N, K, bias, raw)

    def _args(self, q, M):
        if q.tiled == self.rowmajor:
            raise TurboPiError("activation operand and weight are in different operand forms")
        p = ops._ptr
        if self.rowmajor:
            return _lib.GemmArgs(a_packed=p(q.packed), a_pitch=q.pitch, a_sf=p(q.sf), a_pieces=q.pieces,
                                 a_piece_rows=q.piece_rows, a_row_scale=p(q.row_scale), b_packed=p(self.b),
                                 b_pitch=self.b.stride(0), b_sf=p(self.sf), alpha=float(self.g), M=M, N=self.N, K=self.K,
                                 layout=ops.OPERANDS_ROWMAJOR)
        return _lib.GemmArgs(a_packed=p(q.packed), a_pieces=q.pieces, a_row_scale=p(q.row_scale), b_packed=p(self.b),
                             alpha=float(self.g), M=M, N=self.N, K=self.K, layout=ops.OPERANDS_TILED)

    def __call__(self, q, out, activation=ACT_NONE, M=None):
        args = self._args(q, q.M if M is None else M)
        args.bias, args.activation = ops._ptr(self.bias), int(activation)
        args.out, args.out_dtype, args.ldo = ops._ptr(out), ops._dt(out), out.stride(0)
        ops._gemm_ex(args, out.device, self.ws)
        return out

    def qkv(self, q, q_out, k_rows, v_rows, positions, cos, sin, q_dim, M=None):
        M = q.M if M is None else M
        if k_rows.shape[0] < M or v_rows.shape[0] < M or positions.numel() < M:
            raise TurboPiError("fused QKV: cache rows / positions shorter than the token count")
        p = ops._ptr
        args = self._args(q, M)
        args.qkv_q_out, args.qkv_ldq, args.qkv_q_dim = p(q_out), q_out.stride(0), q_dim
        args.qkv_k_rows, args.qkv_v_rows, args.qkv_positions = p(k_rows), p(v_rows), p(positions)
        args.qkv_rope_cos, args.qkv_rope_sin = p(cos), p(sin)
        ops._gemm_ex(args, q_out.device, self.ws)
        return q_out


def sinusoidal_time_embedding(t, dim, min_period=4e-3, max_period=4.0):
    """openpi/src/openpi/models_pytorch/pi0_pytorch.py:53-70 (float64)."""
    frac = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float64)
    period = min_period * (max_period / min_period) ** frac
    ang = (1.0 / period * 2 * math.pi)[None, :] * t.to(torch.float64)[:, None]
    return torch.cat([torch.sin(ang), torch.cos(ang)], dim=1)


class Pi05:
    """Pi0.5-shaped model; `infer(images_u8, tokens, noise, num_steps)` -> actions [50, 32].

    Pi05(cfg, device, seed=...)            seeded random weights (benchmarks, tests)
    Pi05.from_state_dict(sd, cfg, device)  tensors under the reference's names (weights.reference_state_dict_names)
    Pi05.from_file(path, device)           a container written by `save()`
    """

    def __init__(self, cfg: Pi05Config, device, seed=0, keep_raw=False, pdl=True, state_dict=None, _prepared=None):
        self.cfg, self.device = cfg, device
        c = cfg
        if c.prefix_len + c.action_horizon > c.max_seq:
            raise TurboPiError(f"prefix ({c.prefix_len}) + action horizon ({c.action_horizon}) exceed the KV cache "
                               f"({c.max_seq} rows)")
        # programmatic dependent launch across the GEMM / row-kernel chain: each kernel's launch and set-up
        # overlap the tail of the one before it
        self.launch_flags = ops.FLAG_PDL if pdl else ops.FLAG_NONE
        self.keep_raw = keep_raw
        self.patch_k = (3 * c.patch * c.patch + 15) // 16 * 16
        self.n_norms = 2 * c.expert_layers + 1
        self.workspace = ops.gemm_workspace(device)       # split-K scratch of THIS pipeline's launches
        if _prepared is not None:
            self._from_prepared(_prepared)
        else:
            self._from_tensors(self._random_source(seed) if state_dict is None else self._dict_source(state_dict))
        self.cos, self.sin = ops.rope_tables(c.max_seq, c.head_dim, device=device)
        if self.cos.shape[0] != c.max_seq:
            raise TurboPiError("RoPE table and KV cache disagree on the number of positions")
        self._alloc()
        self._graph = None
        self._graph_steps = None
        self._time_emb = {}
        self._mod = {}            # per step count: the adaptive norms' modulation table
        self.set_valid()

    @classmethod
    def from_state_dict(cls, state_dict, cfg: Pi05Config, device, **kw):
        return cls(cfg, device, state_dict=state_dict, **kw)

    @classmethod
    def from_file(cls, path, device, **kw):
        tensors, meta = weights.load_container(path, device)
        if meta.get("kind") != "pi05":
            raise TurboPiError(f"{path}: not a Pi0.5 weight container")
        return cls(Pi05Config(**meta["config"]), device, _prepared=(tensors, meta), **kw)

    # ------------------------------------------------------------------ weights
    def _random_source(self, seed):
        g = torch.Generator(device=self.device).manual_seed(seed)
        shapes = weights.reference_state_dict_names(self.cfg)

        def get(name):
            shape = shapes[name]
            norm = len(shape) == 1 and ("layernorm" in name or "layer_norm" in name)
            # norm parameters: small random values so that the norms are not the identity
            t = torch.randn(shape, generator=g, device=self.device) * (0.1 if norm else 0.02)
            if norm and name.endswith(".weight") and ("layer_norm" in name or "post_layernorm" in name):
                t = t + 1.0
            return t
        return get

    def _dict_source(self, sd):
        shapes = weights.reference_state_dict_names(self.cfg)
        missing = [n for n in shapes if n not in sd]
        if missing:
            raise TurboPiError(f"state dict lacks {len(missing)} tensors, e.g. {missing[:3]}")

        def get(name):
            t = sd[name]
            if tuple(t.shape) != tuple(shapes[name]):
                raise TurboPiError(f"{name}: shape {tuple(t.shape)}, expected {tuple(shapes[name])}")
            return t.to(self.device).float()
        return get

    def _from_tensors(self, get):
        """Quantise, permute and tile every linear; norms, embeddings and tables go to bf16."""
        c, kr = self.cfg, self.keep_raw
        bf = torch.bfloat16
        V = "paligemma_with_expert.paligemma.model.vision_tower.vision_model."
        PG = "paligemma_with_expert.paligemma.model."
        EX = "paligemma_with_expert.gemma_expert.model."

        # Operand form per linear: the tiled image for the large prefix MLP matrices (gate_up, down), row-major
        # for everything else (the vision tower, the attention projections, the action expert, the small projections).
        def lin(wname, bias=True, perm=None, rm=True):
            return TcLinear.from_weight(get(wname + ".weight"), get(wname + ".bias") if bias else None, perm, kr, rm)

        def stacked(names, bias, perm=None, rm=True):
            w = torch.cat([get(n + ".weight") for n in names], 0)
            b = torch.cat([get(n + ".bias") for n in names], 0) if bias else None
            return TcLinear.from_weight(w, b, perm, kr, rm)

        vw = c.vision_width
        wp = torch.zeros(vw, self.patch_k, device=self.device)
        wp[:, :3 * c.patch * c.patch] = get(V + "embeddings.patch_embedding.weight").reshape(vw, -1)   # (c, i, j)
        self.patch_embed = TcLinear.from_weight(wp, get(V + "embeddings.patch_embedding.bias"), None, kr, True)
        self.pos_emb = get(V + "embeddings.position_embedding.weight").to(bf)
        self.vision = []
        for i in range(c.vision_layers):
            L = f"{V}encoder.layers.{i}."
            self.vision.append(dict(
                ln1_w=get(L + "layer_norm1.weight").to(bf), ln1_b=get(L + "layer_norm1.bias").to(bf),
                qkv=stacked([L + "self_attn.q_proj", L + "self_attn.k_proj", L + "self_attn.v_proj"], True),
                out=lin(L + "self_attn.out_proj"),
                ln2_w=get(L + "layer_norm2.weight").to(bf), ln2_b=get(L + "layer_norm2.bias").to(bf),
                fc1=lin(L + "mlp.fc1"), fc2=lin(L + "mlp.fc2")))
        self.post_ln_w, self.post_ln_b = get(V + "post_layernorm.weight").to(bf), get(V + "post_layernorm.bias").to(bf)
        self.projector = lin(PG + "multi_modal_projector.linear")

        perm = ops.qkv_tile_permutation(c.q_dim).to(self.device)
        self.embed_tokens = get(PG + "language_model.embed_tokens.weight").to(bf)

        def decoder(prefix, mlp_rm):
            a = prefix + "self_attn."
            return dict(qkv=stacked([a + "q_proj", a + "k_proj", a + "v_proj"], False, perm),
                        o=lin(a + "o_proj", False),
                        gate_up=stacked([prefix + "mlp.gate_proj", prefix + "mlp.up_proj"], False, rm=mlp_rm),
                        down=lin(prefix + "mlp.down_proj", False, rm=mlp_rm))

        self.prefix = []
        for i in range(c.prefix_layers):
            L = f"{PG}language_model.layers.{i}."
            d = decoder(L, False)
            d["in_norm"] = get(L + "input_layernorm.weight").to(bf)
            d["post_norm"] = get(L + "post_attention_layernorm.weight").to(bf)
            self.prefix.append(d)

        self.action_in = lin("action_in_proj")
        self.action_out = lin("action_out_proj")
        self.time_mlp_in = lin("time_mlp_in")
        self.time_mlp_out = lin("time_mlp_out")
        self.expert, dense = [], []
        for i in range(c.expert_layers):
            L = f"{EX}layers.{i}."
            self.expert.append(decoder(L, True))
            dense += [L + "input_layernorm.dense", L + "post_attention_layernorm.dense"]
        self.ada_dense = stacked(dense + [EX + "norm.dense"], True)    # every adaptive norm's dense(cond), stacked

    _LINEAR_SLOTS = ("qkv", "out", "fc1", "fc2", "o", "gate_up", "down")

    def _named_parts(self):
        """(name, object) of everything `save()` stores: TcLinear objects and plain tensors."""
        yield "patch_embed", self.patch_embed
        yield "pos_emb", self.pos_emb
        for group, layers in (("vision", self.vision), ("prefix", self.prefix), ("expert", self.expert)):
            for i, L in enumerate(layers):
                for k, v in L.items():
                    yield f"{group}.{i}.{k}", v
        for k in ("post_ln_w", "post_ln_b", "projector", "embed_tokens", "action_in", "action_out", "time_mlp_in",
                  "time_mlp_out", "ada_dense"):
            yield k, getattr(self, k)

    def _export(self):
        """(tensors, meta) of the prepared model: what `save` writes and `_from_prepared` reads.  The tensors are
        the model's own, not copies."""
        tensors, linears = {}, {}
        for name, obj in self._named_parts():
            if isinstance(obj, TcLinear):
                if obj.rowmajor:
                    tensors[name + ".codes"] = obj.b
                    tensors[name + ".scale_atoms"] = obj.sf
                else:
                    tensors[name + ".image"] = obj.b
                if obj.bias is not None:
                    tensors[name + ".bias"] = obj.bias
                linears[name] = {"N": obj.N, "K": obj.K, "global_scale": obj.g,
                                 "form": "rowmajor" if obj.rowmajor else "tiled"}
            else:
                tensors[name] = obj
        cfgd = {k: getattr(self.cfg, k) for k in self.cfg.__dataclass_fields__}
        return tensors, {"kind": "pi05", "config": cfgd, "linears": linears}

    def save(self, path):
        """Write the prepared model (4-bit operands in the form each linear runs in, bf16 tables) to a container file."""
        tensors, meta = self._export()
        return weights.save_container(path, tensors, meta)

    @classmethod
    def sharing_weights(cls, other, **kw):
        """A second pipeline over `other`'s weights (the same device tensors, no copy) with buffers, KV cache,
        split-K and attention scratch of its own: two such pipelines can run at the same time on two streams of
        one GPU (every kernel's scratch is per pipeline, split-K launches are cooperative launches)."""
        kw.setdefault("pdl", other.launch_flags == ops.FLAG_PDL)
        return cls(other.cfg, other.device, _prepared=other._export(), **kw)

    def _from_prepared(self, prepared):
        tensors, meta = prepared
        lins = meta["linears"]

        def part(name):
            if name in lins:
                e = lins[name]
                if e.get("form", "tiled") == "rowmajor":
                    return TcLinear(tensors[name + ".codes"], e["global_scale"], e["N"], e["K"], tensors.get(name + ".bias"),
                                    sf=tensors[name + ".scale_atoms"])
                return TcLinear(tensors[name + ".image"], e["global_scale"], e["N"], e["K"], tensors.get(name + ".bias"))
            return tensors[name]

        c = self.cfg
        self.patch_embed, self.pos_emb = part("patch_embed"), part("pos_emb")
        self.vision = [{k: part(f"vision.{i}.{k}") for k in ("ln1_w", "ln1_b", "qkv", "out", "ln2_w", "ln2_b", "fc1", "fc2")}
                       for i in range(c.vision_layers)]
        self.prefix = [{k: part(f"prefix.{i}.{k}") for k in ("qkv", "o", "gate_up", "down", "in_norm", "post_norm")}
                       for i in range(c.prefix_layers)]
        self.expert = [{k: part(f"expert.{i}.{k}") for k in ("qkv", "o", "gate_up", "down")}
                       for i in range(c.expert_layers)]
        for k in ("post_ln_w", "post_ln_b", "projector", "embed_tokens", "action_in", "action_out", "time_mlp_in",
                  "time_mlp_out", "ada_dense"):
            setattr(self, k, part(k))

    # ------------------------------------------------------------------ buffers
    def _alloc(self):
        c, d, P = self.cfg, self.device, self.cfg.pieces
        bf = torch.bfloat16
        T = c.num_images * c.image_tokens
        vw = c.vision_width
        S = c.prefix_len
        A = c.action_horizon
        ew = c.expert_width
        self.cache = torch.zeros((c.prefix_layers, 2, c.max_seq, c.head_dim), dtype=bf, device=d)
        self.b = dict(
            # vision
            patches=torch.zeros((T, self.patch_k), dtype=bf, device=d), q_patch=QuantBuf(T, self.patch_k, P, d, tiled=False),
            vh=torch.empty((T, vw), dtype=bf, device=d), vy=torch.empty((T, vw), dtype=bf, device=d),
            q_v=QuantBuf(T, vw, P, d, tiled=False), v_qkv=torch.empty((T, 3 * vw), dtype=bf, device=d),
            v_attn=torch.empty((T, vw), dtype=bf, device=d),
            v_fc1=torch.empty((T, c.vision_mlp), dtype=bf, device=d), q_vmlp=QuantBuf(T, c.vision_mlp, P, d, tiled=False),
            # prefix
            ph=torch.empty((S, c.width), dtype=bf, device=d), py=torch.empty((S, c.width), dtype=bf, device=d),
            q_p=QuantBuf(S, c.width, P, d), q_pqkv=QuantBuf(S, c.width, P, d, tiled=False), p_q=torch.empty((S, c.q_dim), dtype=bf, device=d),
            q_pattn=QuantBuf(S, c.q_dim, P, d, tiled=False), p_gu=torch.empty((S, 2 * c.mlp), dtype=bf, device=d),
            q_pmlp=QuantBuf(S, c.mlp, P, d), pos_prefix=torch.arange(S, dtype=torch.int32, device=d),
            # expert
            x_t=torch.zeros((A, c.action_dim), dtype=torch.float32, device=d),
            x_bf=torch.zeros((A, c.action_dim), dtype=bf, device=d), q_act=QuantBuf(A, c.action_dim, P, d, tiled=False),
            eh=torch.empty((A, ew), dtype=bf, device=d), ey=torch.empty((A, ew), dtype=bf, device=d),
            q_e=QuantBuf(A, ew, P, d, tiled=False), e_q=torch.empty((A, c.q_dim), dtype=bf, device=d),
            q_eattn=QuantBuf(A, c.q_dim, P, d, tiled=False), e_gu=torch.empty((A, 2 * c.expert_mlp), dtype=bf, device=d),
            q_emlp=QuantBuf(A, c.expert_mlp, P, d, tiled=False), v_out=torch.empty((A, c.action_dim), dtype=torch.float32, device=d),
            pos_suffix=torch.arange(S, S + A, dtype=torch.int32, device=d),
        )
        for _, obj in self._named_parts():
            if isinstance(obj, TcLinear):
                obj.ws = self.workspace
        # additive attention bias per key (0 or the reference's mask value) over the cache rows
        self.key_bias = torch.zeros((c.max_seq,), dtype=bf, device=d)
        # scratch of the attention kernel (partial results of the key tiles), sized for the largest call
        lib = _lib.load()
        hd_v = c.vision_width // c.vision_heads
        need = max(lib.tpb200_attention_workspace_size(S * c.heads, S, c.head_dim, 1),
                   lib.tpb200_attention_workspace_size(A * c.heads, S + A, c.head_dim, 1),
                   lib.tpb200_attention_workspace_size(c.image_tokens, c.image_tokens, hd_v, c.num_images * c.vision_heads))
        self.attn_ws = torch.empty(int(need), dtype=torch.uint8, device=d)
        self.tokens = torch.zeros((c.text_len,), dtype=torch.long, device=d)
        self.images = torch.zeros((c.num_images, c.image_size, c.image_size, 3), dtype=torch.uint8, device=d)
        self.noise = torch.zeros((A, c.action_dim), dtype=torch.float32, device=d)
        self.actions = torch.zeros((A, c.action_dim), dtype=torch.float32, device=d)

    # ------------------------------------------------------------------ stages
    def set_valid(self, image_valid=None, prompt_len=None):
        """Declare which prefix tokens exist: `image_valid[i]` per camera, and the number of prompt tokens
        before the padding.  Updates the position ids (`cumsum(valid) - 1`; action tokens continue at
        `sum(valid)`) and the additive key bias in place, so a captured graph picks them up on its next replay."""
        c = self.cfg
        image_valid = [True] * c.num_images if image_valid is None else [bool(v) for v in image_valid]
        prompt_len = c.text_len if prompt_len is None else int(prompt_len)
        if len(image_valid) != c.num_images or not 0 <= prompt_len <= c.text_len:
            raise TurboPiError("set_valid: one flag per camera and 0 <= prompt_len <= text_len")
        key = (tuple(image_valid), prompt_len)
        if getattr(self, "_valid_key", None) == key:       # the same mask as last time: the device tables stand
            return
        valid = torch.cat([torch.full((c.image_tokens,), v) for v in image_valid] + [torch.arange(c.text_len) < prompt_len])
        if not bool(valid.any()):
            raise TurboPiError("set_valid: at least one prefix token must be valid")
        pos = (torch.cumsum(valid.long(), 0) - 1).clamp_min(0)
        first = int(valid.sum())
        S, A = c.prefix_len, c.action_horizon
        bias = torch.zeros(c.max_seq, dtype=torch.float32)
        bias[:S][~valid] = -2.3819763e38                      # the reference's mask value (pi0_pytorch.py:185-188)
        self.b["pos_prefix"].copy_(pos.to(torch.int32))
        self.b["pos_suffix"].copy_(torch.arange(first, first + A, dtype=torch.int32))
        self.key_bias.copy_(bias.to(torch.bfloat16))
        self.valid = valid
        self._valid_key = key

    def _attention(self, q, k, v, out):
        """q [L, H*D] -> softmax(q k^T / sqrt(D) + key bias) v, all heads sharing one K/V head.  Prefix
        tokens see every valid prefix token, action tokens see the valid prefix and each other.  The
        (token, head) pairs are rows of one [L * H, D] problem for the tensor-core kernel."""
        c = self.cfg
        L = q.shape[0]
        ops.attention(q.view(L * c.heads, c.head_dim), k, v, out.view(L * c.heads, c.head_dim), c.head_dim ** -0.5,
                      self.key_bias, self.attn_ws)

    def _attention_to_operand(self, q, k, v, quant):
        """The same attention, its result written only as the operand of the output projection that follows
        (the merge kernel quantises each token's H * D row itself: no bf16 round trip, no row-kernel launch)."""
        c = self.cfg
        L = q.shape[0]
        ops.attention(q.view(L * c.heads, c.head_dim), k, v, None, c.head_dim ** -0.5, self.key_bias, self.attn_ws,
                      quant=quant, rows_per_token=c.heads)

    def vision_tower(self):
        c, b = self.cfg, self.b
        T, vw = c.num_images * c.image_tokens, c.vision_width
        n = c.image_size // c.patch
        img = self.images.float().div_(127.5).sub_(1.0)                               # [-1, 1]
        pt = img.view(c.num_images, n, c.patch, n, c.patch, 3).permute(0, 1, 3, 5, 2, 4).reshape(T, -1)   # (c, i, j)
        b["patches"][:, :pt.shape[1]].copy_(pt)
        rowop(_lib.ROW_NONE, b["patches"], self.patch_k, b["q_patch"])
        self.patch_embed(b["q_patch"], b["vh"])
        b["vh"].view(c.num_images, c.image_tokens, vw).add_(self.pos_emb)
        hd = vw // c.vision_heads
        first = True
        for L in self.vision:
            if first:
                rowop(_lib.ROW_LAYERNORM, b["vh"], vw, b["q_v"], w0=L["ln1_w"], w1=L["ln1_b"], eps=c.eps)
                first = False
            else:
                rowop(_lib.ROW_LAYERNORM, b["vy"], vw, b["q_v"], res_in=b["vh"], h_out=b["vh"], w0=L["ln1_w"],
                      w1=L["ln1_b"], eps=c.eps)
            L["qkv"](b["q_v"], b["v_qkv"])
            qkv = b["v_qkv"].view(c.num_images, c.image_tokens, 3, c.vision_heads, hd).permute(2, 0, 3, 1, 4)
            ops.attention(qkv[0], qkv[1], qkv[2],
                          b["v_attn"].view(c.num_images, c.image_tokens, c.vision_heads, hd).permute(0, 2, 1, 3),
                          hd ** -0.5, None, self.attn_ws)
            rowop(_lib.ROW_NONE, b["v_attn"], vw, b["q_v"])
            L["out"](b["q_v"], b["vy"])
            rowop(_lib.ROW_LAYERNORM, b["vy"], vw, b["q_v"], res_in=b["vh"], h_out=b["vh"], w0=L["ln2_w"], w1=L["ln2_b"],
                  eps=c.eps)
            L["fc1"](b["q_v"], b["v_fc1"], ACT_GELU)
            rowop(_lib.ROW_NONE, b["v_fc1"], c.vision_mlp, b["q_vmlp"])
            L["fc2"](b["q_vmlp"], b["vy"])
        rowop(_lib.ROW_LAYERNORM, b["vy"], vw, b["q_v"], res_in=b["vh"], h_out=b["vh"], w0=self.post_ln_w,
              w1=self.post_ln_b, eps=c.eps)
        self.projector(b["q_v"], b["ph"][:T])                                          # image tokens of the prefix

    def prefix_pass(self):
        c, b = self.cfg, self.b
        T, S = c.num_images * c.image_tokens, c.prefix_len
        b["ph"][T:].copy_(self.embed_tokens[self.tokens] * math.sqrt(c.width))
        first = True
        for l, L in enumerate(self.prefix):
            if first:
                rowop(_lib.ROW_RMSNORM, b["ph"], c.width, b["q_pqkv"], w0=L["in_norm"], eps=c.eps)
                first = False
            else:
                rowop(_lib.ROW_RMSNORM, b["py"], c.width, b["q_pqkv"], res_in=b["ph"], h_out=b["ph"], w0=L["in_norm"],
                      eps=c.eps)
            L["qkv"].qkv(b["q_pqkv"], b["p_q"], self.cache[l, 0], self.cache[l, 1], b["pos_prefix"], self.cos, self.sin,
                         c.q_dim)
            self._attention_to_operand(b["p_q"], self.cache[l, 0, :S], self.cache[l, 1, :S], b["q_pattn"])
            L["o"](b["q_pattn"], b["py"])
            rowop(_lib.ROW_RMSNORM, b["py"], c.width, b["q_p"], res_in=b["ph"], h_out=b["ph"], w0=L["post_norm"],
                  eps=c.eps)
            # GELU(gate) * up rides in the row kernel: in the GEMM's epilogue (ACT_GEGLU) it would sit between
            # the accumulator reads of a 128 x 256 tile and hold up the next tile's MMAs
            L["gate_up"](b["q_p"], b["p_gu"])
            rowop(_lib.ROW_GELU_MUL, b["p_gu"], c.mlp, b["q_pmlp"])
            L["down"](b["q_pmlp"], b["py"])

    def _ada_modulation(self, num_steps):
        """adarms_cond per step and every adaptive norm's (scale, shift, gate): [steps, n_norms, 3, width]
        (pi0_pytorch.py:817-839; GemmaRMSNorm.dense, modeling_gemma.py:96-103)."""
        c, d = self.cfg, self.device
        ew = c.expert_width
        if num_steps not in self._time_emb:      # host-side constants: made once, outside any graph capture
            dt = -1.0 / num_steps
            ts = torch.tensor([1.0 + i * dt for i in range(num_steps)], dtype=torch.float32)
            self._time_emb[num_steps] = sinusoidal_time_embedding(ts, ew).to(torch.bfloat16).to(d)
        emb = self._time_emb[num_steps]
        qb = QuantBuf(num_steps, ew, c.pieces, d, tiled=False)
        t1 = torch.empty((num_steps, ew), dtype=torch.bfloat16, device=d)
        rowop(_lib.ROW_NONE, emb, ew, qb)
        self.time_mlp_in(qb, t1, ACT_SILU)
        rowop(_lib.ROW_NONE, t1, ew, qb)
        self.time_mlp_out(qb, t1, ACT_SILU)
        rowop(_lib.ROW_NONE, t1, ew, qb)
        mod = torch.empty((num_steps, self.n_norms * 3 * ew), dtype=torch.bfloat16, device=d)
        self.ada_dense(qb, mod)
        return mod.view(num_steps, self.n_norms, 3, ew)

    def denoise_step(self, mod, dt):
        """One Euler step: v = expert(x_t | cache); x_t += dt * v."""
        c, b = self.cfg, self.b
        S, A, ew = c.prefix_len, c.action_horizon, c.expert_width
        b["x_bf"].copy_(b["x_t"])
        rowop(_lib.ROW_NONE, b["x_bf"], c.action_dim, b["q_act"])
        self.action_in(b["q_act"], b["eh"])
        prev_gate = None
        for l, L in enumerate(self.expert):
            m_in, m_post = mod[2 * l], mod[2 * l + 1]
            if prev_gate is None:
                rowop(_lib.ROW_ADARMS, b["eh"], ew, b["q_e"], w0=m_in[0], w1=m_in[1], eps=c.eps)
            else:
                rowop(_lib.ROW_ADARMS, b["ey"], ew, b["q_e"], res_in=b["eh"], gate=prev_gate, h_out=b["eh"], w0=m_in[0],
                      w1=m_in[1], eps=c.eps)
            L["qkv"].qkv(b["q_e"], b["e_q"], self.cache[l, 0, S:], self.cache[l, 1, S:], b["pos_suffix"], self.cos,
                         self.sin, c.q_dim)
            self._attention_to_operand(b["e_q"], self.cache[l, 0, :S + A], self.cache[l, 1, :S + A], b["q_eattn"])
            L["o"](b["q_eattn"], b["ey"])
            rowop(_lib.ROW_ADARMS, b["ey"], ew, b["q_e"], res_in=b["eh"], gate=m_in[2], h_out=b["eh"], w0=m_post[0],
                  w1=m_post[1], eps=c.eps)
            L["gate_up"](b["q_e"], b["e_gu"])
            rowop(_lib.ROW_GELU_MUL, b["e_gu"], c.expert_mlp, b["q_emlp"])
            L["down"](b["q_emlp"], b["ey"])
            prev_gate = m_post[2]
        m_f = mod[2 * c.expert_layers]
        rowop(_lib.ROW_ADARMS, b["ey"], ew, b["q_e"], res_in=b["eh"], gate=prev_gate, h_out=b["eh"], w0=m_f[0], w1=m_f[1],
              eps=c.eps)
        self.action_out(b["q_e"], b["v_out"])
        b["x_t"].add_(b["v_out"], alpha=dt)

    def _modulation(self, num_steps):
        """The adaptive norms' (scale, shift, gate) for every step of an `num_steps` schedule.  They depend on
        the schedule and the weights only, not on the observation (the reference precomputes the per-step
        conditioning vectors for its graphs too: pi0_pytorch.py:770-839), so they are computed once per schedule -- by
        the warm-up pass that precedes a capture -- and stay out of the per-inference graph."""
        mod = self._mod.get(num_steps)
        if mod is None:
            if torch.cuda.is_current_stream_capturing():
                raise TurboPiError("the modulation table of a new schedule must be built before the capture")
            mod = self._mod[num_steps] = self._ada_modulation(num_steps)
        return mod

    def denoise_loop(self, num_steps):
        mod = self._modulation(num_steps)
        self.b["x_t"].copy_(self.noise)
        dt = -1.0 / num_steps
        for i in range(num_steps):
            self.denoise_step(mod[i], dt)
        self.actions.copy_(self.b["x_t"])

    def forward(self, num_steps):
        with ops.launch_flags(self.launch_flags):
            self.vision_tower()
            self.prefix_pass()
            self.denoise_loop(num_steps)

    # ------------------------------------------------------------------ public API
    def capture(self, num_steps):
        """Capture vision + prefix + the whole denoise loop as one CUDA graph."""
        side = torch.cuda.Stream(device=self.device)
        with torch.cuda.stream(side):
            self.forward(num_steps)            # warm-up: attribute setup, allocator pools
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            self.forward(num_steps)
        self._graph, self._graph_steps = g, num_steps

    @torch.no_grad()
    def infer(self, images_u8, tokens, noise, num_steps=10, use_graph=True, image_valid=None, prompt_len=None):
        """images_u8 [num_images, H, W, 3] uint8, tokens [text_len] int64, noise [horizon, action_dim] fp32
        (host or device tensors); `image_valid` / `prompt_len` as in `set_valid` (default: everything valid).
        Returns the device tensor of actions [horizon, action_dim] fp32."""
        if image_valid is not None or prompt_len is not None or not bool(self.valid.all()):
            self.set_valid(image_valid, prompt_len)
        self.images.copy_(images_u8, non_blocking=True)
        self.tokens.copy_(tokens, non_blocking=True)
        self.noise.copy_(noise, non_blocking=True)
        if use_graph:
            if self._graph is None or self._graph_steps != num_steps:
                self.capture(num_steps)
            self._graph.replay()
        else:
            self.forward(num_steps)
        return self.actions
