"""Pi0.5-shaped inference pipeline on the turbopi_b200 kernels.

SigLIP-So400m/14 vision tower -> Gemma-2B prefix (image + text tokens, fills the KV cache) ->
Gemma-300M action expert running N flow-matching Euler steps over 50 action tokens against that
cache (`PI0Pytorch.sample_actions`, openpi/src/openpi/models_pytorch/pi0_pytorch.py:876-937;
cached denoise step :524-654; adaptive RMSNorm / gated residual / MLP,
transformers_replace/models/gemma/modeling_gemma.py:49-129,212-230).

Every linear layer runs as NVFP4 weights x bf16 activations on the tcgen05 GEMM (activations
carried as residual e2m1 pieces); norms, residuals and GELU*up are the fused row kernels that
write the next GEMM's operand directly; Q/K/V + RoPE + KV-cache append is the GEMM's fused
epilogue.  Attention itself is torch's scaled_dot_product_attention for now.  All buffers are
allocated once, so the whole inference (or just the denoise loop) replays as ONE CUDA graph.
Weights are random-initialised (there is no checkpoint to load here).
"""
import ctypes
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _lib, ops
from ._lib import ACT_GELU, ACT_NONE, ACT_SILU
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
    an fp32 global scale).  `raw` keeps the reference-layout codes / scale bytes for dequantisation."""

    def __init__(self, weight, bias=None, row_perm=None, keep_raw=False):
        N, K = weight.shape
        packed, scales, g = quantize_nvfp4_two_level(weight, 16)
        self.N, self.K, self.g = N, K, g
        if keep_raw:
            self.raw = (packed.clone(), scales.clone(), g)
        if row_perm is not None:
            packed, scales = packed[row_perm], scales[row_perm]
        pitch = ops.packed_pitch(K)
        b = torch.zeros((N, pitch), dtype=torch.uint8, device=weight.device)
        b[:, :K // 2] = packed
        # the GEMM streams the tiled image; the row-major operand is only its source
        self.b = ops.tile_weights(b, ops.swizzle_scales(scales.contiguous()), N, K)
        self.bias = None if bias is None else bias.float().contiguous()

    # split-K scratch shared by every linear of a device (the model runs them one after another)
    _workspaces = {}

    @classmethod
    def workspace(cls, device):
        key = str(device)
        if key not in cls._workspaces:
            cls._workspaces[key] = ops.gemm_workspace(device)
        return cls._workspaces[key]

    def __call__(self, q, out, activation=ACT_NONE, M=None):
        M = q.M if M is None else M
        p = ops._ptr
        args = _lib.GemmArgs(a_packed=p(q.packed), a_pieces=q.pieces, a_row_scale=p(q.row_scale), b_packed=p(self.b),
                             alpha=float(self.g), bias=p(self.bias), activation=int(activation), out=p(out),
                             out_dtype=ops._dt(out), ldo=out.stride(0), M=M, N=self.N, K=self.K,
                             layout=ops.OPERANDS_TILED)
        ops._gemm_ex(args, out.device, self.workspace(out.device))
        return out

    def qkv(self, q, q_out, k_rows, v_rows, positions, cos, sin, q_dim, M=None):
        M = q.M if M is None else M
        p = ops._ptr
        args = _lib.GemmArgs(a_packed=p(q.packed), a_pieces=q.pieces, a_row_scale=p(q.row_scale), b_packed=p(self.b),
                             alpha=float(self.g), M=M, N=self.N, K=self.K, layout=ops.OPERANDS_TILED,
                             qkv_q_out=p(q_out), qkv_ldq=q_out.stride(0), qkv_q_dim=q_dim, qkv_k_rows=p(k_rows),
                             qkv_v_rows=p(v_rows), qkv_positions=p(positions), qkv_rope_cos=p(cos), qkv_rope_sin=p(sin))
        ops._gemm_ex(args, q_out.device, self.workspace(q_out.device))
        return q_out


def sinusoidal_time_embedding(t, dim, min_period=4e-3, max_period=4.0):
    """openpi/src/openpi/models_pytorch/pi0_pytorch.py:53-70 (float64)."""
    frac = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float64)
    period = min_period * (max_period / min_period) ** frac
    ang = (1.0 / period * 2 * math.pi)[None, :] * t.to(torch.float64)[:, None]
    return torch.cat([torch.sin(ang), torch.cos(ang)], dim=1)


class Pi05:
    """Random-init Pi0.5-shaped model; `infer(images_u8, tokens, noise, num_steps)` -> actions [50, 32]."""

    def __init__(self, cfg: Pi05Config, device, seed=0, keep_raw=False, pdl=True):
        self.cfg, self.device = cfg, device
        # programmatic dependent launch across the GEMM / row-kernel chain: each kernel's launch and set-up
        # overlap the tail of the one before it
        self.launch_flags = ops.FLAG_PDL if pdl else ops.FLAG_NONE
        g = torch.Generator(device=device).manual_seed(seed)
        self.keep_raw = keep_raw

        def W(n, k, std=0.02):
            return torch.randn(n, k, generator=g, device=device) * std

        def Bv(n, std=0.02):
            return torch.randn(n, generator=g, device=device) * std

        def lin(n, k, bias=False, perm=None):
            return TcLinear(W(n, k), Bv(n) if bias else None, perm, keep_raw)

        def nw(n):   # norm parameters: small random values so that the norms are not the identity
            return (torch.randn(n, generator=g, device=device) * 0.1).to(torch.bfloat16)

        c = cfg
        vw, pk = c.vision_width, 3 * c.patch * c.patch
        self.patch_k = (pk + 15) // 16 * 16
        wp = torch.zeros(vw, self.patch_k, device=device)
        wp[:, :pk] = W(vw, pk)
        self.patch_embed = TcLinear(wp, Bv(vw), None, keep_raw)
        self.pos_emb = (torch.randn(c.image_tokens, vw, generator=g, device=device) * 0.02).to(torch.bfloat16)
        self.vision = []
        for _ in range(c.vision_layers):
            self.vision.append(dict(
                ln1_w=(1.0 + nw(vw).float()).to(torch.bfloat16), ln1_b=nw(vw),
                qkv=lin(3 * vw, vw, True), out=lin(vw, vw, True),
                ln2_w=(1.0 + nw(vw).float()).to(torch.bfloat16), ln2_b=nw(vw),
                fc1=lin(c.vision_mlp, vw, True), fc2=lin(vw, c.vision_mlp, True)))
        self.post_ln_w, self.post_ln_b = (1.0 + nw(vw).float()).to(torch.bfloat16), nw(vw)
        self.projector = lin(c.width, vw, True)

        perm = ops.qkv_tile_permutation(c.q_dim).to(device)
        self.embed_tokens = (torch.randn(c.vocab, c.width, generator=g, device=device) * 0.02).to(torch.bfloat16)
        self.prefix = []
        for _ in range(c.prefix_layers):
            self.prefix.append(dict(
                in_norm=nw(c.width), qkv=lin(c.q_dim + 2 * c.head_dim, c.width, False, perm),
                o=lin(c.width, c.q_dim), post_norm=nw(c.width),
                gate_up=lin(2 * c.mlp, c.width), down=lin(c.width, c.mlp)))

        ew = c.expert_width
        self.action_in = lin(ew, c.action_dim, True)
        self.action_out = lin(c.action_dim, ew, True)
        self.time_mlp_in = lin(ew, ew, True)
        self.time_mlp_out = lin(ew, ew, True)
        self.n_norms = 2 * c.expert_layers + 1
        self.ada_dense = lin(self.n_norms * 3 * ew, ew, True)       # every adaptive norm's dense(cond), stacked
        self.expert = []
        for _ in range(c.expert_layers):
            self.expert.append(dict(qkv=lin(c.q_dim + 2 * c.head_dim, ew, False, perm), o=lin(ew, c.q_dim),
                                    gate_up=lin(2 * c.expert_mlp, ew), down=lin(ew, c.expert_mlp)))

        self.cos, self.sin = ops.rope_tables(c.max_seq, c.head_dim, device=device)
        self._alloc()
        self._graph = None
        self._graph_steps = None
        self._time_emb = {}

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
            patches=torch.zeros((T, self.patch_k), dtype=bf, device=d), q_patch=QuantBuf(T, self.patch_k, P, d),
            vh=torch.empty((T, vw), dtype=bf, device=d), vy=torch.empty((T, vw), dtype=bf, device=d),
            q_v=QuantBuf(T, vw, P, d), v_qkv=torch.empty((T, 3 * vw), dtype=bf, device=d),
            v_attn=torch.empty((T, vw), dtype=bf, device=d),
            v_fc1=torch.empty((T, c.vision_mlp), dtype=bf, device=d), q_vmlp=QuantBuf(T, c.vision_mlp, P, d),
            # prefix
            ph=torch.empty((S, c.width), dtype=bf, device=d), py=torch.empty((S, c.width), dtype=bf, device=d),
            q_p=QuantBuf(S, c.width, P, d), p_q=torch.empty((S, c.q_dim), dtype=bf, device=d),
            q_pattn=QuantBuf(S, c.q_dim, P, d), p_gu=torch.empty((S, 2 * c.mlp), dtype=bf, device=d),
            q_pmlp=QuantBuf(S, c.mlp, P, d), pos_prefix=torch.arange(S, dtype=torch.int32, device=d),
            # expert
            x_t=torch.zeros((A, c.action_dim), dtype=torch.float32, device=d),
            x_bf=torch.zeros((A, c.action_dim), dtype=bf, device=d), q_act=QuantBuf(A, c.action_dim, P, d),
            eh=torch.empty((A, ew), dtype=bf, device=d), ey=torch.empty((A, ew), dtype=bf, device=d),
            q_e=QuantBuf(A, ew, P, d), e_q=torch.empty((A, c.q_dim), dtype=bf, device=d),
            q_eattn=QuantBuf(A, c.q_dim, P, d), e_gu=torch.empty((A, 2 * c.expert_mlp), dtype=bf, device=d),
            q_emlp=QuantBuf(A, c.expert_mlp, P, d), v_out=torch.empty((A, c.action_dim), dtype=torch.float32, device=d),
            pos_suffix=torch.arange(S, S + A, dtype=torch.int32, device=d),
        )
        self.tokens = torch.zeros((c.text_len,), dtype=torch.long, device=d)
        self.images = torch.zeros((c.num_images, c.image_size, c.image_size, 3), dtype=torch.uint8, device=d)
        self.noise = torch.zeros((A, c.action_dim), dtype=torch.float32, device=d)
        self.actions = torch.zeros((A, c.action_dim), dtype=torch.float32, device=d)

    # ------------------------------------------------------------------ stages
    def _attention(self, q, k, v, out):
        """q [L, H*D] -> softmax(q k^T / sqrt(D)) v, all heads sharing one K/V head; no mask
        (prefix tokens are mutually visible, action tokens see the whole prefix and each other)."""
        c = self.cfg
        L = q.shape[0]
        qh = q.view(L, c.heads, c.head_dim).transpose(0, 1).unsqueeze(0)
        o = F.scaled_dot_product_attention(qh, k[None, None], v[None, None], enable_gqa=True)
        out.view(L, c.heads, c.head_dim).copy_(o[0].transpose(0, 1))

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
            o = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])
            b["v_attn"].view(c.num_images, c.image_tokens, c.vision_heads, hd).copy_(o.transpose(1, 2))
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
                rowop(_lib.ROW_RMSNORM, b["ph"], c.width, b["q_p"], w0=L["in_norm"], eps=c.eps)
                first = False
            else:
                rowop(_lib.ROW_RMSNORM, b["py"], c.width, b["q_p"], res_in=b["ph"], h_out=b["ph"], w0=L["in_norm"],
                      eps=c.eps)
            L["qkv"].qkv(b["q_p"], b["p_q"], self.cache[l, 0], self.cache[l, 1], b["pos_prefix"], self.cos, self.sin,
                         c.q_dim)
            self._attention(b["p_q"], self.cache[l, 0, :S], self.cache[l, 1, :S], b["p_q"])
            rowop(_lib.ROW_NONE, b["p_q"], c.q_dim, b["q_pattn"])
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
        qb = QuantBuf(num_steps, ew, c.pieces, d)
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
            self._attention(b["e_q"], self.cache[l, 0, :S + A], self.cache[l, 1, :S + A], b["e_q"])
            rowop(_lib.ROW_NONE, b["e_q"], c.q_dim, b["q_eattn"])
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

    def denoise_loop(self, num_steps):
        mod = self._ada_modulation(num_steps)
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
    def infer(self, images_u8, tokens, noise, num_steps=10, use_graph=True):
        """images_u8 [num_images, H, W, 3] uint8, tokens [text_len] int64, noise [horizon, action_dim] fp32
        (host or device tensors).  Returns the device tensor of actions [horizon, action_dim] fp32."""
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
