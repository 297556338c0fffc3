"""Fused QKV projection with direct KV-cache writes.

Mirrors openpi/kv_fuse_plugin/python/kv_fuse.py: quantize_to_fp4 (sign taken from the input, so small
negatives become code 8), pack_fp4 / unpack_fp4 and FusedQKVProjection with the same buffers
(Wq/Wk/Wv packed + fp32 block-32 scales) and the same forward contract: one token per batch row,
Q returned, K and V rows written in place at cache[:, cache_pos] of fp32 caches shaped
[B, max_seq, kv_heads, head_dim] -- no RoPE, as in the reference kernel
(openpi/kv_fuse_plugin/src/fused_qkv_fp4.cu:282-376).  The three projections run as ONE grouped GEMV
launch whose K/V problems point straight at the cache rows (16 batch rows per launch).
For prefix-shaped inputs with RoPE see turbopi_b200.ops.fused_qkv_rope_append.
"""
from typing import Tuple

import torch
import torch.nn as nn

from . import ops
from .nvfp4_packed import NVFP4_MAX, NVFP4_VALUES, _nearest_index

BLOCK_SIZE = 32


def quantize_to_fp4(tensor: torch.Tensor, block_size: int = BLOCK_SIZE) -> Tuple[torch.Tensor, torch.Tensor]:
    """[N, K] -> (packed uint8 [N, K/2], fp32 scales [N, K/block]); scale = max(|block|, 1e-8) / 6."""
    N, K = tensor.shape
    tb = tensor.float().reshape(N, K // block_size, block_size)
    scales = tb.abs().amax(dim=-1, keepdim=True).clamp(min=1e-8) / NVFP4_MAX
    norm = (tb / scales).reshape(-1)
    q = (_nearest_index(norm.abs()) + (norm < 0).long() * 8).reshape(N, K).to(torch.uint8)
    packed = (q[:, 0::2] & 0xF) | ((q[:, 1::2] & 0xF) << 4)
    return packed.to(torch.uint8), scales.squeeze(-1).float()


def pack_fp4(quantized: torch.Tensor) -> torch.Tensor:
    return ((quantized[:, 0::2] & 0xF) | ((quantized[:, 1::2] & 0xF) << 4)).to(torch.uint8)


def unpack_fp4(packed: torch.Tensor, N: int, K: int) -> torch.Tensor:
    out = torch.zeros(N, K, dtype=torch.uint8, device=packed.device)
    out[:, 0::2] = packed & 0xF
    out[:, 1::2] = (packed >> 4) & 0xF
    return out


class FusedQKVProjection(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, max_seq_len: int = 2048,
                 block_size: int = BLOCK_SIZE):
        super().__init__()
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.max_seq_len, self.block_size = max_seq_len, block_size
        self.q_dim, self.kv_dim = num_heads * head_dim, num_kv_heads * head_dim
        for name in ("Wq_packed", "scale_Wq", "Wk_packed", "scale_Wk", "Wv_packed", "scale_Wv"):
            self.register_buffer(name, None)

    @classmethod
    def from_qkv_weights(cls, Wq, Wk, Wv, num_heads, num_kv_heads, head_dim, max_seq_len=2048, block_size=BLOCK_SIZE):
        layer = cls(Wq.size(1), num_heads, num_kv_heads, head_dim, max_seq_len, block_size)
        with torch.no_grad():
            layer.Wq_packed, layer.scale_Wq = quantize_to_fp4(Wq.float(), block_size)
            layer.Wk_packed, layer.scale_Wk = quantize_to_fp4(Wk.float(), block_size)
            layer.Wv_packed, layer.scale_Wv = quantize_to_fp4(Wv.float(), block_size)
        return layer

    def forward(self, x: torch.Tensor, K_cache: torch.Tensor, V_cache: torch.Tensor, cache_pos: int):
        """x [B, hidden]; caches [B, max_seq, kv_heads, head_dim] fp32, written in place at cache_pos."""
        B = x.shape[0]
        if K_cache.dtype != torch.float32 or not K_cache.is_contiguous() or not V_cache.is_contiguous():
            raise ops.TurboPiError("K/V caches must be contiguous fp32 [B, max_seq, kv_heads, head_dim]")
        x32 = x.float().contiguous()
        Q = torch.empty((B, self.q_dim), dtype=torch.float32, device=x.device)
        for b0 in range(0, B, 16):
            b1 = min(B, b0 + 16)
            xs = x32[b0:b1]
            k_rows = K_cache[b0:b1, cache_pos].view(b1 - b0, self.kv_dim)         # strided views into the caches
            v_rows = V_cache[b0:b1, cache_pos].view(b1 - b0, self.kv_dim)
            probs = [dict(x=xs, weight_packed=self.Wq_packed, weight_scales=self.scale_Wq, out=Q[b0:b1]),
                     dict(x=xs, weight_packed=self.Wk_packed, weight_scales=self.scale_Wk, out=k_rows),
                     dict(x=xs, weight_packed=self.Wv_packed, weight_scales=self.scale_Wv, out=v_rows)]
            ops.GroupedGemv(probs, self.block_size).launch()
        return Q, K_cache, V_cache


def fused_qkv_fp4(x, Wq_packed, scale_Wq, Wk_packed, scale_Wk, Wv_packed, scale_Wv, K_cache, V_cache, hidden_size,
                  num_heads, num_kv_heads, head_dim, cache_pos):
    """Function form with the reference extension's argument list
    (openpi/kv_fuse_plugin/src/fused_qkv_fp4.cu:382-467): returns Q, mutates the caches."""
    layer = FusedQKVProjection(hidden_size, num_heads, num_kv_heads, head_dim, K_cache.shape[1])
    layer.Wq_packed, layer.scale_Wq = Wq_packed.contiguous(), scale_Wq.float().contiguous()
    layer.Wk_packed, layer.scale_Wk = Wk_packed.contiguous(), scale_Wk.float().contiguous()
    layer.Wv_packed, layer.scale_Wv = Wv_packed.contiguous(), scale_Wv.float().contiguous()
    return layer(x, K_cache, V_cache, cache_pos)[0]
