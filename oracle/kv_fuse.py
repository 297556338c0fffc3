"""Fused QKV projection + RoPE + KV-cache append oracle.

Test infrastructure; see oracle/__init__.py.
"""
import numpy as np

from .formats import E2M1_MAGNITUDES, round_to_bf16
from . import nvfp4


def kv_fuse_dequantize(packed, scales, block_size=32):
    """`FusedQKVProjection._dequantize` (openpi/kv_fuse_plugin/python/kv_fuse.py:282-312):
    magnitude[code % 8] * (1 - 2 * (code >= 8)) * scale; code 8 decodes to +0."""
    codes = nvfp4.unpack_codes(packed)
    vals = E2M1_MAGNITUDES[codes % 8] * (1.0 - 2.0 * (codes >= 8).astype(np.float32))
    s = np.repeat(np.asarray(scales, dtype=np.float32), block_size, axis=1)
    return (vals * s).astype(np.float32)


def fused_qkv_fallback(x, wq, sq, wk, sk, wv, sv, k_cache, v_cache, cache_pos,
                       num_kv_heads=1, head_dim=256, block_size=32):
    """`FusedQKVProjection._forward_fallback` (openpi/kv_fuse_plugin/python/kv_fuse.py:257-280):
    Q = x Wq^T returned; K, V rows written in place at cache[:, cache_pos, :, :]
    of caches shaped [B, max_seq, kv_heads, head_dim].  No RoPE.  fp64 accumulate."""
    x = np.asarray(x, dtype=np.float64)
    Wq = kv_fuse_dequantize(wq, sq, block_size).astype(np.float64)
    Wk = kv_fuse_dequantize(wk, sk, block_size).astype(np.float64)
    Wv = kv_fuse_dequantize(wv, sv, block_size).astype(np.float64)
    Q = x @ Wq.T
    K = x @ Wk.T
    V = x @ Wv.T
    B = x.shape[0]
    k_cache[:, cache_pos, :, :] = K.reshape(B, num_kv_heads, head_dim)
    v_cache[:, cache_pos, :, :] = V.reshape(B, num_kv_heads, head_dim)
    return Q


def rope_cos_sin(positions, head_dim=256, theta=10000.0, inv_freq_bf16=True, out_bf16=True):
    """`RotaryEmbedding` (openpi/src/openpi/inference/w4a16_tvm_kv_cache.py:136-162;
    same arithmetic as GemmaRotaryEmbedding.forward,
    openpi/src/openpi/models_pytorch/transformers_replace/models/gemma/modeling_gemma.py:152-166).

    inv_freq = 1 / theta**(2i/d) in fp32, then cast to the model dtype (bf16);
    freqs = pos * inv_freq in fp32; emb = [freqs, freqs]; cos/sin cast to x.dtype.
    Returns (cos, sin) of shape (S, head_dim), float32 values (bf16-representable
    when out_bf16)."""
    i = np.arange(0, head_dim, 2, dtype=np.float32)
    inv_freq = (np.float32(1.0) / np.power(np.float32(theta), i / np.float32(head_dim), dtype=np.float32)
                ).astype(np.float32)
    if inv_freq_bf16:
        inv_freq = round_to_bf16(inv_freq)
    pos = np.asarray(positions, dtype=np.float32)
    freqs = (pos[:, None] * inv_freq[None, :]).astype(np.float32)
    emb = np.concatenate([freqs, freqs], axis=-1)
    cos = np.cos(emb.astype(np.float64)).astype(np.float32)
    sin = np.sin(emb.astype(np.float64)).astype(np.float32)
    if out_bf16:
        cos, sin = round_to_bf16(cos), round_to_bf16(sin)
    return cos, sin


def rotate_half(x):
    """modeling_gemma.py:169-173."""
    h = x.shape[-1] // 2
    return np.concatenate([-x[..., h:], x[..., :h]], axis=-1)


def apply_rope_bf16(x, cos, sin):
    """`apply_rotary_pos_emb` in bf16 (modeling_gemma.py:176-197): every product and
    the sum are rounded to bf16, as torch does for bf16 tensors.
    x: (S, heads, d) bf16-valued; cos, sin: (S, d)."""
    x = round_to_bf16(x)
    a = round_to_bf16(x * cos[:, None, :])
    b = round_to_bf16(rotate_half(x) * sin[:, None, :])
    return round_to_bf16(a + b)


def fused_qkv_rope_append(x, w_q, w_k, w_v, cache, layer, positions, cache_pos0,
                          num_heads=8, num_kv_heads=1, head_dim=256, theta=10000.0, cos_sin=None):
    """Prefix-shaped fused projection: the computation of
    `compute_prefix_kv_cache` for one layer's attention inputs
    (openpi/src/openpi/models_pytorch/pi0_pytorch.py:455-473): q/k/v = x W^T rounded
    to bf16, RoPE on q and k, K stored post-RoPE and V raw.

    `w_*` are already-dequantised float32 weights [out, in]; `cache` is the
    StaticKVCache buffer [layers, 2, max_seq, head_dim] (batch = kv heads = 1 of
    openpi/src/openpi/modules/static_vlm.py:32-62), written in place at rows
    cache_pos0 .. cache_pos0+S-1 of `layer`.  Returns Q (S, heads*d) bf16-valued
    and the exact (unrounded) pre-RoPE fp64 Q, K, V for tolerance checks."""
    xb = round_to_bf16(x).astype(np.float64)
    S = xb.shape[0]
    q = xb @ np.asarray(w_q, dtype=np.float64).T
    k = xb @ np.asarray(w_k, dtype=np.float64).T
    v = xb @ np.asarray(w_v, dtype=np.float64).T
    cos, sin = cos_sin if cos_sin is not None else rope_cos_sin(positions, head_dim, theta)
    qb = round_to_bf16(q.astype(np.float32)).reshape(S, num_heads, head_dim)
    kb = round_to_bf16(k.astype(np.float32)).reshape(S, num_kv_heads, head_dim)
    vb = round_to_bf16(v.astype(np.float32)).reshape(S, num_kv_heads, head_dim)
    q_rot = apply_rope_bf16(qb, cos, sin)
    k_rot = apply_rope_bf16(kb, cos, sin)
    assert num_kv_heads == 1
    cache[layer, 0, cache_pos0:cache_pos0 + S, :] = k_rot[:, 0, :]
    cache[layer, 1, cache_pos0:cache_pos0 + S, :] = vb[:, 0, :]
    return q_rot.reshape(S, num_heads * head_dim), (q, k, v)
