"""Packed signed-INT4 KV cache codec and q_len=1 GQA decode attention (test oracle, numpy).

Restates ``hybrid_quant/int4_8b_attention.py``: ``int4_quant_dequant`` (:21-29),
``_pack_int4_kv_kernel`` (:56-111; scale :75-76, round-to-nearest-even ``cvt.rni`` :77-84, clamp
:85, nibble order :86-97), ``_int4_decode_attention_kernel`` (:301-402) and
``_decode_attention_mask`` (:569-591).  The pack kernel itself cannot run under the Triton
interpreter (inline PTX), so the codec is pinned through ``int4_quant_dequant``, whose scale,
rounding and clamp are the same expressions; attention is pinned against the reference kernel
run under the interpreter.  Attention here accumulates in float64 and is the "exact" value the
fp32-accumulating kernels are compared with under a tolerance.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def int4_encode(x: np.ndarray, group_size: int):
    """fp32 ``x[..., D]`` -> (codes int8 in [-8,7] [..., D], scale fp32 [..., D/gs]).
    scale = max(absmax/7, 1e-8); code = clamp(rint(x/scale), -8, 7)  (:75-85 == :27-28)."""
    x = np.asarray(x, dtype=F32)
    d = x.shape[-1]
    if d % group_size:
        raise ValueError(f"head_dim={d} must be divisible by group_size={group_size}")
    g = x.reshape(*x.shape[:-1], d // group_size, group_size)
    scale = np.maximum(np.abs(g).max(axis=-1, keepdims=True) / F32(7.0), F32(1.0e-8))
    q = np.clip(np.rint(g / scale), -8.0, 7.0)
    return q.reshape(x.shape).astype(np.int8), scale[..., 0].astype(F32)


def int4_decode(codes: np.ndarray, scale: np.ndarray, group_size: int) -> np.ndarray:
    """codes * scale in fp32 (:336-347)."""
    return (codes.astype(F32) * np.repeat(scale, group_size, axis=-1)).astype(F32)


def int4_pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """byte j = (code[2j] & 15) | (code[2j+1] & 15) << 4  (:86-97)."""
    u = (codes.astype(np.int16) & 15).astype(np.uint8)
    return (u[..., 0::2] | (u[..., 1::2] << 4)).astype(np.uint8)


def int4_unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    """nibble >= 8 -> nibble - 16  (:336-337)."""
    lo = (packed & 15).astype(np.int16)
    hi = (packed >> 4).astype(np.int16)
    both = np.stack([lo, hi], axis=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    return np.where(both >= 8, both - 16, both).astype(np.int8)


def int4_quant_dequant(x: np.ndarray, group_size: int = 64) -> np.ndarray:
    """fp32 fake-quant (:21-29) without the final cast back to the input dtype."""
    q, s = int4_encode(x, group_size)
    return int4_decode(q, s, group_size)


def decode_attention_mask(mask, batch: int, seq_len: int):
    """2-D keep-mask or 4-D bool/additive mask -> additive fp32 [B, L] bias for the single query
    row (:569-591); None stays None."""
    if mask is None:
        return None
    mask = np.asarray(mask)
    if mask.ndim == 4:
        m = mask[:, 0, -1, :seq_len]
        if m.dtype == np.bool_:
            return np.where(m, F32(0.0), F32(-np.inf)).astype(F32)
        return m.astype(F32)
    if mask.ndim == 2:
        m = mask[:, -seq_len:]
        keep = m if m.dtype == np.bool_ else (m != 0)
        return np.where(keep, F32(0.0), F32(-np.inf)).astype(F32)
    raise ValueError(f"INT4 decode attention only supports 2D or 4D attention_mask, got {mask.ndim}D")


def int4_decode_attention(q, k_packed, v_packed, k_scale, v_scale, seq_len: int, group_size: int,
                          bias=None) -> np.ndarray:
    """q [B,Hq,D] (fp32 values of the bf16 query); caches [B,Hkv,cap,D/2] u8 and [B,Hkv,cap,D/gs]
    fp32; only the first ``seq_len`` rows are read.  bias: additive [B, L] (tokens >= L are
    masked out, :351-358).  Returns float64 [B,Hq,D]: softmax2(q.K^T*log2(e)/sqrt(D) + bias) . V with softmax2 taken base 2."""
    q = np.asarray(q, dtype=np.float64)
    bsz, hq, d = q.shape
    hkv = k_packed.shape[1]
    ratio = hq // hkv
    k = int4_decode(int4_unpack_nibbles(k_packed[:, :, :seq_len]), k_scale[:, :, :seq_len], group_size).astype(np.float64)
    v = int4_decode(int4_unpack_nibbles(v_packed[:, :, :seq_len]), v_scale[:, :, :seq_len], group_size).astype(np.float64)
    k = np.repeat(k, ratio, axis=1)  # kv_head = q_head // ratio (:304)
    v = np.repeat(v, ratio, axis=1)
    s = np.einsum("bhd,bhtd->bht", q, k) / np.sqrt(float(d))
    if bias is not None:
        full = np.full((bsz, seq_len), -np.inf)
        l = min(seq_len, bias.shape[-1])
        full[:, :l] = bias[:, :l]
        # the kernel adds the bias to scores already scaled by log2(e)/sqrt(D) and exponentiates
        # with exp2 (:350-361): one unit of bias is a factor of 2, not of e
        s = s + full[:, None, :] * np.log(2.0)
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p = p / p.sum(axis=-1, keepdims=True)
    return np.einsum("bht,bhtd->bhd", p, v)


def int4_prefill_attention(q, k_packed, v_packed, k_scale, v_scale, first_len: int, group_size: int) -> np.ndarray:
    """Causal attention of q [B,Hq,Tq,D] over the packed cache: query i sees rows [0, first_len + i)
    (the reference's unused _int4_prefill_attention_kernel, :160-251, has first_len = 1 through
    causal_len = q_pos + 1).  Returns float64 [B,Hq,Tq,D]."""
    q = np.asarray(q, dtype=np.float64)
    bsz, hq, tq, d = q.shape
    hkv = k_packed.shape[1]
    ratio = hq // hkv
    total = first_len + tq - 1
    k = np.repeat(int4_decode(int4_unpack_nibbles(k_packed[:, :, :total]), k_scale[:, :, :total], group_size).astype(np.float64), ratio, axis=1)
    v = np.repeat(int4_decode(int4_unpack_nibbles(v_packed[:, :, :total]), v_scale[:, :, :total], group_size).astype(np.float64), ratio, axis=1)
    s = np.einsum("bhqd,bhtd->bhqt", q, k) / np.sqrt(float(d))
    allowed = np.arange(total)[None, :] < (first_len + np.arange(tq))[:, None]
    s = np.where(allowed[None, None], s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p = p / p.sum(axis=-1, keepdims=True)
    return np.einsum("bhqt,bhtd->bhqd", p, v)
