"""Packed INT4 KV cache and fused q_len = 1 GQA decode attention: host-side mirror of the
reference module ``hybrid_quant/int4_8b_attention.py`` (phcool/Layer_Quant) over the sm_100a
library.

=============================================  ==========================================
here                                           reference (int4_8b_attention.py)
=============================================  ==========================================
``Int4KVLayerCache``                           :12-18
``int4_quant_dequant``                         :21-29
``_cache_dict`` / ``_positions``               :405-420
``_allocate_layer_cache`` / ``_ensure_...``    :423-474
``_pack_kv_into_cache``                        :477-515  (one launch for K and V)
``_decode_attention``                          :518-566  (split over the context)
``_decode_attention_mask``                     :569-591
``_forward_fused_int4_kv``                     :628-714  (decode: append fused into attention)
``patch_nemotron_h_attention_int4_kv``         :717-731
``_prefill_attention``                         :114-251  (kernel the reference never calls)
=============================================  ==========================================

The cache tensors have exactly the reference's shapes, dtypes and bit layout.  As in the reference,
prefill attends over the un-quantised K/V with torch SDPA after packing; the reference's unused
``_int4_prefill_attention_kernel`` (:114-251) has its counterpart in ``_prefill_attention`` (causal
attention over the quantised cache), used by the forward only when ``PREFILL_FROM_INT4_CACHE`` is set.
"""
from __future__ import annotations

import ctypes as ct
import math
from dataclasses import dataclass
from types import MethodType

import torch

from . import _lib


@dataclass
class Int4KVLayerCache:
    k_packed: torch.Tensor
    v_packed: torch.Tensor
    k_scale: torch.Tensor
    v_scale: torch.Tensor
    length: int = 0
    # Not in the reference: the same length kept on the device (one int64) once prepare_graph_decode has
    # run; decode steps then read it inside the kernel and advance it on the stream, with no host sync.
    length_counter: torch.Tensor | None = None


def int4_quant_dequant(x: torch.Tensor, group_size: int = 64) -> torch.Tensor:
    """Fake-quantise ``x[..., D]`` to signed INT4 per group of ``group_size`` and back, in torch
    (any device).  Same arithmetic as the cache codec: scale = max(absmax/7, 1e-8),
    code = clamp(round_half_even(x/scale), -8, 7)."""
    d = x.shape[-1]
    if d % group_size != 0:
        raise ValueError(f"head_dim={d} must be divisible by group_size={group_size}")
    g = x.to(torch.float32).unflatten(-1, (d // group_size, group_size))
    scale = (g.abs().amax(dim=-1, keepdim=True) / 7.0).clamp_min(1.0e-8)
    codes = (g / scale).round().clamp(-8.0, 7.0)
    return (codes * scale).flatten(-2).to(x.dtype)


def _cache_dict(past_key_value) -> dict[int, Int4KVLayerCache]:
    caches = getattr(past_key_value, "_int4_kv_layer_caches", None)
    if caches is None:
        caches = {}
        past_key_value._int4_kv_layer_caches = caches
    return caches


def _positions(cache_position, q_len: int, device: torch.device) -> torch.Tensor:
    if cache_position is None:
        return torch.arange(q_len, device=device, dtype=torch.long)
    if cache_position.numel() == q_len:
        return cache_position.to(device=device, dtype=torch.long)
    raise ValueError(f"cache_position has {cache_position.numel()} entries for q_len={q_len}")


def _allocate_layer_cache(batch: int, kv_heads: int, capacity: int, head_dim: int, groups: int,
                          device: torch.device) -> Int4KVLayerCache:
    def u8():
        return torch.empty((batch, kv_heads, capacity, head_dim // 2), device=device, dtype=torch.uint8)

    def f32():
        return torch.empty((batch, kv_heads, capacity, groups), device=device, dtype=torch.float32)

    return Int4KVLayerCache(k_packed=u8(), v_packed=u8(), k_scale=f32(), v_scale=f32())


def _pow2_capacity(required_len: int) -> int:
    return 1 << max(0, math.ceil(math.log2(max(required_len, 1))))


def _ensure_layer_cache(past_key_value, layer_idx: int, batch: int, kv_heads: int, required_len: int, head_dim: int,
                        group_size: int, device: torch.device) -> Int4KVLayerCache:
    """The layer's cache with room for ``required_len`` tokens: created at max(16, next power of
    two), doubled (with a copy of the old rows) when it overflows."""
    caches = _cache_dict(past_key_value)
    cur = caches.get(layer_idx)
    groups = head_dim // group_size
    if cur is None:
        cur = _allocate_layer_cache(batch, kv_heads, max(16, _pow2_capacity(required_len)), head_dim, groups, device)
        caches[layer_idx] = cur
        return cur
    if cur.k_packed.shape[:2] != (batch, kv_heads):
        raise ValueError(
            f"Layer {layer_idx} INT4 cache shape {tuple(cur.k_packed.shape[:2])} "
            f"does not match batch/kv_heads {(batch, kv_heads)}"
        )
    old_cap = cur.k_packed.shape[2]
    if required_len <= old_cap:
        return cur
    grown = _allocate_layer_cache(batch, kv_heads, _pow2_capacity(required_len), head_dim, groups, device)
    for name in ("k_packed", "v_packed", "k_scale", "v_scale"):
        getattr(grown, name)[:, :, :old_cap].copy_(getattr(cur, name))
    grown.length = cur.length
    caches[layer_idx] = grown
    return grown


def _cache_struct(cache: Int4KVLayerCache, group_size: int) -> _lib.Int4Cache:
    _lib.require_cuda(cache.k_packed, cache.v_packed, cache.k_scale, cache.v_scale)
    c = _lib.Int4Cache()
    c.k_packed, c.v_packed = cache.k_packed.data_ptr(), cache.v_packed.data_ptr()
    c.k_scale, c.v_scale = cache.k_scale.data_ptr(), cache.v_scale.data_ptr()
    for i in range(4):
        c.kp_stride[i] = cache.k_packed.stride(i)
        c.vp_stride[i] = cache.v_packed.stride(i)
        c.ks_stride[i] = cache.k_scale.stride(i)
        c.vs_stride[i] = cache.v_scale.stride(i)
    c.batch, c.kv_heads, c.capacity = cache.k_packed.shape[:3]
    c.head_dim = cache.k_packed.shape[3] * 2
    c.group_size = group_size
    if cache.k_scale.shape[3] * group_size != c.head_dim:
        raise ValueError(f"cache holds {cache.k_scale.shape[3]} scale groups per row; group_size={group_size} "
                         f"needs {c.head_dim // max(group_size, 1)}")
    return c


def _required_len(positions: torch.Tensor, cache_position, q_len: int) -> int:
    """max(positions) + 1 as the reference computes it (:667), without the device round trip when the
    positions are known on the host (no cache_position: arange; a CPU cache_position)."""
    if cache_position is None:
        return q_len
    if cache_position.device.type == "cpu":
        return int(cache_position.max()) + 1
    return int(positions.max().item()) + 1


def _pack_kv_into_cache(cache: Int4KVLayerCache, key_states: torch.Tensor, value_states: torch.Tensor,
                        positions: torch.Tensor, group_size: int, *, known_len: int | None = None) -> None:
    """Quantise ``key_states`` / ``value_states`` [B, Hkv, q_len, D] and write them to cache rows
    ``positions`` (int64 [q_len], shared by the batch).  ``known_len`` = max(positions) + 1 when the
    caller already has it (saves the read-back the reference does at :515)."""
    batch, kv_heads, q_len, head_dim = key_states.shape
    if value_states.shape != key_states.shape or value_states.dtype != key_states.dtype:
        raise ValueError("key_states and value_states must agree in shape and dtype")
    dev = _lib.require_cuda(key_states, value_states, positions)
    c = _cache_struct(cache, group_size)
    if (c.batch, c.kv_heads, c.head_dim) != (batch, kv_heads, head_dim):
        raise ValueError(f"cache [{c.batch},{c.kv_heads},*,{c.head_dim}] does not match K/V {tuple(key_states.shape)}")
    positions = positions.to(device=dev, dtype=torch.long).contiguous()
    if positions.numel() != q_len:
        raise ValueError(f"positions has {positions.numel()} entries for q_len={q_len}")
    ks = (ct.c_int64 * 4)(*key_states.stride())
    vs = (ct.c_int64 * 4)(*value_states.stride())
    _lib.check(_lib.lib().lq_int4_kv_append(ct.byref(c), key_states.data_ptr(), ks, value_states.data_ptr(), vs,
                                           _lib.dtype_code(key_states), positions.data_ptr(), q_len, _lib.stream_ptr(dev)))
    cache.length = max(cache.length, known_len if known_len is not None else int(positions.max().item()) + 1)


def _decode_attention_mask(attention_mask: torch.Tensor | None, batch: int, seq_len: int,
                           device: torch.device) -> torch.Tensor | None:
    """Additive fp32 bias [B,1,1,L] for the single query row, from a 4-D (bool or additive) or a
    2-D keep mask; None stays None."""
    if attention_mask is None:
        return None
    if attention_mask.dim() == 4:
        last = attention_mask[:, :, -1:, :seq_len].to(device=device)
        if last.dtype == torch.bool:
            return torch.zeros(last.shape, device=device, dtype=torch.float32).masked_fill_(~last, -float("inf"))
        return last.to(dtype=torch.float32).contiguous()
    if attention_mask.dim() == 2:
        tail = attention_mask[:, -seq_len:].to(device=device)
        keep = tail if tail.dtype == torch.bool else tail != 0
        bias = torch.zeros((batch, 1, 1, seq_len), device=device, dtype=torch.float32)
        return bias.masked_fill_(~keep[:, None, None, :], -float("inf"))
    raise ValueError(f"INT4 decode attention only supports 2D or 4D attention_mask, got {attention_mask.dim()}D")


_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch for the split merge, one per (device, stream), grown on demand.
    The kernel leaves its ticket counters at zero, so the buffer is cleared only when created."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def _decode_args(query_states, cache, seq_len, group_size, mask, k_new=None, v_new=None, splits=0, out=None,
                 seq_len_counter=None):
    """Fill the argument block of ``lq_int4_decode_attn``.  Returns (args, out, tensors the block points to)."""
    batch, n_heads, q_len, head_dim = query_states.shape
    dev = _lib.require_cuda(query_states, mask, k_new, v_new, seq_len_counter)
    if out is None:
        out = torch.empty((batch, n_heads, head_dim), device=dev, dtype=query_states.dtype)
    a = _lib.Int4DecodeArgs()
    a.cache = _cache_struct(cache, group_size)
    if a.cache.batch != batch or a.cache.head_dim != head_dim:
        raise ValueError(f"cache [{a.cache.batch},*,*,{a.cache.head_dim}] does not match query {tuple(query_states.shape)}")
    a.q = query_states.data_ptr()
    a.q_stride[0], a.q_stride[1], a.q_stride[2] = query_states.stride(0), query_states.stride(1), query_states.stride(3)
    a.out = out.data_ptr()
    for i in range(3):
        a.out_stride[i] = out.stride(i)
    a.dtype = _lib.dtype_code(query_states)
    a.q_heads = n_heads
    a.seq_len = seq_len
    if mask is not None:
        a.mask = mask.data_ptr()
        a.mask_stride_b, a.mask_stride_k, a.mask_k_len = mask.stride(0), mask.stride(3), mask.shape[-1]
    if k_new is not None:
        a.k_new, a.v_new = k_new.data_ptr(), v_new.data_ptr()
        for i, ax in enumerate((0, 1, 3)):
            a.k_new_stride[i] = k_new.stride(ax)
            a.v_new_stride[i] = v_new.stride(ax)
    if seq_len_counter is not None:
        if seq_len_counter.dtype != torch.int64 or seq_len_counter.numel() != 1:
            raise TypeError("seq_len_counter must be a one-element int64 CUDA tensor")
        a.seq_len_counter = seq_len_counter.data_ptr()
    l = _lib.lib()
    if splits <= 0:
        splits = l.lq_int4_decode_auto_splits(batch, a.cache.kv_heads, max(seq_len - (1 if k_new is not None else 0), 1))
    a.splits = splits
    ws = None
    if splits > 1:
        need = l.lq_int4_decode_workspace_bytes(batch, n_heads, a.cache.kv_heads, head_dim, splits)
        ws = _workspace(dev, need)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    return a, out, (query_states, cache, mask, k_new, v_new, seq_len_counter, ws, out)


def _launch_decode(query_states, cache, seq_len, group_size, mask, k_new=None, v_new=None, splits=0, out=None):
    a, out, _keep = _decode_args(query_states, cache, seq_len, group_size, mask, k_new, v_new, splits, out)
    _lib.check(_lib.lib().lq_int4_decode_attn(ct.byref(a), _lib.stream_ptr(out.device)))
    return out


class Int4DecodePlan:
    """A decode-attention launch prepared once (not in the reference, which rebuilds its launch every
    step, int4_8b_attention.py:518-566): the argument block is filled here and ``launch()`` is a single
    foreign call on the current stream, reading whatever the bound tensors hold at that time.

    With ``seq_len_counter`` (one-element int64 CUDA tensor) the kernel takes the sequence length from
    the device when it runs; ``seq_len`` then only sizes the launch.  Such a plan can be recorded in a
    CUDA graph once and replayed for every decode step: write the new token's q / k / v into the bound
    tensors, replay, and advance the counter on the stream (``advance_seq_len``).  The caller keeps the
    cache capacity ahead of the counter."""

    def __init__(self, query_states, cache, seq_len, group_size, *, k_new=None, v_new=None, mask=None, splits=0,
                 out=None, seq_len_counter=None):
        if query_states.shape[2] != 1:
            raise ValueError(f"Fused INT4 decode attention expects q_len=1, got {query_states.shape[2]}")
        self.args, self.out, self._keep = _decode_args(query_states, cache, seq_len, group_size, mask, k_new, v_new, splits,
                                                       out, seq_len_counter)
        self._ref = ct.byref(self.args)
        self._fn = _lib.lib().lq_int4_decode_attn
        self.device = self.out.device
        self.seq_len_counter = seq_len_counter

    def launch(self) -> torch.Tensor:
        _lib.check(self._fn(self._ref, _lib.stream_ptr(self.device)))
        return self.out


def advance_seq_len(seq_len_counter: torch.Tensor, inc: int = 1) -> None:
    """``*seq_len_counter += inc`` on the current stream (a one-thread kernel; records into CUDA graphs)."""
    _lib.check(_lib.lib().lq_counter_add(seq_len_counter.data_ptr(), int(inc), _lib.stream_ptr(seq_len_counter.device)))


def _decode_attention(query_states: torch.Tensor, cache: Int4KVLayerCache, seq_len: int, num_key_value_groups: int,
                      group_size: int, attention_mask: torch.Tensor | None = None, *, splits: int = 0) -> torch.Tensor:
    """softmax(q K^T / sqrt(D) [+ mask]) V over cache rows [0, seq_len) for one query token.
    query_states [B, Hq, 1, D] -> [B, Hq, D] in the query's dtype."""
    batch, n_heads, q_len, head_dim = query_states.shape
    if q_len != 1:
        raise ValueError(f"Fused INT4 decode attention expects q_len=1, got {q_len}")
    if n_heads != cache.k_packed.shape[1] * num_key_value_groups:
        raise ValueError(f"{n_heads} query heads != {cache.k_packed.shape[1]} kv heads x {num_key_value_groups}")
    mask = _decode_attention_mask(attention_mask, batch, seq_len, query_states.device)
    return _launch_decode(query_states, cache, seq_len, group_size, mask, splits=splits)


def _append_decode_attention(query_states, key_states, value_states, cache, seq_len, num_key_value_groups, group_size,
                             attention_mask=None, *, splits: int = 0) -> torch.Tensor:
    """Decode step in one launch: quantise the new K/V row [B, Hkv, 1, D] into cache row
    ``seq_len - 1`` and attend over rows [0, seq_len).  Equals ``_pack_kv_into_cache`` followed by
    ``_decode_attention``."""
    batch, n_heads, q_len, head_dim = query_states.shape
    if q_len != 1 or key_states.shape[2] != 1:
        raise ValueError(f"Fused INT4 decode attention expects q_len=1, got {q_len}")
    mask = _decode_attention_mask(attention_mask, batch, seq_len, query_states.device)
    out = _launch_decode(query_states, cache, seq_len, group_size, mask, k_new=key_states, v_new=value_states, splits=splits)
    cache.length = max(cache.length, seq_len)
    return out


# When True, prefill (q_len > 1, no attention_mask) attends the quantised cache, as the reference's unused
# prefill kernel would (:114-251), instead of the un-quantised K / V of the live path (:693-714).
PREFILL_FROM_INT4_CACHE = False


def _prefill_attention(query_states: torch.Tensor, cache: Int4KVLayerCache, num_key_value_groups: int, group_size: int, *,
                       first_len: int = 1, out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of the q_len query positions of ``query_states`` [B, Hq, Tq, D] over cache rows that
    already hold their K / V: position i attends rows [0, first_len + i).  Returns [B, Hq, Tq, D] in the
    query's dtype.  Positional arguments as the reference's ``_prefill_attention`` (:594-625, the launcher of its
    unused ``_int4_prefill_attention_kernel``, :114-251), which is ``first_len = 1``: a prompt from position 0;
    larger values (keyword-only, not in the reference) continue an existing context."""
    batch, n_heads, q_len, head_dim = query_states.shape
    if n_heads != cache.k_packed.shape[1] * num_key_value_groups:
        raise ValueError(f"{n_heads} query heads != {cache.k_packed.shape[1]} kv heads x {num_key_value_groups}")
    dev = _lib.require_cuda(query_states, out)
    if out is None:
        out = torch.empty((batch, n_heads, q_len, head_dim), device=dev, dtype=query_states.dtype)
    a = _lib.Int4PrefillArgs()
    a.cache = _cache_struct(cache, group_size)
    if a.cache.batch != batch or a.cache.head_dim != head_dim:
        raise ValueError(f"cache [{a.cache.batch},*,*,{a.cache.head_dim}] does not match query {tuple(query_states.shape)}")
    a.q, a.out = query_states.data_ptr(), out.data_ptr()
    for i in range(4):
        a.q_stride[i], a.out_stride[i] = query_states.stride(i), out.stride(i)
    a.dtype = _lib.dtype_code(query_states)
    a.q_heads, a.q_len, a.first_len = n_heads, q_len, first_len
    _lib.check(_lib.lib().lq_int4_prefill_attn(ct.byref(a), _lib.stream_ptr(dev)))
    return out


def prepare_graph_decode(past_key_value, max_len: int) -> None:
    """Make the decode steps that follow replayable from a CUDA graph (not in the reference, which
    reads the position back on the host every step, :515 / :667): every layer cache is grown once to
    hold ``max_len`` tokens (no reallocation later) and gets its length as a device counter.  From
    then on a q_len = 1 forward appends at the counter's position, attends over [0, position] and
    advances the counter on the stream; no ``.item()``, no allocation, arguments that stay valid for
    every replay.  ``cache.length`` on the host is no longer advanced; ``sync_graph_decode`` reads it
    back.  A step beyond ``max_len`` is clamped by the kernel and reported by ``lq_device_status``."""
    caches = _cache_dict(past_key_value)
    if not caches:
        raise ValueError("prepare_graph_decode needs the caches of a finished prefill")
    for idx, cur in list(caches.items()):
        batch, kv_heads, cap, half = cur.k_packed.shape
        groups = cur.k_scale.shape[3]
        if cap < max_len:
            cur = _ensure_layer_cache(past_key_value, idx, batch, kv_heads, max_len, 2 * half, (2 * half) // groups,
                                      cur.k_packed.device)
        cur.length_counter = torch.full((1,), cur.length, device=cur.k_packed.device, dtype=torch.int64)
        caches[idx] = cur


def sync_graph_decode(past_key_value) -> None:
    """Copy the device-side lengths back into ``cache.length`` (one read-back per layer cache)."""
    for cur in _cache_dict(past_key_value).values():
        if cur.length_counter is not None:
            cur.length = int(cur.length_counter.item())


def _graph_decode_step(query_states, key_states, value_states, cache, group_size, attention_mask):
    if attention_mask is not None:
        raise NotImplementedError("recorded decode steps take no attention_mask: a mask's length changes every step")
    advance_seq_len(cache.length_counter)  # the new token's position + 1
    capacity = cache.k_packed.shape[2]
    a, out, keep = _decode_args(query_states, cache, capacity, group_size, None, key_states, value_states,
                                seq_len_counter=cache.length_counter)
    _lib.check(_lib.lib().lq_int4_decode_attn(ct.byref(a), _lib.stream_ptr(out.device)))
    return out


def _forward_fused_int4_kv(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                           output_attentions=False, use_cache=False, cache_position=None):
    """Replacement ``forward`` of a Nemotron-H attention mixer (no RoPE in this architecture):
    project, append K/V to the INT4 cache, then fused decode attention (q_len = 1) or torch SDPA
    over the un-quantised K/V (prefill).  Returns (attn_output, None, past_key_value)."""
    if output_attentions or hidden_states.device.type != "cuda" or past_key_value is None:
        return self._int4_kv_original_forward(
            hidden_states=hidden_states, attention_mask=attention_mask, position_ids=position_ids,
            past_key_value=past_key_value, output_attentions=output_attentions, use_cache=use_cache,
            cache_position=cache_position)

    bsz, q_len, _ = hidden_states.size()
    group_size = self._int4_kv_group_size
    if self.head_dim % group_size != 0:
        raise ValueError(f"head_dim={self.head_dim} must be divisible by group_size={group_size}")
    if group_size % 2 != 0:
        raise ValueError(f"group_size={group_size} must be even for INT4 packing")

    def heads(t, n):
        return t.view(bsz, q_len, n, self.head_dim).transpose(1, 2)  # [B, n, q_len, D] view; kernels take strides

    query_states = heads(self.q_proj(hidden_states), self.num_heads)
    key_states = heads(self.k_proj(hidden_states), self.num_key_value_heads)
    value_states = heads(self.v_proj(hidden_states), self.num_key_value_heads)

    graph_cache = _cache_dict(past_key_value).get(self.layer_idx) if q_len == 1 else None
    if graph_cache is not None and graph_cache.length_counter is not None:
        # prepared for recorded decode steps: position = the device-side length, nothing read back
        attn = _graph_decode_step(query_states, key_states, value_states, graph_cache, group_size, attention_mask)
        return self.o_proj(attn.reshape(bsz, 1, -1)), None, past_key_value

    positions = _positions(cache_position, q_len, hidden_states.device)
    required_len = _required_len(positions, cache_position, q_len)
    layer_cache = _ensure_layer_cache(past_key_value, self.layer_idx, bsz, self.num_key_value_heads, required_len,
                                      self.head_dim, group_size, hidden_states.device)

    if q_len == 1:
        attn = _append_decode_attention(query_states, key_states, value_states, layer_cache, required_len,
                                        self.num_key_value_groups, group_size, attention_mask=attention_mask)
        return self.o_proj(attn.reshape(bsz, 1, -1)), None, past_key_value

    _pack_kv_into_cache(layer_cache, key_states, value_states, positions, group_size, known_len=required_len)
    if PREFILL_FROM_INT4_CACHE and attention_mask is None and group_size in (32, 64, 128):
        # contiguous positions ending at required_len - 1 (what _positions hands out for a prompt or a chunk)
        attn = _prefill_attention(query_states, layer_cache, self.num_key_value_groups, group_size, first_len=required_len - q_len + 1)
        return self.o_proj(attn.transpose(1, 2).reshape(bsz, q_len, -1)), None, past_key_value
    k_full = self._int4_kv_repeat_kv(key_states, self.num_key_value_groups)
    v_full = self._int4_kv_repeat_kv(value_states, self.num_key_value_groups)
    causal_mask = attention_mask
    if attention_mask is not None:
        causal_mask = attention_mask[:, :, :, : k_full.shape[-2]]
        query_states, k_full, v_full = query_states.contiguous(), k_full.contiguous(), v_full.contiguous()
    attn = torch.nn.functional.scaled_dot_product_attention(
        query_states, k_full, v_full, attn_mask=causal_mask,
        dropout_p=self.attention_dropout if self.training else 0.0,
        is_causal=causal_mask is None and q_len > 1)
    attn = attn.transpose(1, 2).reshape(bsz, q_len, -1)
    return self.o_proj(attn), None, past_key_value


def patch_nemotron_h_attention_int4_kv(model, group_size: int = 64):
    """Swap the forward of every attention mixer of ``model.backbone.layers`` for the INT4-KV one."""
    remote_module = __import__(model.__class__.__module__, fromlist=["repeat_kv"])
    for layer in model.backbone.layers:
        attn = getattr(layer, "mixer", None)
        if getattr(layer, "block_type", None) != "attention" or attn is None or getattr(attn, "_int4_kv_patched", False):
            continue
        attn._int4_kv_original_forward = attn.forward
        attn._int4_kv_group_size = group_size
        attn._int4_kv_repeat_kv = remote_module.repeat_kv
        attn.forward = MethodType(_forward_fused_int4_kv, attn)
        attn._int4_kv_patched = True
