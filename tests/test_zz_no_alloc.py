"""lq_int4_decode_attn_static: decode attention whose split-merge scratch is built into the library,
for callers that cannot allocate device memory themselves (a process whose memory pool already owns
all of HBM, a thread that must not take the allocator's device-wide lock).  Called through the C ABI
and compared with lq_int4_decode_attn on the same inputs, twice in a row because every call reuses
the same built-in array and finds the previous call's contents in it."""
import ctypes as ct

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(m, _lib, q, cache, seq_len, gs, splits, out, workspace=None):
    a = _lib.Int4DecodeArgs()
    a.cache = m._cache_struct(cache, gs)
    a.q = q.data_ptr()
    a.q_stride[0], a.q_stride[1], a.q_stride[2] = q.stride(0), q.stride(1), q.stride(3)
    a.out = out.data_ptr()
    for i in range(3):
        a.out_stride[i] = out.stride(i)
    a.dtype = _lib.dtype_code(q)
    a.q_heads = q.shape[1]
    a.seq_len = seq_len
    a.splits = splits
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    return a


def test_static_scratch_variant_matches_workspace_variant():
    from layer_quant_b200 import _lib
    from layer_quant_b200 import int4_8b_attention as m
    lib = _lib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev).cuda_stream
    gen = torch.Generator(device=dev).manual_seed(7)
    assert lib.lq_int4_static_scratch_bytes() >= 8192 * 130 * 4
    # the second problem is larger than the first, so it meets leftovers of the first in the array
    for b, tlen, splits in ((2, 700, 5), (4, 1500, 8), (4, 1500, 0)):
        hq, hkv, gs = 32, 8, 32
        k = torch.randn((b, hkv, tlen, 128), generator=gen, device=dev).bfloat16()
        v = torch.randn((b, hkv, tlen, 128), generator=gen, device=dev).bfloat16()
        q = torch.randn((b, hq, 1, 128), generator=gen, device=dev).bfloat16()
        cache = m._allocate_layer_cache(b, hkv, 2048, 128, 128 // gs, dev)
        m._pack_kv_into_cache(cache, k, v, torch.arange(tlen, device=dev), gs)
        use = splits or lib.lq_int4_decode_auto_splits(b, hkv, tlen)
        ws = torch.zeros(lib.lq_int4_decode_workspace_bytes(b, hq, hkv, 128, max(use, 1)), dtype=torch.uint8, device=dev)
        want = torch.empty((b, hq, 128), dtype=torch.bfloat16, device=dev)
        a_ref = _args(m, _lib, q, cache, tlen, gs, use, want, ws)
        _lib.check(lib.lq_int4_decode_attn(ct.byref(a_ref), stream))
        for call in range(2):
            got = torch.full((b, hq, 128), float("nan"), dtype=torch.bfloat16, device=dev)
            a = _args(m, _lib, q, cache, tlen, gs, splits, got)
            _lib.check(lib.lq_int4_decode_attn_static(ct.byref(a), stream))
            torch.cuda.synchronize(dev)
            diff = (got.float() - want.float()).abs().max().item()
            scale = want.float().abs().max().item()
            # same kernel, same split count when given explicitly: identical; with the library's own
            # choice of splits the merge order may differ by a rounding of the bf16 output
            assert diff <= (0.0 if splits else 2.0 ** -7 * scale), (b, tlen, splits, call, diff)
    assert _lib.device_status() == 0


def _problem(m, b, hq, hkv, tlen, gs, gen, dev, capacity=None):
    k = torch.randn((b, hkv, tlen, 128), generator=gen, device=dev).bfloat16()
    v = torch.randn((b, hkv, tlen, 128), generator=gen, device=dev).bfloat16()
    q = torch.randn((b, hq, 1, 128), generator=gen, device=dev).bfloat16()
    cache = m._allocate_layer_cache(b, hkv, capacity or tlen, 128, 128 // gs, dev)
    m._pack_kv_into_cache(cache, k, v, torch.arange(tlen, device=dev), gs)
    return q, cache


def test_static_scratch_limits():
    """The edges of the built-in scratch: exactly as many partial results as it holds, the library's own split count
    clamped to fit, a problem too wide for any splitting (one split is always accepted), and an explicit split count
    that is capped by the number of tiles before it is held against the limit."""
    from layer_quant_b200 import _lib
    from layer_quant_b200 import int4_8b_attention as m
    lib = _lib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev).cuda_stream
    gen = torch.Generator(device=dev).manual_seed(11)
    slots = 8192

    def both(q, cache, tlen, splits_static, splits_ref, tol_ulp):
        b, hq = q.shape[0], q.shape[1]
        hkv = cache.k_packed.shape[1]
        ws = torch.zeros(lib.lq_int4_decode_workspace_bytes(b, hq, hkv, 128, max(splits_ref, 1)), dtype=torch.uint8, device=dev)
        want = torch.empty((b, hq, 128), dtype=torch.bfloat16, device=dev)
        _lib.check(lib.lq_int4_decode_attn(ct.byref(_args(m, _lib, q, cache, tlen, 32, splits_ref, want, ws)), stream))
        for _ in range(2):
            got = torch.full((b, hq, 128), float("nan"), dtype=torch.bfloat16, device=dev)
            _lib.check(lib.lq_int4_decode_attn_static(ct.byref(_args(m, _lib, q, cache, tlen, 32, splits_static, got)), stream))
            torch.cuda.synchronize(dev)
            diff = (got.float() - want.float()).abs().max().item()
            assert diff <= tol_ulp * 2.0 ** -7 * want.float().abs().max().item(), (b, hq, tlen, splits_static, diff)

    # exactly 8192 partial results: 8 x 32 heads x 32 splits
    q, cache = _problem(m, 8, 32, 8, 2048, 32, gen, dev)
    both(q, cache, 2048, 32, 32, 0)
    # the library's own choice (4 splits here) does not fit 129 x 16 heads: it is clamped to 3
    b, hq, hkv, tlen = 129, 16, 2, 8192
    assert lib.lq_int4_decode_auto_splits(b, hkv, tlen) * b * hq > slots
    q, cache = _problem(m, b, hq, hkv, tlen, 32, gen, dev)
    both(q, cache, tlen, 0, slots // (b * hq), 0)
    # batch x heads alone exceeds the scratch: one split, no scratch needed; two splits are refused
    q, cache = _problem(m, 300, 32, 8, 200, 32, gen, dev, capacity=256)
    both(q, cache, 200, 0, 1, 0)
    both(q, cache, 200, 1, 1, 0)
    got = torch.empty((300, 32, 128), dtype=torch.bfloat16, device=dev)
    rc = lib.lq_int4_decode_attn_static(ct.byref(_args(m, _lib, q, cache, 200, 32, 2, got)), stream)
    assert rc == _lib.LQ_ERR_WORKSPACE and b"exceed the built-in scratch" in lib.lq_last_error_string()
    # 100 splits asked of a 3-tile context: used as 3, which fits
    q, cache = _problem(m, 64, 32, 8, 130, 32, gen, dev, capacity=256)
    both(q, cache, 130, 100, 3, 0)
    assert _lib.device_status() == 0
