"""ctypes binding of ``liblayer_quant_b200.so`` (the C ABI in ``include/layer_quant_b200.h``).

PyTorch is used only as the owner of device memory and streams: tensors are handed to the library
as raw pointers plus element strides, kernels are launched on ``torch.cuda.current_stream()``.
There is no CPU path: if the shared library is missing this module raises at first use.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

import os

PKG = Path(__file__).resolve().parent
#: the shared library; LAYER_QUANT_B200_LIB selects another build of it (same ABI), e.g. one compiled with other options
LIB_PATH = Path(os.environ.get("LAYER_QUANT_B200_LIB") or PKG / "liblayer_quant_b200.so")

LQ_OK = 0
LQ_ERR_INVALID_ARGUMENT = -1
LQ_ERR_UNSUPPORTED = -2
LQ_ERR_CUDA = -3
LQ_ERR_WORKSPACE = -4
LQ_ERR_DEVICE_STATUS = -5

LQ_BF16, LQ_F16, LQ_F32 = 0, 1, 2
LQ_MX_LAYOUT_REFERENCE, LQ_MX_LAYOUT_PACKED = 0, 1
(LQ_ROUND_HALF_UP, LQ_ROUND_HALF_EVEN, LQ_ROUND_PHILOX_REF, LQ_ROUND_SUPPLIED, LQ_ROUND_PHILOX_LAYERED,
 LQ_ROUND_SUPPLIED_FIXED, LQ_ROUND_PHILOX_LAYERED4) = range(7)

_DTYPES = {torch.bfloat16: LQ_BF16, torch.float16: LQ_F16, torch.float32: LQ_F32}


class MxState(C.Structure):
    _fields_ = [
        ("q_state", C.c_void_p), ("shared_exp", C.c_void_p), ("micro_exp", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("exp_stride", C.c_int64 * 3), ("micro_stride", C.c_int64 * 3),
        ("batch", C.c_int32), ("heads", C.c_int32), ("dim", C.c_int32), ("dstate", C.c_int32),
        ("format_bits", C.c_int32), ("layout", C.c_int32),
    ]


class Rounding(C.Structure):
    _fields_ = [
        ("mode", C.c_int32), ("layer", C.c_uint32), ("seed", C.c_uint64), ("step", C.c_uint64),
        ("rng_offset", C.c_uint64), ("words", C.c_void_p), ("step_counter", C.c_void_p),
    ]


def _operand(name: str, nstride: int):
    return [(name, C.c_void_p), (f"{name}_stride", C.c_int64 * nstride), (f"{name}_dtype", C.c_int32)]


class MxUpdateArgs(C.Structure):
    _fields_ = (
        [("state", MxState)]
        + _operand("x", 3) + _operand("dt", 3) + _operand("dt_bias", 2) + _operand("A", 3) + _operand("B", 3)
        + _operand("C", 3) + _operand("D", 2) + _operand("z", 3) + _operand("out", 3)
        + [("ngroups", C.c_int32), ("dt_softplus", C.c_int32), ("rounding", Rounding), ("h_out", C.c_void_p)]
    )


class DenseUpdateArgs(C.Structure):
    _fields_ = (
        [("state", C.c_void_p), ("state_stride", C.c_int64 * 4), ("state_dtype", C.c_int32),
         ("batch", C.c_int32), ("heads", C.c_int32), ("dim", C.c_int32), ("dstate", C.c_int32)]
        + _operand("x", 3) + _operand("dt", 3) + _operand("dt_bias", 2) + _operand("A", 3) + _operand("B", 3)
        + _operand("C", 3) + _operand("D", 2) + _operand("z", 3) + _operand("out", 3)
        + [("ngroups", C.c_int32), ("dt_softplus", C.c_int32)]
    )


class Conv1dUpdateArgs(C.Structure):
    _fields_ = (
        [("conv_state", C.c_void_p), ("state_stride", C.c_int64 * 3), ("state_dtype", C.c_int32)]
        + _operand("x", 2) + _operand("weight", 2) + _operand("bias", 1) + _operand("out", 2)
        + [("batch", C.c_int32), ("channels", C.c_int32), ("width", C.c_int32), ("silu", C.c_int32)]
    )


class Int4Cache(C.Structure):
    _fields_ = [
        ("k_packed", C.c_void_p), ("v_packed", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("kp_stride", C.c_int64 * 4), ("vp_stride", C.c_int64 * 4), ("ks_stride", C.c_int64 * 4), ("vs_stride", C.c_int64 * 4),
        ("batch", C.c_int32), ("kv_heads", C.c_int32), ("capacity", C.c_int32), ("head_dim", C.c_int32),
        ("group_size", C.c_int32),
    ]


class Int4DecodeArgs(C.Structure):
    _fields_ = [
        ("cache", Int4Cache),
        ("q", C.c_void_p), ("q_stride", C.c_int64 * 3),
        ("out", C.c_void_p), ("out_stride", C.c_int64 * 3),
        ("dtype", C.c_int32), ("q_heads", C.c_int32), ("seq_len", C.c_int32),
        ("mask", C.c_void_p), ("mask_stride_b", C.c_int64), ("mask_stride_k", C.c_int64), ("mask_k_len", C.c_int32),
        ("splits", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("k_new", C.c_void_p), ("k_new_stride", C.c_int64 * 3),
        ("v_new", C.c_void_p), ("v_new_stride", C.c_int64 * 3),
        ("seq_len_counter", C.c_void_p),
    ]


class Int4PrefillArgs(C.Structure):
    _fields_ = [
        ("cache", Int4Cache),
        ("q", C.c_void_p), ("q_stride", C.c_int64 * 4),
        ("out", C.c_void_p), ("out_stride", C.c_int64 * 4),
        ("dtype", C.c_int32), ("q_heads", C.c_int32), ("q_len", C.c_int32), ("first_len", C.c_int32),
    ]


_lib = None


def lib() -> C.CDLL:
    """Load the shared library once; fail loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m layer_quant_b200.build` "
            "(layer_quant_b200 has no CPU or Triton fallback)")
    l = C.CDLL(str(LIB_PATH))
    l.lq_abi_version.restype = C.c_int
    l.lq_last_error_string.restype = C.c_char_p
    l.lq_device_status.argtypes = [C.POINTER(C.c_int32)]
    l.lq_mx_state_update.argtypes = [C.POINTER(MxUpdateArgs), C.c_void_p]
    l.lq_mx_quantize.argtypes = [C.POINTER(MxState), C.c_void_p, C.c_int32, C.c_int64, C.POINTER(Rounding), C.c_void_p]
    l.lq_mx_dequantize.argtypes = [C.POINTER(MxState), C.c_void_p, C.c_int64, C.c_void_p]
    l.lq_counter_add.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p]
    l.lq_mx_convert_layout.argtypes = [C.POINTER(MxState), C.POINTER(MxState), C.c_void_p]
    l.lq_int4_kv_append.argtypes = [C.POINTER(Int4Cache), C.c_void_p, C.POINTER(C.c_int64), C.c_void_p, C.POINTER(C.c_int64),
                                    C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]
    l.lq_int4_decode_attn.argtypes = [C.POINTER(Int4DecodeArgs), C.c_void_p]
    l.lq_int4_decode_attn_static.argtypes = [C.POINTER(Int4DecodeArgs), C.c_void_p]
    l.lq_int4_prefill_attn.argtypes = [C.POINTER(Int4PrefillArgs), C.c_void_p]
    l.lq_int4_static_scratch_bytes.restype = C.c_size_t
    l.lq_int4_decode_workspace_bytes.argtypes = [C.c_int32] * 5
    l.lq_int4_decode_workspace_bytes.restype = C.c_size_t
    l.lq_int4_decode_auto_splits.argtypes = [C.c_int32] * 3
    l.lq_int4_decode_auto_splits.restype = C.c_int32
    l.lq_dense_state_update.argtypes = [C.POINTER(DenseUpdateArgs), C.c_void_p]
    l.lq_causal_conv1d_update.argtypes = [C.POINTER(Conv1dUpdateArgs), C.c_void_p]
    l.lq_abi_sizeof.argtypes = [C.c_int]
    for which, struct in enumerate((MxState, Rounding, MxUpdateArgs, Int4Cache, Int4DecodeArgs, DenseUpdateArgs, Conv1dUpdateArgs,
                                    Int4PrefillArgs)):
        if l.lq_abi_sizeof(which) != C.sizeof(struct):
            raise RuntimeError(f"{LIB_PATH}: struct {struct.__name__} is {l.lq_abi_sizeof(which)} bytes in the library, "
                               f"{C.sizeof(struct)} in the binding; rebuild the library")
    if l.lq_abi_version() != 1:
        raise RuntimeError(f"{LIB_PATH}: ABI version {l.lq_abi_version()} != 1; rebuild the library")
    _lib = l
    return l


def check(rc: int) -> None:
    """Map a status code to the exception the reference raises in the same situation."""
    if rc == LQ_OK:
        return
    msg = lib().lq_last_error_string().decode("utf-8", "replace")
    if rc == LQ_ERR_INVALID_ARGUMENT:
        raise ValueError(msg)
    if rc == LQ_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(f"layer_quant_b200 error {rc}: {msg}")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}; expected bfloat16, float16 or float32") from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if t.device.type != "cuda":
            raise RuntimeError(f"layer_quant_b200 kernels need CUDA tensors, got {t.device} (no CPU fallback)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"tensors on different devices: {dev} and {t.device}")
    return dev


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device: torch.device) -> int:
    """cudaStream_t of torch's current stream on ``device`` (the raw-pointer query where torch offers it: it is
    several times cheaper than building a Stream object, and this sits on every launch)."""
    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


def set_ptr_strides(struct, name: str, t: torch.Tensor | None, nstride: int, with_dtype: bool = True) -> None:
    """Fill ``name``, ``name_stride`` (last ``nstride`` dims) and ``name_dtype`` of a ctypes struct."""
    if t is None:
        setattr(struct, name, None)
        return
    setattr(struct, name, t.data_ptr())
    st = t.stride()
    arr = getattr(struct, f"{name}_stride")
    for i in range(nstride):
        arr[i] = st[len(st) - nstride + i]
    if with_dtype:
        setattr(struct, f"{name}_dtype", dtype_code(t))


def device_status() -> int:
    v = C.c_int32(0)
    check(lib().lq_device_status(C.byref(v)))
    return v.value
