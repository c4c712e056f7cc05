"""No-GPU checks of the C ABI: the shared library builds, loads, exports every symbol the header
declares, agrees with the ctypes mirror on struct sizes, and rejects bad arguments before it
touches a device."""
import ctypes as ct
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from layer_quant_b200 import _lib, build
    build.build()
    return _lib.lib()


def declared_symbols():
    text = (ROOT / "include" / "layer_quant_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lq_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/layer_quant_b200.h but not exported"


def test_struct_sizes_agree(lib):
    from layer_quant_b200 import _lib
    structs = (_lib.MxState, _lib.Rounding, _lib.MxUpdateArgs, _lib.Int4Cache, _lib.Int4DecodeArgs, _lib.DenseUpdateArgs,
               _lib.Conv1dUpdateArgs, _lib.Int4PrefillArgs)
    for which, struct in enumerate(structs):
        assert lib.lq_abi_sizeof(which) == ct.sizeof(struct), struct.__name__
    assert lib.lq_abi_sizeof(len(structs)) == -1
    assert lib.lq_abi_sizeof(99) == -1
    assert lib.lq_abi_version() == 1


def test_header_compiles_as_c(tmp_path):
    import subprocess
    src = tmp_path / "t.c"
    src.write_text('#include "layer_quant_b200.h"\nint main(void){lq_int4_decode_args a; lq_mx_update_args b; (void)a; (void)b; return 0;}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(ROOT / "include"), "-c", str(src), "-o", str(tmp_path / "t.o")], check=True)


def test_argument_validation_needs_no_device(lib):
    from layer_quant_b200 import _lib
    assert lib.lq_mx_state_update(None, None) == _lib.LQ_ERR_INVALID_ARGUMENT
    a = _lib.MxUpdateArgs()
    assert lib.lq_mx_state_update(ct.byref(a), None) == _lib.LQ_ERR_INVALID_ARGUMENT
    assert b"null state pointer" in lib.lq_last_error_string()
    a.state.q_state, a.state.shared_exp, a.state.micro_exp = 256, 512, 768
    a.state.batch, a.state.heads, a.state.dim, a.state.dstate = 1, 1, 1, 24
    a.state.format_bits = 6
    assert lib.lq_mx_state_update(ct.byref(a), None) == _lib.LQ_ERR_INVALID_ARGUMENT
    assert b"Only MX8 and MX4" in lib.lq_last_error_string()
    a.state.format_bits = 8
    assert lib.lq_mx_state_update(ct.byref(a), None) == _lib.LQ_ERR_INVALID_ARGUMENT
    assert b"divisible by 16" in lib.lq_last_error_string()
    with pytest.raises(ValueError, match="divisible by 16"):
        _lib.check(_lib.LQ_ERR_INVALID_ARGUMENT)
    d = _lib.Int4DecodeArgs()
    assert lib.lq_int4_decode_attn(ct.byref(d), None) == _lib.LQ_ERR_INVALID_ARGUMENT
    c = d.cache
    c.k_packed, c.v_packed, c.k_scale, c.v_scale = 256, 512, 768, 1024
    c.batch, c.kv_heads, c.capacity, c.head_dim, c.group_size = 1, 2, 16, 128, 48
    assert lib.lq_int4_decode_attn(ct.byref(d), None) == _lib.LQ_ERR_INVALID_ARGUMENT
    assert b"must be divisible by group_size=48" in lib.lq_last_error_string()
    c.group_size = 32
    d.q, d.out, d.q_heads, d.seq_len = 2048, 4096, 8, 17
    assert lib.lq_int4_decode_attn(ct.byref(d), None) == _lib.LQ_ERR_INVALID_ARGUMENT
    assert b"seq_len=17 outside [1, capacity=16]" in lib.lq_last_error_string()


def test_workspace_size_and_split_heuristic(lib):
    assert lib.lq_int4_decode_workspace_bytes(0, 32, 8, 128, 4) == 0
    n = lib.lq_int4_decode_workspace_bytes(2, 32, 8, 128, 4)
    assert n == 65536 * 4 + 2048 + 2 * 32 * 4 * 128 * 4
    assert lib.lq_int4_decode_auto_splits(1, 8, 1) == 1
    assert lib.lq_int4_decode_auto_splits(1, 8, 64) == 1
    s = lib.lq_int4_decode_auto_splits(1, 8, 131072)
    assert 8 <= s <= 128  # a single sequence with a long context is spread over the SMs
    assert lib.lq_int4_decode_auto_splits(256, 8, 131072) <= 4


def test_no_fallback_when_library_missing(monkeypatch, tmp_path):
    from layer_quant_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "missing.so")
    with pytest.raises(RuntimeError, match="no CPU or Triton fallback"):
        _lib.lib()
