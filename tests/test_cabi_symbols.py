"""The C-ABI library builds, loads without a GPU, and exports exactly what include/dejavu_b200.h declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "dejavu_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(djv_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from dejavu_b200 import build, _lib

    build.build()
    return _lib.load()


def test_header_declares_functions():
    names = declared_functions()
    assert "djv_gather_gemv" in names and "djv_attn_step" in names and len(names) >= 25


def test_every_declared_symbol_is_exported(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_table_matches_header(lib):
    from dejavu_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_host_only_calls_work_without_a_gpu(lib):
    assert lib.djv_version() >= 100
    assert lib.djv_status_string(0) == b"ok"
    assert lib.djv_status_string(-4).startswith(b"scratch")
    assert lib.djv_gather_transposed_gemv_scratch_bytes(1, 12288, 512) > 4096
    assert lib.djv_attn_step_scratch_bytes(12, 128, 2048) > 4096


def test_argument_validation_happens_before_any_launch(lib):
    """Bad shapes are refused on the host with a message; nothing is launched (no GPU needed)."""
    from dejavu_b200 import _lib

    before = lib.djv_launch_count()
    fake = ctypes.c_void_p(0x1000)  # aligned, never dereferenced on the host
    rc = lib.djv_gather_gemv(fake, fake, fake, None, None, 1, 100, 4, 100, 0, 1, None)  # N % 8 != 0
    assert rc == _lib.ERR_INVALID and b"multiple of 8" in lib.djv_last_error()
    rc = lib.djv_gather_gemv(fake, fake, fake, None, None, 33, 128, 4, 128, 0, 1, None)  # batch too large
    assert rc == _lib.ERR_INVALID
    rc = lib.djv_gather_gemv(None, fake, fake, None, None, 1, 128, 4, 128, 0, 1, None)
    assert rc == _lib.ERR_INVALID and b"null" in lib.djv_last_error()
    rc = lib.djv_topk(fake, None, fake, 10, 11, 0, None)  # K > n
    assert rc == _lib.ERR_INVALID
    rc = lib.djv_topk(fake, None, fake, 1000000, 5, 0, None)  # too large for the shared memory of 8 blocks
    assert rc == _lib.ERR_UNSUPPORTED
    rc = lib.djv_qkv_proj_sparse(fake, fake, fake, fake, fake, None, 17, 256, 4, 64, 2, None)  # 17 rows
    assert rc == _lib.ERR_INVALID
    rc = lib.djv_out_proj_sparse(fake, fake, fake, fake, None, None, 1, 256, 4, 48, 2, None)  # head_dim 48
    assert rc == _lib.ERR_INVALID
    assert lib.djv_launch_count() == before


def test_static_scratch_entry_point_checks_alignment_on_the_host(lib):
    """The allocation-free fc2 entry point validates like the regular one: a y or bias pointer that is not
    16-byte aligned is refused before anything is launched (the kernel stores and loads 16 bytes at a time)."""
    from dejavu_b200 import _lib

    before = lib.djv_launch_count()
    ok, odd = ctypes.c_void_p(0x1000), ctypes.c_void_p(0x1002)
    rc = lib.djv_gather_transposed_gemv_static(odd, ok, ok, ok, None, 1, 128, 4, 128, 0, None)
    assert rc == _lib.ERR_INVALID and b"y must be 16-byte aligned" in lib.djv_last_error()
    rc = lib.djv_gather_transposed_gemv_static(ok, ok, ok, ok, odd, 1, 128, 4, 128, 0, None)
    assert rc == _lib.ERR_INVALID and b"bias must be 16-byte aligned" in lib.djv_last_error()
    rc = lib.djv_gather_transposed_gemv_static(ok, odd, ok, ok, None, 1, 128, 4, 128, 0, None)
    assert rc == _lib.ERR_INVALID
    assert lib.djv_launch_count() == before


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    from dejavu_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(ImportError, match="no fallback"):
        _lib.load()


def test_operators_refuse_cpu_tensors():
    import torch
    from dejavu_b200 import ops

    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.gather_gemv(torch.zeros(1, 64, dtype=torch.float16), torch.zeros(8, 64, dtype=torch.float16),
                        torch.arange(4))
