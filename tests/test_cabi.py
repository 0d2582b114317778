"""The C-ABI library loads without a GPU, exports everything include/ftb200.h
declares, and rejects bad arguments before touching a device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from fractaltensor_b200 import _lib
    return _lib.lib


def _declared():
    text = open(os.path.join(ROOT, "include", "ftb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ftb_\w+)\s*\(", text)))


def test_header_declares_the_entry_points():
    names = _declared()
    for n in ("ftb_lstm_stacked_fwd", "ftb_lstm_dilated_fwd", "ftb_grid_rnn_fwd", "ftb_b2b_gemm",
              "ftb_flash_attn_fwd", "ftb_lstm_pack_weights", "ftb_read_status"):
        assert n in names


def test_library_exports_every_declared_symbol(lib):
    from fractaltensor_b200 import _lib
    for name in _declared():
        assert hasattr(lib, name), name
        assert name in _lib.SIGNATURES, "binding missing for " + name


def test_status_strings(lib):
    assert lib.ftb_status_str(0) == b"ok"
    assert b"workspace" in lib.ftb_status_str(3)
    assert lib.ftb_workspace_bytes() >= 4
    assert lib.ftb_version() >= 1


def test_bad_arguments_are_rejected_without_a_device(lib):
    z = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)  # never dereferenced: argument checks come first
    assert lib.ftb_lstm_stacked_fwd(z, z, z, z, z, 1, 1, 1, 64, 64, 2, None, z, 0, z) == 1
    # H not a multiple of 64
    assert lib.ftb_lstm_stacked_fwd(one, one, z, one, one, 1, 1, 1, 64, 48, 2, None, one, 256, z) == 1
    # I != H with more than one layer
    assert lib.ftb_lstm_stacked_fwd(one, one, z, one, one, 2, 1, 1, 128, 64, 2, None, one, 256, z) == 1
    # missing workspace
    assert lib.ftb_lstm_stacked_fwd(one, one, z, one, one, 1, 1, 1, 64, 64, 2, None, z, 0, z) == 3
    assert lib.ftb_b2b_gemm(one, one, one, one, 1, 128, 64, 128, 128, 1, one, 256, z) == 1   # N not 128/256/512
    assert lib.ftb_b2b_gemm(one, one, one, one, 1, 128, 512, 64, 128, 1, one, 256, z) == 1   # B, C too large for one SM
    assert lib.ftb_b2b_gemm(one, one, one, one, 1, 100, 128, 128, 128, 1, one, 256, z) == 1  # M % 128
    assert lib.ftb_b2b_gemm(one, one, one, one, 1, 128, 128, 128, 128, 0, one, 256, z) == 1  # fp32
    assert lib.ftb_flash_attn_fwd(one, one, one, one, 1, 1, 256, 64, 1.0, 1, one, 256, z) == 1  # d != 128
    assert lib.ftb_flash_attn_fwd(one, one, one, one, 1, 1, 100, 128, 1.0, 1, one, 256, z) == 1  # S % 256
    assert lib.ftb_flash_attn_causal_fwd(one, one, one, one, 1, 1, 256, 128, 0.0, 1, one, 256, z) == 1  # scale <= 0
    assert lib.ftb_flash_attn_causal_fwd(one, one, one, one, 1, 1, 100, 128, 1.0, 1, one, 256, z) == 1  # S % 256
    assert lib.ftb_flash_attn_window_fwd(one, one, one, one, 1, 1, 256, 128, 0, 1.0, 1, one, 256, z) == 1  # window < 1
    assert lib.ftb_flash_attn_local_fwd(one, one, one, one, 1, 1, 256, 128, -1, 0, 1.0, 1, one, 256, z) == 1  # left < 0
    assert lib.ftb_flash_attn_local_fwd(one, one, one, one, 1, 1, 256, 128, 0, -2, 1.0, 1, one, 256, z) == 1  # right < 0
    assert lib.ftb_gemm_nt(one, one, one, 8, 128, 60, 1, None, one, 256, z) == 1  # K % 64
    sp = lambda **kw: lib.ftb_sparse_attn_fwd(
        one, one, one, kw.get("pos", one), one, 1, 1, kw.get("S", 16), kw.get("d", 64), kw.get("window", 5),
        kw.get("dilation", 2), kw.get("ng", 3), kw.get("R", 3), 1.0, 0, 0, one, 256, z)
    assert sp(window=4) == 1          # even windows are not defined by ops.shifted_slide
    assert sp(dilation=0) == 1
    assert sp(d=48) == 1
    assert sp(ng=9) == 1              # 2 * n_global > S
    assert sp(window=9, dilation=4) == 1   # half = 16 >= S: the wrap is a single step
    assert sp(window=63, dilation=1, S=128, R=2) == 1  # more than 64 keys per token
    assert sp(pos=z) == 1             # R > 0 without positions
    ra = lambda **kw: lib.ftb_rnn_attention_fwd(
        one, one, one, one, z, z, one, one, z, one, kw.get("scores", one), one, one, kw.get("Ls", 4), kw.get("Lt", 3),
        2, kw.get("H", 64), 1, one, 256, z)
    assert ra(H=48) == 1
    assert ra(Ls=0) == 1
    assert ra(Ls=20000) == 1          # the scores of one sequence must fit in shared memory
    assert ra(scores=z) == 1
    assert lib.ftb_rnn_pack_weights(one, one, z, 64, 64, 1, z) == 1
    rows = (ctypes.c_int * 3)(4, 5, 1)  # not sorted by decreasing length
    assert lib.ftb_lstm_stacked_varlen_fwd(one, one, z, one, one, rows, 1, 3, 64, 64, 1, None, one, 256, z) == 1
    rows = (ctypes.c_int * 3)(4, 2, 0)  # a step without sequences
    assert lib.ftb_lstm_stacked_varlen_fwd(one, one, z, one, one, rows, 1, 3, 64, 64, 1, None, one, 256, z) == 1
    rows = (ctypes.c_int * 3)(4, 2, 1)
    assert lib.ftb_lstm_stacked_varlen_fwd(one, one, z, one, one, rows, 1, 3, 64, 64, 1, None, z, 0, z) == 3
    assert lib.ftb_lstm_stacked_varlen_workspace_bytes(16, 100) > lib.ftb_workspace_bytes()
    dil = (ctypes.c_int * 2)(1, 0)
    assert lib.ftb_lstm_dilated_fwd(one, one, z, one, one, dil, 2, 4, 1, 64, 1, None, one, 256, z) == 1  # dilation 0


def test_misaligned_pointers_are_rejected_without_a_device(lib):
    """Every kernel moves 16 bytes at a time (float4 on the fp32 path, TMA on the 16-bit path): a
    pointer off a 16-byte boundary is answered with FTB_ERR_ALIGN (2) before any launch."""
    z = ctypes.c_void_p(0)
    ok, off = ctypes.c_void_p(4096), ctypes.c_void_p(4096 + 4)
    for dtype in (0, 1, 2):
        assert lib.ftb_lstm_stacked_fwd(off, ok, z, ok, ok, 1, 1, 1, 64, 64, dtype, None, ok, 256, z) == 2
        assert lib.ftb_lstm_stacked_fwd(ok, ok, z, off, ok, 1, 1, 1, 64, 64, dtype, None, ok, 256, z) == 2
        assert lib.ftb_lstm_stacked_fwd(ok, ok, off, ok, ok, 1, 1, 1, 64, 64, dtype, None, ok, 256, z) == 2
    dil = (ctypes.c_int * 1)(1)
    assert lib.ftb_lstm_dilated_fwd(ok, off, z, ok, ok, dil, 1, 4, 1, 64, 0, None, ok, 256, z) == 2
    assert lib.ftb_grid_rnn_fwd(ok, ok, ok, ok, z, z, ok, off, 1, 2, 2, 1, 64, 0, ok, 256, z) == 2
    assert lib.ftb_gemm_nt(ok, ok, off, 8, 128, 64, 0, None, ok, 256, z) == 2
    rows = (ctypes.c_int * 2)(2, 1)
    assert lib.ftb_lstm_stacked_varlen_fwd(ok, ok, z, ok, off, rows, 1, 2, 64, 64, 0, None, ok, 256, z) == 2
    assert lib.ftb_sparse_attn_fwd(ok, off, ok, ok, ok, 1, 1, 16, 64, 5, 2, 3, 3, 1.0, 0, 0, ok, 256, z) == 2


def test_no_fallback_when_library_is_missing(monkeypatch, tmp_path):
    from fractaltensor_b200 import _lib
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        _lib.load()
