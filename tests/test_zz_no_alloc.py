"""The allocation-free stacked-LSTM entry point against the regular one.

ftb_lstm_stacked_fwd_noalloc serves hosts that cannot allocate device memory where they run
the forward pass (a plugin that only receives input/output buffers, a real-time loop that
must stay out of the allocator, a process whose pool is fully committed): its schedule tables and counters live in a
fixed array inside the library instead of a caller workspace.  It must give exactly the
result of ftb_lstm_stacked_fwd, call after call, although every call reuses the same array.

This file sorts last on purpose: if it fails under ``pytest -x``, every other test has
already run.
"""
import ctypes

import pytest
import torch

from oracle import dense

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, x, Wp, bias_p, hs, c, D, L, N, I, H, dtype_code):
    scratch = ctypes.c_void_p(0)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ftb_lstm_stacked_fwd_noalloc(ptr(x), ptr(Wp), ptr(bias_p), ptr(hs), ptr(c), D, L, N, I, H, dtype_code,
                                          None, ctypes.byref(scratch), stream)
    return rc, scratch


def test_noalloc_entry_matches_regular_entry_twice_in_a_row():
    assert torch.cuda.is_available()
    from fractaltensor_b200 import ops
    from fractaltensor_b200._lib import lib

    D, L, N, H = 3, 6, 256, 256
    for call, seed in enumerate((21, 22)):  # two calls in a row share the built-in scratch array
        x, W, U, b = dense.make_lstm_inputs(D, L, N, H, H, seed, 1.0 / 8, dtype=torch.bfloat16, bias=True)
        xd, Wd, Ud, bd = (t.cuda() for t in (x, W, U, b))
        Wp, bp = ops.lstm_pack_weights(Wd, Ud, bd)
        ref_h, ref_c = ops.lstm_stacked(xd, Wp, bp, schedule=2)
        ops.check_status()

        hs = torch.full((D, L, N, H), float("nan"), dtype=torch.bfloat16, device="cuda")
        c = torch.full((D, N, H), float("nan"), dtype=torch.float32, device="cuda")
        if call == 0:
            # The first call on a device looks the scratch array's address up; measure the second.
            rc, _ = _call_noalloc(lib, xd, Wp, bp, hs, c, D, L, N, H, H, 2)
            assert rc == 0, lib.ftb_status_str(rc)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]  # the driver's view: sees a cudaMalloc made inside the library too
        rc, scratch = _call_noalloc(lib, xd, Wp, bp, hs, c, D, L, N, H, H, 2)
        assert rc == 0, lib.ftb_status_str(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before
        status = ctypes.c_int(-1)
        assert scratch.value
        assert lib.ftb_read_status(scratch, ctypes.byref(status), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
        assert status.value == 0, lib.ftb_status_str(status.value)
        # same kernel, same schedule: identical bits; and within tolerance of the oracle
        assert torch.equal(hs, ref_h), "call %d: hidden states differ" % call
        assert torch.equal(c, ref_c), "call %d: cell states differ" % call
        want, _ = dense.stacked_lstm_dense(x.float(), W.float(), U.float(), b.float())
        assert (hs.float().cpu() - want).abs().max().item() <= 2e-2


def test_noalloc_entry_rejects_what_does_not_fit():
    from fractaltensor_b200._lib import lib
    one = ctypes.c_void_p(16)  # never dereferenced: the size check comes first
    z = ctypes.c_void_p(0)
    # 64 layers x 4096 steps of H=1024 needs far more than the 4 MiB built-in array
    rc = lib.ftb_lstm_stacked_fwd_noalloc(one, one, z, one, one, 64, 4096, 256, 1024, 1024, 2, None, None, z)
    assert rc == 7
    assert b"static" in lib.ftb_status_str(7)
    # fp32 has no persistent schedule
    assert lib.ftb_lstm_stacked_fwd_noalloc(one, one, z, one, one, 2, 4, 32, 64, 64, 0, None, None, z) == 1
