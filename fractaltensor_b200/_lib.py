"""ctypes binding of libftb200.so, the C-ABI library declared in include/ftb200.h.

The library is the only compute path: there is no CPU or PyTorch fallback.  If
the shared object is missing, importing this module raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libftb200.so")

DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2

# name -> (restype, argtypes); mirrors include/ftb200.h one to one.
_vp, _i, _sz, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_float
SIGNATURES = {
    "ftb_version": (_i, []),
    "ftb_status_str": (ctypes.c_char_p, [_i]),
    "ftb_workspace_bytes": (_sz, []),
    "ftb_launch_count": (ctypes.c_longlong, []),
    "ftb_read_status": (_i, [_vp, ctypes.POINTER(_i), _vp]),
    "ftb_lstm_pack_weights": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "ftb_lstm_stacked_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "ftb_lstm_stacked_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, ctypes.POINTER(_i), _vp, _sz, _vp]),
    "ftb_lstm_stacked_fwd_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, ctypes.POINTER(_i),
                                          ctypes.POINTER(_vp), _vp]),
    "ftb_lstm_stacked_varlen_workspace_bytes": (_sz, [_i, _i]),
    "ftb_lstm_stacked_varlen_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, ctypes.POINTER(_i), _i, _i, _i, _i, _i, ctypes.POINTER(_i), _vp, _sz, _vp]),
    "ftb_lstm_dilated_workspace_bytes": (_sz, [_i, _i]),
    "ftb_lstm_dilated_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, ctypes.POINTER(_i), _i, _i, _i, _i, _i, ctypes.POINTER(_i), _vp, _sz, _vp]),
    "ftb_grid_pack_weights": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "ftb_grid_rnn_workspace_bytes": (_sz, [_i, _i, _i]),
    "ftb_grid_rnn_tables_bytes": (_sz, [_i, _i, _i]),
    "ftb_grid_rnn_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "ftb_b2b_gemm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "ftb_flash_attn_fwd": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp, _sz, _vp]),
    "ftb_flash_attn_causal_fwd": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp, _sz, _vp]),
    "ftb_flash_attn_window_fwd": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _vp, _sz, _vp]),
    "ftb_flash_attn_local_fwd": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _sz, _vp]),
    "ftb_rnn_pack_weights": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "ftb_rnn_attention_fwd": (_i, [_vp] * 13 + [_i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "ftb_sparse_attn_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _sz, _vp]),
    "ftb_embedding_gather": (_i, [_vp, _vp, _vp, ctypes.c_longlong, ctypes.c_longlong, _i, _i, _vp, _sz, _vp]),
    "ftb_online_softmax": (_i, [_vp, _vp, _i, _i, _vp]),
    "ftb_projection_padded_cols": (_i, [_i]),
    "ftb_projection_pack": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "ftb_lstm_project_softmax": (_i, [_vp, _vp, _vp, ctypes.c_longlong, _i, _i, _i, _vp, _sz, _vp]),
    "ftb_gemm_nt": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, ctypes.POINTER(_i), _vp, _sz, _vp]),
}


def load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libftb200.so is not built (%s); run `python -m fractaltensor_b200.build`. "
            "There is no fallback path." % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing
        fn.restype = res
        fn.argtypes = args
    return lib


lib = load()


class FtbError(RuntimeError):
    def __init__(self, code, where):
        self.code = code
        msg = lib.ftb_status_str(code).decode()
        super().__init__("%s failed with status %d: %s" % (where, code, msg))


def check(code, where):
    if code != 0:
        raise FtbError(code, where)
