"""Tensor-level operators: torch CUDA tensors in, torch CUDA tensors out, all
compute in libftb200.so.  PyTorch is used for device memory and streams only.

Layouts follow the reference's C++ benchmarks (time-major activations
``[L, N, H]``, per-layer states ``[D, L, N, H]``:
benchmarks/rnn/fractaltensor/stacked_lstm/lstm.cu:31-38); the model-level
functions in :mod:`fractaltensor_b200.frontend` convert from and to the nested
FractalTensor views of the reference's Python programs.
"""
import ctypes

import torch

from . import _lib
from ._lib import check, lib

_DT = {torch.float32: _lib.DTYPE_F32, torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16}

_workspaces = {}


def _dtype_code(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError("unsupported dtype %s (float32, float16 or bfloat16)" % t.dtype)


def _req(t, name, dtype=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError("%s must be a torch.Tensor" % name)
    if not t.is_cuda:
        raise RuntimeError("%s must live on a CUDA device: there is no CPU path" % name)
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous" % name)
    if dtype is not None and t.dtype != dtype:
        raise TypeError("%s must have dtype %s, got %s" % (name, dtype, t.dtype))
    return t


def _req_like(t, name, dtype, shape, ref):
    """A caller-supplied buffer or parameter: the C side builds its addresses from the problem sizes,
    not from the buffer, so shape, dtype and device are checked here."""
    _req(t, name, dtype)
    if tuple(t.shape) != tuple(shape):
        raise ValueError("%s must have shape %s, got %s" % (name, tuple(shape), tuple(t.shape)))
    if t.device != ref.device:
        raise ValueError("%s lives on %s, the inputs on %s" % (name, t.device, ref.device))
    return t


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def workspace(device, nbytes=0):
    """The per-device workspace handed to every call: the status word, plus the
    schedule tables and completion counters of a persistent wavefront.  Grown on demand."""
    key = torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    need = max(int(nbytes), lib.ftb_workspace_bytes())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=torch.device("cuda", key))
        _workspaces[key] = ws
    return ws


def _tuning(layers_per_group=0, bn=0, schedule=0, skew=0, pair=0, fine_deps=0, resident=0):
    return (ctypes.c_int * 7)(int(layers_per_group), int(bn), int(schedule), int(skew), int(pair), int(fine_deps),
                              int(resident))


def check_status(device=None):
    """Synchronises the current stream and raises if a device wait ran out in
    the last call on `device`."""
    ws = workspace(device if device is not None else torch.cuda.current_device())
    out = ctypes.c_int(0)
    check(lib.ftb_read_status(_ptr(ws), ctypes.byref(out), _stream()), "ftb_read_status")
    if out.value != 0:
        ws[:8].zero_()  # the status word is sticky for some entry points: clear it for the next call
    check(out.value, "device kernel")


# ----------------------------------------------------------------------- LSTM
def lstm_pack_weights(W, U, bias=None):
    """W: [D,4,I,H], U: [D,4,H,H], bias: [D,4,H] or [D,4,1,H] -> (Wp [D,4H,I+H], bias_p fp32 [D,4H] | None)."""
    _req(W, "W")
    _req(U, "U", W.dtype)
    D, four, I, H = W.shape
    if four != 4 or tuple(U.shape) != (D, 4, H, H):
        raise ValueError("expected W [D,4,I,H] and U [D,4,H,H], got %s and %s" % (tuple(W.shape), tuple(U.shape)))
    Wp = torch.empty(D, 4 * H, I + H, dtype=W.dtype, device=W.device)
    bias_p = None
    if bias is not None:
        bias = _req(bias.reshape(D, 4, H).contiguous(), "bias", W.dtype)
        bias_p = torch.empty(D, 4 * H, dtype=torch.float32, device=W.device)
    with torch.cuda.device(W.device):
        check(lib.ftb_lstm_pack_weights(_ptr(W), _ptr(U), _ptr(bias), _ptr(Wp), _ptr(bias_p), D, I, H,
                                        _dtype_code(W), _stream()), "ftb_lstm_pack_weights")
    return Wp, bias_p


def lstm_stacked(x, Wp, bias_p=None, hs=None, c=None, layers_per_group=0, bn=0, schedule=0, skew=0, pair=0,
                 fine_deps=0, resident=0):
    """x: [L,N,I]; Wp: [D,4H,I+H] -> (hs [D,L,N,H], c fp32 [D,N,H]).
    schedule: 0 auto, 1 one launch per anti-diagonal, 2 one persistent kernel, 3 static tile ownership
    (CTA pairs on 256 batch rows), 4 static tile ownership with the batch on the N side of the MMA
    (at most 128 sequences; `resident`: recurrent weight blocks kept on chip, 0 auto, -1 none);
    pair: 0 auto, 1 single CTAs, 2 CTA pairs."""
    _req(x, "x")
    _req(Wp, "Wp", x.dtype)
    L, N, I = x.shape
    D, H4, K = Wp.shape
    H = H4 // 4
    if K != I + H or H4 != 4 * H or Wp.device != x.device:
        raise ValueError("Wp %s does not match x %s" % (tuple(Wp.shape), tuple(x.shape)))
    if bias_p is not None:
        _req_like(bias_p, "bias_p", torch.float32, (D, 4 * H), x)
    if hs is None:
        hs = torch.empty(D, L, N, H, dtype=x.dtype, device=x.device)
    if c is None:
        c = torch.empty(D, N, H, dtype=torch.float32, device=x.device)
    _req_like(hs, "hs", x.dtype, (D, L, N, H), x)
    _req_like(c, "c", torch.float32, (D, N, H), x)
    ws = workspace(x.device, lib.ftb_lstm_stacked_workspace_bytes(D, L, N, H))
    with torch.cuda.device(x.device):
        check(lib.ftb_lstm_stacked_fwd(_ptr(x), _ptr(Wp), _ptr(bias_p), _ptr(hs), _ptr(c), D, L, N, I, H,
                                       _dtype_code(x),
                                       _tuning(layers_per_group, bn, schedule, skew, pair, fine_deps, resident),
                                       _ptr(ws), ws.numel(),
                                       _stream()), "ftb_lstm_stacked_fwd")
    return hs, c


def lstm_stacked_varlen(x, active_rows, Wp, bias_p=None, hs=None, c=None, layers_per_group=0, bn=0, schedule=0,
                        pair=0):
    """Stacked LSTM over a length-sorted batch of variable-length sequences, time-major packed.

    active_rows: L non-increasing ints, the sequences still running at each step; x: [T,I] with
    T = sum(active_rows), rows of step t after those of step t-1; Wp: [D,4H,I+H]
    -> (hs [D,T,H] in the same packed order, c fp32 [D,N,H] with N = active_rows[0]).
    schedule: 0 auto, 1 one launch per anti-diagonal, 2 one persistent kernel."""
    _req(x, "x")
    _req(Wp, "Wp", x.dtype)
    active_rows = [int(n) for n in active_rows]
    L = len(active_rows)
    if L == 0 or active_rows[-1] <= 0 or any(a < b for a, b in zip(active_rows, active_rows[1:])):
        raise ValueError("active_rows must be non-increasing and positive (sort the batch by decreasing length)")
    T, I = x.shape
    D, H4, K = Wp.shape
    H = H4 // 4
    if K != I + H or H4 != 4 * H or T != sum(active_rows) or Wp.device != x.device:
        raise ValueError("Wp %s / active_rows (sum %d) do not match x %s" % (tuple(Wp.shape), sum(active_rows),
                                                                           tuple(x.shape)))
    if bias_p is not None:
        _req_like(bias_p, "bias_p", torch.float32, (D, 4 * H), x)
    N = active_rows[0]
    if hs is None:
        hs = torch.empty(D, T, H, dtype=x.dtype, device=x.device)
    if c is None:
        c = torch.empty(D, N, H, dtype=torch.float32, device=x.device)
    _req_like(hs, "hs", x.dtype, (D, T, H), x)
    _req_like(c, "c", torch.float32, (D, N, H), x)
    rows = (ctypes.c_int * L)(*active_rows)
    ws = workspace(x.device, lib.ftb_lstm_stacked_varlen_workspace_bytes(D, L))
    with torch.cuda.device(x.device):
        check(lib.ftb_lstm_stacked_varlen_fwd(_ptr(x), _ptr(Wp), _ptr(bias_p), _ptr(hs), _ptr(c), rows, D, L, I, H,
                                              _dtype_code(x), _tuning(layers_per_group, bn, schedule, 0, pair, 0),
                                              _ptr(ws), ws.numel(), _stream()), "ftb_lstm_stacked_varlen_fwd")
    return hs, c


def lstm_dilated(x, Wp, dilations, bias_p=None, hs=None, c=None, bn=0, pair=0, schedule=0):
    """x: [L,N,H]; Wp: [D,4H,2H]; dilations: D ints -> (hs [D,L,N,H], c fp32 [D,max_dil*N,H]).
    schedule: 0 auto, 1 one launch per level, 2 generic persistent kernel, 4 cluster kernel (H of 64, 128
    or 256: weights resident in tensor memory, one thread-block cluster per layer and batch slice)."""
    _req(x, "x")
    _req(Wp, "Wp", x.dtype)
    L, N, H = x.shape
    D = Wp.shape[0]
    if tuple(Wp.shape) != (D, 4 * H, 2 * H) or len(dilations) != D or Wp.device != x.device:
        raise ValueError("Wp %s / dilations do not match x %s" % (tuple(Wp.shape), tuple(x.shape)))
    if bias_p is not None:
        _req_like(bias_p, "bias_p", torch.float32, (D, 4 * H), x)
    md = max(int(d) for d in dilations)
    if hs is None:
        hs = torch.empty(D, L, N, H, dtype=x.dtype, device=x.device)
    if c is None:
        c = torch.empty(D, md * N, H, dtype=torch.float32, device=x.device)
    _req_like(hs, "hs", x.dtype, (D, L, N, H), x)
    _req_like(c, "c", torch.float32, (D, md * N, H), x)
    dil = (ctypes.c_int * D)(*[int(d) for d in dilations])
    ws = workspace(x.device, lib.ftb_lstm_dilated_workspace_bytes(D, L))
    with torch.cuda.device(x.device):
        check(lib.ftb_lstm_dilated_fwd(_ptr(x), _ptr(Wp), _ptr(bias_p), _ptr(hs), _ptr(c), dil, D, L, N, H,
                                       _dtype_code(x), _tuning(bn=bn, pair=pair, schedule=schedule), _ptr(ws), ws.numel(),
                                       _stream()), "ftb_lstm_dilated_fwd")
    return hs, c


# ------------------------------------------------------------------- grid RNN
def grid_pack_weights(i2h, h2h):
    """i2h: [D,2H,H], h2h: [D,H,H] -> Wp [D,H,3H]."""
    _req(i2h, "i2h")
    _req(h2h, "h2h", i2h.dtype)
    D, H2, H = i2h.shape
    if H2 != 2 * H or tuple(h2h.shape) != (D, H, H):
        raise ValueError("expected i2h [D,2H,H] and h2h [D,H,H]")
    Wp = torch.empty(D, H, 3 * H, dtype=i2h.dtype, device=i2h.device)
    with torch.cuda.device(i2h.device):
        for d in range(D):
            check(lib.ftb_grid_pack_weights(_ptr(i2h[d]), _ptr(h2h[d]), _ptr(Wp[d]), H, _dtype_code(i2h), _stream()),
                  "ftb_grid_pack_weights")
    return Wp


def grid_rnn(X, Y, Wpx, Wpy, bias_x=None, bias_y=None, schedule=0):
    """X,Y: [A,B,N,H]; Wpx,Wpy: [D,H,3H]; bias fp32 [D,H] -> (hx, hy) each [D,A,B,N,H].
    schedule: 0 auto (16-bit inputs: the cluster kernel where it applies, else the generic persistent
    kernel), 1 one launch per anti-diagonal, 2 the generic persistent kernel."""
    _req(X, "X")
    _req(Y, "Y", X.dtype)
    _req(Wpx, "Wpx", X.dtype)
    _req(Wpy, "Wpy", X.dtype)
    A, B, N, H = X.shape
    D = Wpx.shape[0]
    if tuple(Y.shape) != (A, B, N, H) or tuple(Wpx.shape) != (D, H, 3 * H) or tuple(Wpy.shape) != (D, H, 3 * H):
        raise ValueError("grid_rnn: inconsistent shapes")
    for b in (bias_x, bias_y):
        if b is not None:
            _req_like(b, "bias", torch.float32, (D, H), X)
    hx = torch.empty(D, A, B, N, H, dtype=X.dtype, device=X.device)
    hy = torch.empty_like(hx)
    # The library picks the schedule by the room the workspace offers: status word only -> one launch
    # per level; the tables -> generic persistent kernel; tables and flags -> cluster kernel.
    ws = workspace(X.device, 0 if schedule == 1 else lib.ftb_grid_rnn_workspace_bytes(D, A, B))
    ws_bytes = {1: lib.ftb_workspace_bytes(), 2: lib.ftb_grid_rnn_tables_bytes(D, A, B)}.get(schedule, ws.numel())
    with torch.cuda.device(X.device):
        check(lib.ftb_grid_rnn_fwd(_ptr(X), _ptr(Y), _ptr(Wpx), _ptr(Wpy), _ptr(bias_x), _ptr(bias_y), _ptr(hx),
                                   _ptr(hy), D, A, B, N, H, _dtype_code(X), _ptr(ws), ws_bytes, _stream()),
              "ftb_grid_rnn_fwd")
    return hx, hy


# ------------------------------------------------------------ B2B GEMM / attention
def b2b_gemm(A, B, C, out=None):
    """A: [batch,M,K]; B: [batch,N,K]; C: [batch,P,N] -> D [batch,M,P] = (A.B^T).C^T per batch entry."""
    _req(A, "A")
    _req(B, "B", A.dtype)
    _req(C, "C", A.dtype)
    batch, M, K = A.shape
    N = B.shape[1]
    P = C.shape[1]
    if tuple(B.shape) != (batch, N, K) or tuple(C.shape) != (batch, P, N):
        raise ValueError("b2b_gemm: inconsistent shapes")
    if out is None:
        out = torch.empty(batch, M, P, dtype=A.dtype, device=A.device)
    _req_like(out, "out", A.dtype, (batch, M, P), A)
    ws = workspace(A.device)
    with torch.cuda.device(A.device):
        check(lib.ftb_b2b_gemm(_ptr(A), _ptr(B), _ptr(C), _ptr(out), batch, M, N, K, P, _dtype_code(A), _ptr(ws),
                               ws.numel(), _stream()), "ftb_b2b_gemm")
    return out


def flash_attention(q, k, v, scale=None, out=None, causal=False, window=None, local=None):
    """q,k,v: [B,heads,S,d] -> softmax(scale * q k^T) v, same shape; `causal`: keys 0..i for query i;
    `window` (with causal): keys i-window+1..i; `local=(left, right)`: keys i-left..i+right."""
    _req(q, "q")
    _req(k, "k", q.dtype)
    _req(v, "v", q.dtype)
    B, heads, S, d = q.shape
    if tuple(k.shape) != tuple(q.shape) or tuple(v.shape) != tuple(q.shape):
        raise ValueError("flash_attention: q, k, v must have the same shape")
    if scale is None:
        scale = 1.0
    if out is None:
        out = torch.empty_like(q)
    _req_like(out, "out", q.dtype, q.shape, q)
    ws = workspace(q.device)
    with torch.cuda.device(q.device):
        if local is not None:
            if causal or window is not None:
                raise ValueError("flash_attention: local=(left, right) stands alone")
            check(lib.ftb_flash_attn_local_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(out), B, heads, S, d, int(local[0]),
                                               int(local[1]), float(scale), _dtype_code(q), _ptr(ws), ws.numel(),
                                               _stream()), "ftb_flash_attn_local_fwd")
            return out
        if window is not None:
            if not causal:
                raise ValueError("flash_attention: a window needs causal=True (the window ends at the query)")
            check(lib.ftb_flash_attn_window_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(out), B, heads, S, d, int(window),
                                                float(scale), _dtype_code(q), _ptr(ws), ws.numel(), _stream()),
                  "ftb_flash_attn_window_fwd")
            return out
        name = "ftb_flash_attn_causal_fwd" if causal else "ftb_flash_attn_fwd"
        check(getattr(lib, name)(_ptr(q), _ptr(k), _ptr(v), _ptr(out), B, heads, S, d, float(scale),
                                 _dtype_code(q), _ptr(ws), ws.numel(), _stream()), name)
    return out


def sparse_attention(q, k, v, rand_pos, window_size=5, dilation=2, n_global=3, scale=1.0, as_shipped=False,
                     out=None):
    """Token-level sparse attention (examples/sparse_attention/sparse_attention.py:41-76).

    q, k, v: [B, heads, S, d] (fp32, fp16 or bf16; d 32, 64, 128 or 256); rand_pos: int32
    [B, heads, S - 2 * n_global, R].  The first and last `n_global` tokens attend to each other;
    token i in between attends to the `window_size` keys at i - half + j * dilation (wrapped as
    ops.shifted_slide wraps them) and to the keys at rand_pos[..., i - n_global, :].
    `as_shipped=True` reproduces the softmax dimension the example actually runs with (dim 0:
    windowed tokens get the plain sum of their values, the global block is normalised over the
    queries); False normalises over the keys."""
    _req(q, "q")
    _req(k, "k", q.dtype)
    _req(v, "v", q.dtype)
    if q.dim() != 4 or tuple(k.shape) != tuple(q.shape) or tuple(v.shape) != tuple(q.shape):
        raise ValueError("sparse_attention: q, k, v must be [B, heads, S, d] of one shape")
    B, heads, S, d = q.shape
    inner = S - 2 * int(n_global)
    if inner < 0:
        raise ValueError("sparse_attention: 2 * n_global exceeds the sequence length")
    if rand_pos is None:
        R = 0
    else:
        if rand_pos.dtype != torch.int32 or not rand_pos.is_cuda or not rand_pos.is_contiguous():
            raise ValueError("sparse_attention: rand_pos must be a contiguous int32 CUDA tensor")
        if rand_pos.dim() != 4 or tuple(rand_pos.shape[:3]) != (B, heads, inner):
            raise ValueError("sparse_attention: rand_pos must be [B, heads, S - 2 * n_global, R]")
        if rand_pos.device != q.device:
            raise ValueError("sparse_attention: rand_pos is on another device")
        R = rand_pos.shape[3]
    if out is None:
        out = torch.empty_like(q)
    _req_like(out, "out", q.dtype, q.shape, q)
    ws = workspace(q.device)
    with torch.cuda.device(q.device):
        check(lib.ftb_sparse_attn_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(rand_pos) if R else None, _ptr(out), B, heads,
                                      S, d, int(window_size), int(dilation), int(n_global), R, float(scale),
                                      1 if as_shipped else 0, _dtype_code(q), _ptr(ws), ws.numel(), _stream()),
              "ftb_sparse_attn_fwd")
    return out


def rnn_pack_weights(W, U):
    """Tanh RNN cell h = tanh(x W + s U + b): W [I,H], U [H,H] -> Wp [H, I+H] (K-major rows)."""
    _req(W, "W")
    _req(U, "U", W.dtype)
    I, H = W.shape
    if tuple(U.shape) != (H, H):
        raise ValueError("expected W [I,H] and U [H,H]")
    Wp = torch.empty(H, I + H, dtype=W.dtype, device=W.device)
    with torch.cuda.device(W.device):
        check(lib.ftb_rnn_pack_weights(_ptr(W), _ptr(U), _ptr(Wp), I, H, _dtype_code(W), _stream()),
              "ftb_rnn_pack_weights")
    return Wp


def rnn_attention(src, trg, Wp_src, Wp_trg, bias_src, bias_trg, enc_proj, dec_proj, src_lens=None):
    """Attention RNN (examples/rnn_attention/rnn_attention.py:40-110) on time-major padded batches.

    src [Ls,N,H], trg [Lt,N,H]; Wp_* from rnn_pack_weights (I = H); bias_* fp32 [H] or None;
    enc_proj, dec_proj [H]; src_lens int32 [N] on the device or None (every sequence Ls long).
    Returns (enc [Ls,N,H], out [Lt,N,H]): the encoder states and the attention vectors, which are
    the program's result.  Rows past a sequence's own length are not meaningful."""
    _req(src, "src")
    _req(trg, "trg", src.dtype)
    if src.dim() != 3 or trg.dim() != 3 or trg.shape[1:] != src.shape[1:]:
        raise ValueError("rnn_attention: expected src [Ls,N,H] and trg [Lt,N,H]")
    Ls, N, H = src.shape
    Lt = trg.shape[0]
    _req_like(Wp_src, "Wp_src", src.dtype, (H, 2 * H), src)
    _req_like(Wp_trg, "Wp_trg", src.dtype, (H, 2 * H), src)
    _req_like(enc_proj, "enc_proj", src.dtype, (H,), src)
    _req_like(dec_proj, "dec_proj", src.dtype, (H,), src)
    for b_, name in ((bias_src, "bias_src"), (bias_trg, "bias_trg")):
        if b_ is not None:
            _req_like(b_, name, torch.float32, (H,), src)
    if src_lens is not None:
        _req_like(src_lens, "src_lens", torch.int32, (N,), src)
    enc = torch.empty_like(src)
    dec = torch.empty_like(trg)
    out = torch.empty_like(trg)
    scores = torch.empty(Ls, N, dtype=torch.float32, device=src.device)
    ws = workspace(src.device)
    opt = lambda t: _ptr(t) if t is not None else None
    with torch.cuda.device(src.device):
        check(lib.ftb_rnn_attention_fwd(_ptr(src), _ptr(trg), _ptr(Wp_src), _ptr(Wp_trg), opt(bias_src), opt(bias_trg),
                                        _ptr(enc_proj), _ptr(dec_proj), opt(src_lens), _ptr(enc), _ptr(scores),
                                        _ptr(dec), _ptr(out), Ls, Lt, N, H, _dtype_code(src), _ptr(ws), ws.numel(),
                                        _stream()), "ftb_rnn_attention_fwd")
    return enc, out


def gemm_nt(A, Bt, out=None, bn=0, pair=0):
    """A: [M,K]; Bt: [N,K] -> A @ Bt^T."""
    _req(A, "A")
    _req(Bt, "Bt", A.dtype)
    M, K = A.shape
    N = Bt.shape[0]
    if Bt.shape[1] != K:
        raise ValueError("gemm_nt: inner dimensions differ")
    if out is None:
        out = torch.empty(M, N, dtype=A.dtype, device=A.device)
    _req_like(out, "out", A.dtype, (M, N), A)
    ws = workspace(A.device)
    with torch.cuda.device(A.device):
        check(lib.ftb_gemm_nt(_ptr(A), _ptr(Bt), _ptr(out), M, N, K, _dtype_code(A), _tuning(bn=bn, pair=pair), _ptr(ws), ws.numel(),
                              _stream()), "ftb_gemm_nt")
    return out


def online_softmax(x, out=None):
    """Row-wise softmax of an fp32 matrix x [rows, width]: e^(max(x - m, -64)) / d per row."""
    _req(x, "x", torch.float32)
    if x.dim() != 2:
        raise ValueError("online_softmax: expected a matrix, got shape %s" % (tuple(x.shape),))
    if out is None:
        out = torch.empty_like(x)
    _req_like(out, "out", torch.float32, x.shape, x)
    rows, width = x.shape
    with torch.cuda.device(x.device):
        check(lib.ftb_online_softmax(_ptr(x), _ptr(out), rows, width, _stream()), "ftb_online_softmax")
    return out


def projection_pack(P):
    """P: [H,V] (x @ P orientation) -> Pt [Vp,H], one K-major row per vocabulary entry, Vp = V rounded up to 128."""
    _req(P, "P")
    if P.dim() != 2 or P.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("projection_pack: expected a 16-bit [H,V] matrix")
    H, V = P.shape
    Pt = torch.empty(lib.ftb_projection_padded_cols(V), H, dtype=P.dtype, device=P.device)
    with torch.cuda.device(P.device):
        check(lib.ftb_projection_pack(_ptr(P), _ptr(Pt), H, V, _dtype_code(P), _stream()), "ftb_projection_pack")
    return Pt


def lstm_project_softmax(h, Pt, V, out=None):
    """h: [..., H] hidden states (flattened to [T,H]); Pt from projection_pack; V the vocabulary size
    -> fp32 probabilities [T,V] = softmax(h . P) per row (a view of a [T,Vp] buffer)."""
    _req(h, "h")
    _req(Pt, "Pt", h.dtype)
    H = h.shape[-1]
    T = h.numel() // H
    Vp = lib.ftb_projection_padded_cols(int(V))
    if tuple(Pt.shape) != (Vp, H) or Pt.device != h.device:
        raise ValueError("lstm_project_softmax: Pt %s does not match h %s and V=%d" % (tuple(Pt.shape), tuple(h.shape), V))
    if out is None:
        out = torch.empty(T, Vp, dtype=torch.float32, device=h.device)
    _req_like(out, "out", torch.float32, (T, Vp), h)
    ws = workspace(h.device)
    with torch.cuda.device(h.device):
        check(lib.ftb_lstm_project_softmax(_ptr(h), _ptr(Pt), _ptr(out), T, int(V), H, _dtype_code(h), _ptr(ws),
                                           ws.numel(), _stream()), "ftb_lstm_project_softmax")
    return out[:, :V]


def embedding_gather(table, ids, out=None):
    """table: [V,H]; ids: int64 [T] (any nesting flattened) -> out [T,H] = table[ids]."""
    _req(table, "table")
    _req(ids, "ids", torch.int64)
    if table.dim() != 2:
        raise ValueError("embedding_gather: expected a [V,H] table, got shape %s" % (tuple(table.shape),))
    V, H = table.shape
    T = ids.numel()
    if out is None:
        out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    _req_like(out, "out", table.dtype, (T, H), table)
    ws = workspace(table.device)
    with torch.cuda.device(table.device):
        check(lib.ftb_embedding_gather(_ptr(table), _ptr(ids), _ptr(out), T, V, H, _dtype_code(table), _ptr(ws),
                                       ws.numel(), _stream()), "ftb_embedding_gather")
    return out
