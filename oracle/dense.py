"""CPU oracle: dense PyTorch restatements of the reference's model programs.

TEST INFRASTRUCTURE ONLY.  Nothing in the product (``fractaltensor_b200/``) may
import this package; it is imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` as the
checker and the timed CPU baseline, never as the thing shipped.

Each function restates, with whole-batch tensor operations, the arithmetic that
the reference's eager frontend performs one sample and one gate at a time.  The
restatements are pinned against the reference's own frontend programs, executed
from the reference tree, by ``tests/golden/generate.py``; the resulting vectors
are committed under ``tests/golden/`` and checked by ``tests/test_oracle.py``.

All functions compute in the dtype of their inputs (fp32 in every pinned use).
``round_to`` (a 16-bit torch dtype or None) optionally rounds each hidden state
the way a 16-bit kernel has to before feeding it back into a matrix multiply;
the default None is the reference's semantics.
"""
import math

import torch


def _round(t, round_to):
    return t if round_to is None else t.to(round_to).to(t.dtype)


def lstm_cell_dense(x, h, c, W, U, b):
    """One LSTM cell for a whole batch.

    Follows gate_f / lstm_cell (examples/stacked_rnn/stacked_rnn.py:12-36):
    gate k = x @ W[k] + h @ U[k] + b[k], order (i, f, o, c~);
    c' = sigmoid(f) * c + sigmoid(i) * tanh(c~); h' = sigmoid(o) * tanh(c').
    x: [N,I]; h,c: [N,H]; W: [4,I,H]; U: [4,H,H]; b: [4,H] or None.
    """
    g = [x @ W[k] + h @ U[k] + (0 if b is None else b[k]) for k in range(4)]
    i, f, o = torch.sigmoid(g[0]), torch.sigmoid(g[1]), torch.sigmoid(g[2])
    c_new = f * c + i * torch.tanh(g[3])
    h_new = o * torch.tanh(c_new)
    return h_new, c_new


def stacked_lstm_dense(x, W, U, b=None, round_to=None):
    """Stacked LSTM: fold over depth of (map over batch of (scan over time)).

    Follows stacked_lstm / lstm_layer / batched_cell
    (examples/stacked_rnn/stacked_lstm1.py:40-76).  x: [L,N,I] time-major;
    W: [D,4,I,H]; U: [D,4,H,H]; b: [D,4,H] or None.
    Returns hs [D,L,N,H] (hidden state of every layer) and c [D,N,H] (final).
    """
    D = W.shape[0]
    L, N, _ = x.shape
    H = U.shape[-1]
    hs = x.new_zeros(D, L, N, H)
    cs = x.new_zeros(D, N, H)
    inp = x
    for d in range(D):
        h = x.new_zeros(N, H)
        c = x.new_zeros(N, H)
        for t in range(L):
            h, c = lstm_cell_dense(inp[t], h, c, W[d], U[d], None if b is None else b[d])
            h = _round(h, round_to)
            hs[d, t] = h
        cs[d] = c
        inp = hs[d]
    return hs, cs


def stacked_lstm_varlen_dense(x, active_rows, W, U, b=None, round_to=None):
    """Stacked LSTM over a length-sorted, time-major batch of variable-length sequences.

    Follows batched_cell / lstm_layer / stacked_lstm of the time-major program
    (examples/stacked_rnn/stacked_rnn.py:40-79): step t holds only the active_rows[t]
    sequences that are still running (the batch is sorted by decreasing length, so
    these are rows 0..active_rows[t]-1, examples/utils/data_utils.py:42-66) and carries
    ``hs_prev[0:xs.length]``, ``cs_prev[0:xs.length]`` into the cell.
    x: [T,I] with T = sum(active_rows), the rows of step t stored after those of step
    t-1 (the flat FractalTensor buffer); W: [D,4,I,H]; U: [D,4,H,H]; b: [D,4,H] or None.
    Returns hs [D,T,H] in the same packed order and c [D,N,H], N = active_rows[0]: the
    cell state each sequence had after its own last step.
    """
    active_rows = [int(n) for n in active_rows]
    D = W.shape[0]
    H = U.shape[-1]
    T, N = sum(active_rows), active_rows[0]
    off = [0]
    for n in active_rows:
        off.append(off[-1] + n)
    hs = x.new_zeros(D, T, H)
    cs = x.new_zeros(D, N, H)
    inp = x
    for d in range(D):
        h = x.new_zeros(N, H)
        c = x.new_zeros(N, H)
        for t, n in enumerate(active_rows):
            hn, cn = lstm_cell_dense(inp[off[t]:off[t + 1]], h[:n], c[:n], W[d], U[d], None if b is None else b[d])
            hn = _round(hn, round_to)
            h, c = hn, cn
            hs[d, off[t]:off[t + 1]] = hn
            cs[d, :n] = cn
        inp = hs[d]
    return hs, cs


def dilated_lstm_dense(x, W, U, dilations, b=None, round_to=None):
    """Stacked dilated LSTM.

    Follows dilated_layer / model (examples/dilated_rnn/dilated_rnn.py:16-41) with
    DilatedMap (kaleido/frontend/operations/fractaltensor/functional/apply_to_each.py:83-177):
    layer l splits the sequence into dilations[l] interleaved sub-sequences and
    scans each from a zero state, i.e. (h,c)[l][t] = cell((h,c)[l][t-dil], x = h[l-1][t]).
    x: [L,N,H]; W,U: [D,4,H,H].  Returns hs [D,L,N,H].
    """
    D = W.shape[0]
    L, N, H = x.shape
    hs = x.new_zeros(D, L, N, H)
    inp = x
    for l in range(D):
        dil = int(dilations[l])
        cs = [None] * L
        for t in range(L):
            if t >= dil:
                hp, cp = hs[l, t - dil], cs[t - dil]
            else:
                hp, cp = x.new_zeros(N, H), x.new_zeros(N, H)
            h, c = lstm_cell_dense(inp[t], hp, cp, W[l], U[l], None if b is None else b[l])
            hs[l, t] = _round(h, round_to)
            cs[t] = c
        inp = hs[l]
    return hs


def grid_rnn_dense(X, Y, i2h_x, h2h_x, b_x, i2h_y, h2h_y, b_y, round_to=None):
    """Stacked 2-D grid RNN with vanilla tanh cells.

    Follows vanilla_cell / grid_cell / direction_y / direction_x /
    stacked_grid_rnns (examples/grid_rnn/grid_rnn.py:42-122):
    s = cat(state_x, state_y); h_x = tanh(s @ i2h_x + x_t @ h2h_x + b_x), h_y alike
    with the y parameters and y_t; state_x = h_x[a-1][b], state_y = h_y[a][b-1],
    zeros at the borders; the next layer reads (h_x, h_y) of the layer below.
    X,Y: [A,B,N,H]; i2h_*: [D,2H,H]; h2h_*: [D,H,H]; b_*: [D,H] or None.
    Returns hx, hy: [D,A,B,N,H].
    """
    D = i2h_x.shape[0]
    A, B, N, H = X.shape
    hx = X.new_zeros(D, A, B, N, H)
    hy = X.new_zeros(D, A, B, N, H)
    xin, yin = X, Y
    zero = X.new_zeros(N, H)
    for d in range(D):
        bx = 0 if b_x is None else b_x[d]
        by = 0 if b_y is None else b_y[d]
        for a in range(A):
            for b in range(B):
                sx = hx[d, a - 1, b] if a > 0 else zero
                sy = hy[d, a, b - 1] if b > 0 else zero
                s = torch.cat([sx, sy], dim=1)
                hx[d, a, b] = _round(torch.tanh(s @ i2h_x[d] + xin[a, b] @ h2h_x[d] + bx), round_to)
                hy[d, a, b] = _round(torch.tanh(s @ i2h_y[d] + yin[a, b] @ h2h_y[d] + by), round_to)
        xin, yin = hx[d], hy[d]
    return hx, hy


def b2b_gemm_dense(A, B, C):
    """Back-to-back GEMM with the reference kernel's rounding.

    Follows KeBack2BackGemm (kaleido/core/device/kernels/cutlass_wmma.h:489-533):
    P = A.B accumulated in fp32 and rounded to the 16-bit input type, D = P.C
    accumulated in fp32 and rounded again.  A: [batch,M,K]; B: [batch,N,K]
    (the reference's column-major [K,N]); C: [batch,P,N]; returns [batch,M,P].
    """
    lp = A.dtype
    P = (A.float() @ B.float().transpose(-1, -2)).to(lp)
    return (P.float() @ C.float().transpose(-1, -2)).to(lp)


def flash_attention_dense(q, k, v, scale=1.0, block=64):
    """Blockwise attention with the online-softmax carry of the reference.

    Follows attn_func / per_block_func (examples/flash_attention/flash_attention.py:14-60)
    over key/value blocks of `block` rows, for all query rows at once, with the
    carry started at (max, sum, out) = (-float32.max, 0, 0) in that order and
    `scale` multiplied into q @ k^T.  q,k,v: [B,heads,S,d]; returns the same shape.
    """
    Bsz, heads, S, d = q.shape
    m = q.new_full((Bsz, heads, S, 1), -torch.finfo(torch.float32).max)
    l = q.new_zeros(Bsz, heads, S, 1)
    o = q.new_zeros(Bsz, heads, S, d)
    for j0 in range(0, S, block):
        kj, vj = k[:, :, j0:j0 + block], v[:, :, j0:j0 + block]
        w = (q @ kj.transpose(-1, -2)) * scale
        cur_m = w.max(dim=-1, keepdim=True).values
        e = torch.exp(w - cur_m)
        ev = e @ vj
        cur_l = e.sum(dim=-1, keepdim=True)
        new_m = torch.maximum(cur_m, m)
        r_prev = torch.exp(m - new_m)
        r_cur = torch.exp(cur_m - new_m)
        new_l = r_prev * l + r_cur * cur_l
        o = (o * l * r_prev + r_cur * ev) / new_l
        m, l = new_m, new_l
    return o


def online_softmax_dense(x):
    """Row-wise softmax with the reference kernel's clamp.

    Follows ReduceMD / MapRescale (kaleido/core/device/kernels/online_softmax.h:113-163): per row
    m = max x, d = sum e^(x - m), output e^(max(x - m, -64)) / d.  x: [rows, width].
    """
    m = x.max(dim=1, keepdim=True).values
    d = torch.exp(x - m).sum(dim=1, keepdim=True)
    return torch.exp(torch.clamp(x - m, min=-64.0)) / d


def project_softmax_dense(h, P):
    """softmax(h @ P) per row: the vocabulary projection the reference's RNN examples declare behind
    the recurrent layers (prev_softmax_proj [H, vocab], examples/stacked_rnn/rnn_utils.py:45-50),
    with the reference frontend's own softmax (ops.softmax = torch.nn.functional.softmax,
    kaleido/frontend/operations/tensor/arithmetic/reduction.py:24-29).  h: [T,H]; P: [H,V]."""
    return torch.softmax(h @ P, dim=-1)


def sparse_attention_dense(q, k, v, rand_pos, window_size=5, dilation=2, n_global=3, as_shipped=False):
    """Token-level sparse attention of one head: windowed + random + global keys.

    Follows per_head_attn / sparse_attn (examples/sparse_attention/sparse_attention.py:24-76):
    the first and last `n_global` tokens attend to each other only,
    ``softmax(g_query @ g_key.T) @ g_value``; every other token i attends to the `window_size` keys
    of ops.shifted_slide(window_size, dilation) centred on it, i.e. positions
    range(i - half, i + half + 1, dilation) with half = ((window_size - 1) * (dilation - 1) +
    window_size) // 2, wrapped the way ShiftedSlide._ids wraps them (x < 0 -> x + S - 1;
    x >= S -> x - S; kaleido/frontend/operations/fractaltensor/access.py:389-410), plus the
    positions rand_pos[i - n_global]; no scale on the scores.

    `as_shipped`: the example calls ``ops.softmax(x)`` without a dimension, and the reference's
    softmax defaults to dim = 0 (kaleido/frontend/operations/tensor/arithmetic/reduction.py:26):
    on the [1, W + R] score row of a windowed token that normalises over a single element (every
    weight becomes 1: the output is the plain sum of the selected values), and on the global
    block it normalises over the queries instead of the keys.  True reproduces exactly that (it
    is what the golden vector holds); False is the attention the example describes, softmax over
    the keys.
    q, k, v: [..., S, d]; rand_pos: integer [..., S - 2 * n_global, R].  Returns [..., S, d].
    """
    S = q.shape[-2]
    half = ((window_size - 1) * (dilation - 1) + window_size) // 2
    out = torch.empty_like(q)
    gidx = list(range(n_global)) + list(range(S - n_global, S))
    gq, gk, gv = q[..., gidx, :], k[..., gidx, :], v[..., gidx, :]
    out[..., gidx, :] = torch.softmax(gq @ gk.transpose(-1, -2), dim=-2 if as_shipped else -1) @ gv

    def wrap(x):
        return x + S - 1 if x < 0 else (x - S if x >= S else x)

    for i in range(n_global, S - n_global):
        win = torch.tensor([wrap(x) for x in range(i - half, i + half + 1, dilation)], dtype=torch.long)
        pos = rand_pos[..., i - n_global, :].long()
        idx = torch.cat([win.expand(*pos.shape[:-1], win.numel()), pos], dim=-1)  # [..., W + R]
        gather = lambda t: torch.gather(t, -2, idx[..., None].expand(*idx.shape, t.shape[-1]))
        ks, vs = gather(k), gather(v)
        s_row = q[..., i:i + 1, :] @ ks.transpose(-1, -2)
        w = torch.ones_like(s_row) if as_shipped else torch.softmax(s_row, dim=-1)
        out[..., i:i + 1, :] = w @ vs
    return out


def rnn_attention_dense(src, trg, src_lens, trg_lens, Ws, Us, bs, Wt, Ut, bt, enc_proj, dec_proj):
    """Attention RNN: model() of examples/rnn_attention/rnn_attention.py:86-110 behind the lookups.

    Per sequence pair: the encoder is a tanh RNN over the source rows,
    ``e_j = tanh(x_j @ Ws + e_{j-1} @ Us + bs)`` (cell(), lines 40-48, scanned from zeros, 99-103);
    the decoder scan (attn_func / attn_layer, lines 52-83) carries the attention vector:
    ``dec_t = tanh(y_t @ Wt + v_{t-1} @ Ut + bt)``, ``score_j = e_j @ enc_proj + dec_t @ dec_proj``,
    ``w = softmax_j(score)``, ``v_t = sum_j w_j e_j``, v_{-1} = 0; the program returns the v_t.
    src: [sum(src_lens), H] and trg: [sum(trg_lens), H], the sequences one after the other;
    Ws, Us, Wt, Ut: [H, H]; bs, bt: [1, H]; enc_proj, dec_proj: [H, 1].
    Returns (enc [sum(src_lens), H], out [sum(trg_lens), H])."""
    H = src.shape[1]
    encs, outs = [], []
    so = to = 0
    for ls, lt in zip(src_lens, trg_lens):
        ls, lt = int(ls), int(lt)
        e = torch.zeros(1, H, dtype=src.dtype)
        rows = []
        for j in range(ls):
            e = torch.tanh(src[so + j:so + j + 1] @ Ws + e @ Us + bs)
            rows.append(e)
        E = torch.cat(rows, dim=0)  # [ls, H]
        es = E @ enc_proj            # [ls, 1]
        v = torch.zeros(1, H, dtype=src.dtype)
        for t in range(lt):
            dec = torch.tanh(trg[to + t:to + t + 1] @ Wt + v @ Ut + bt)
            w = torch.softmax(es + dec @ dec_proj, dim=0)  # over the encoder positions
            v = (w * E).sum(dim=0, keepdim=True)
            outs.append(v)
        encs.append(E)
        so += ls
        to += lt
    return torch.cat(encs, dim=0), torch.cat(outs, dim=0)


def embedding_gather_dense(table, ids):
    """One table row per word, in the order of the flat word buffer.

    Follows ops.index(ops.slices(embedding, dim=0), word) mapped over a batch of word sequences
    (examples/stacked_rnn/rnn_utils.py:80-90).  table: [V,H]; ids: int64 [T]; returns [T,H].
    """
    return table[ids.reshape(-1)]


def attention_plain(q, k, v, scale=1.0, causal=False, window=None, local=None):
    """softmax(scale * q k^T) v, the closed form the blockwise carry equals.

    `causal`: query i sees keys 0..i (later scores are -inf before the softmax).  The reference
    has no causal program, so this case has no vectors of the reference behind it.
    """
    w = (q @ k.transpose(-1, -2)) * scale
    if local is not None:  # keys i-left .. i+right
        S = q.shape[-2]
        ones = torch.ones(S, S, dtype=torch.bool, device=q.device)
        keep = ones.tril(int(local[1])) & ones.triu(-int(local[0]))
        w = w.masked_fill(~keep, float("-inf"))
    elif causal:
        S = q.shape[-2]
        keep = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        if window is not None:  # keys i-window+1 .. i
            keep &= ~torch.ones(S, S, dtype=torch.bool, device=q.device).tril(-int(window))
        w = w.masked_fill(~keep, float("-inf"))
    return torch.softmax(w, dim=-1) @ v


def flash_attention_causal_dense(q, k, v, scale=1.0, block=64):
    """The blockwise carry of flash_attention_dense with the key walk of each query block cut
    at its diagonal block and the later keys of that block masked to -inf."""
    Bsz, heads, S, d = q.shape
    out = torch.empty_like(q)
    for i0 in range(0, S, block):
        qi = q[:, :, i0:i0 + block]
        m = q.new_full((Bsz, heads, qi.shape[2], 1), -torch.finfo(torch.float32).max)
        l = q.new_zeros(Bsz, heads, qi.shape[2], 1)
        o = q.new_zeros(Bsz, heads, qi.shape[2], d)
        for j0 in range(0, i0 + block, block):
            kj, vj = k[:, :, j0:j0 + block], v[:, :, j0:j0 + block]
            w = (qi @ kj.transpose(-1, -2)) * scale
            if j0 == i0:
                n = w.shape[-1]
                keep = torch.ones(qi.shape[2], n, dtype=torch.bool, device=q.device).tril()
                w = w.masked_fill(~keep, float("-inf"))
            cur_m = w.max(dim=-1, keepdim=True).values
            e = torch.exp(w - cur_m)
            ev = e @ vj
            cur_l = e.sum(dim=-1, keepdim=True)
            new_m = torch.maximum(cur_m, m)
            r_prev = torch.exp(m - new_m)
            r_cur = torch.exp(cur_m - new_m)
            new_l = r_prev * l + r_cur * cur_l
            o = (o * l * r_prev + r_cur * ev) / new_l
            m, l = new_m, new_l
        out[:, :, i0:i0 + block] = o
    return out


# ------------------------------------------------------------------ seeded inputs
def _gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def make_lstm_inputs(D, L, N, I, H, seed, w_bound, dtype=torch.float32, bias=False):
    """x ~ N(0,1) [L,N,I]; W,U ~ U(-w_bound, w_bound); bias 0 or ~U when `bias`."""
    g = _gen(seed)
    x = torch.randn(L, N, I, generator=g)
    W = (torch.rand(D, 4, I, H, generator=g) * 2 - 1) * w_bound
    U = (torch.rand(D, 4, H, H, generator=g) * 2 - 1) * w_bound
    b = (torch.rand(D, 4, H, generator=g) * 2 - 1) * w_bound if bias else None
    cast = lambda t: None if t is None else t.to(dtype)
    return cast(x), cast(W), cast(U), cast(b)


def make_active_rows(L, N, seed, min_len=1):
    """Rows still active at each of L steps for N sequences whose lengths are drawn
    uniformly from [min_len, L] and sorted in decreasing order (the longest has L steps)."""
    g = _gen(seed)
    lens = torch.randint(min_len, L + 1, (N,), generator=g)
    lens[0] = L
    return [int((lens > t).sum()) for t in range(L)]


def make_grid_inputs(D, A, B, N, H, seed, w_bound, dtype=torch.float32, bias=False):
    """src [B,N,H], trg [A,N,H] ~ N(0,1); X[a][b] = src[b], Y[a][b] = trg[a]."""
    g = _gen(seed)
    src = torch.randn(B, N, H, generator=g)
    trg = torch.randn(A, N, H, generator=g)
    X = src[None].expand(A, B, N, H).contiguous()
    Y = trg[:, None].expand(A, B, N, H).contiguous()
    mk = lambda *s: (torch.rand(*s, generator=g) * 2 - 1) * w_bound
    p = dict(i2h_x=mk(D, 2 * H, H), h2h_x=mk(D, H, H), i2h_y=mk(D, 2 * H, H), h2h_y=mk(D, H, H))
    p["b_x"] = mk(D, H) if bias else None
    p["b_y"] = mk(D, H) if bias else None
    cast = lambda t: None if t is None else t.to(dtype)
    return cast(X), cast(Y), {k_: cast(v_) for k_, v_ in p.items()}


def make_b2b_inputs(batch, M, N, K, P, seed, dtype=torch.float16):
    g = _gen(seed)
    s = 1.0 / math.sqrt(128.0)
    A = (torch.randn(batch, M, K, generator=g) * s).to(dtype)
    B = (torch.randn(batch, N, K, generator=g) * s).to(dtype)
    C = (torch.randn(batch, P, N, generator=g) * s).to(dtype)
    return A, B, C


def make_attention_inputs(B, heads, S, d, seed, dtype=torch.float16):
    g = _gen(seed)
    q = torch.randn(B, heads, S, d, generator=g).to(dtype)
    k = torch.randn(B, heads, S, d, generator=g).to(dtype)
    v = torch.randn(B, heads, S, d, generator=g).to(dtype)
    return q, k, v
