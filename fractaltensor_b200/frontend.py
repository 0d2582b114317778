"""Model-level entry points with the signatures of the reference's programs.

The reference expresses the hot path as nested ``ops.fold / scan / map`` programs
over ``FractalTensor`` values (flat ``.data`` buffer plus nested ``.indices``):

    stacked_lstm(embs, Wss, Uss, bss)                  examples/stacked_rnn/stacked_lstm1.py:66-76
    stacked_lstm_time_major(embs, Wss, Uss, bss)       examples/stacked_rnn/stacked_rnn.py:69-79
    dilated_lstm(embs, Wss, Uss, bss)                  examples/dilated_rnn/dilated_rnn.py:16-41 (the fold in model())
    stacked_grid_rnns(src_encs, trg_encs, params)      examples/grid_rnn/grid_rnn.py:111-122
    flash_attention(qsss, ksss, vsss)                  examples/flash_attention/flash_attention.py:75-88
    embed(words, embedding)                            examples/stacked_rnn/rnn_utils.py:80-90 (the lookup in front)
    sparse_attention(query, key, value, random_attn)   examples/sparse_attention/sparse_attention.py:41-76, 109-114
    rnn_attention(src_embs, trg_embs, ...)             examples/rnn_attention/rnn_attention.py:86-110 (behind the lookups)

The functions here keep those argument lists and return the same nested values,
but run the whole nest as one fused wavefront on the GPU.  Arguments may be the
reference's own ``kaleido.FractalTensor`` objects (only ``.data``, ``.indices``
and ``.element_shape`` are read) or the light ``FractalTensor`` defined here.  A
FractalTensor whose nesting is rectangular is exactly a dense array
``[n1, ..., nk, *element_shape]``.  The stacked LSTM also takes ragged batches
(sequences of different lengths): time-major and sorted by decreasing length as
the reference builds them, or batch-major in any order.  The other programs
reject ragged nestings, since there is no CPU fallback to hand them to.
"""
import torch

from . import ops


class FractalTensor(object):
    """Minimal stand-in for kaleido.FractalTensor (kaleido/frontend/fractal_tensor.py:85-181):
    a flat ``data`` buffer, nested-list ``indices`` and the shape of the stored tensors."""

    def __init__(self, data, indices, element_shape):
        self.data = data.reshape(-1)
        self.indices = indices
        self.element_shape = tuple(element_shape)

    @staticmethod
    def from_dense(t, depth):
        """t: [n1, ..., n_depth, *element_shape]."""
        dims = list(t.shape[:depth])

        def nest(ds):
            if len(ds) == 1:
                return list(range(ds[0]))
            return [nest(ds[1:]) for _ in range(ds[0])]

        return FractalTensor(t.contiguous(), nest(dims), t.shape[depth:])

    @property
    def depth(self):
        d, x = 0, self.indices
        while isinstance(x, list):
            d, x = d + 1, (x[0] if x else None)
        return d

    def __len__(self):
        return len(self.indices)

    def to_dense(self):
        return _dense(self)

    @property
    def element_type(self):
        """The type singleton of the stored numbers (types.float32, types.float16, types.bfloat16, ...)."""
        from . import types
        return types.torch_type_to_internal_type(self.data.dtype)

    def astype(self, dtype):
        """The same nesting with the numbers converted; dtype: a type singleton or a torch dtype."""
        from . import types
        if isinstance(dtype, types.Number):
            dtype = types.internal_type_to_torch_type(dtype)
        return FractalTensor(self.data.to(dtype), self.indices, self.element_shape)


def _nest_dims(indices):
    """Lengths of a rectangular nesting; raises ValueError for a ragged one."""
    dims = []
    level = [indices]
    while level and isinstance(level[0], list):
        n = len(level[0])
        if any(len(x) != n for x in level):
            raise ValueError("ragged FractalTensor: variable-length nestings are not accelerated "
                             "and there is no CPU fallback")
        dims.append(n)
        level = [y for x in level for y in x]
    return dims


def _dense(x):
    """Dense [n1,...,nk,*element_shape] view of a FractalTensor-like value (or a tensor as is)."""
    if isinstance(x, torch.Tensor):
        return x
    if not (hasattr(x, "data") and hasattr(x, "indices")):
        raise TypeError("expected a FractalTensor or a torch.Tensor, got %s" % type(x).__name__)
    dims = _nest_dims(x.indices)
    return x.data.reshape(*dims, *tuple(x.element_shape))


def _cuda(t, dtype=None):
    if not t.is_cuda:
        raise RuntimeError("inputs must already live on a CUDA device: there is no CPU path")
    return t if dtype is None else t.to(dtype)


def embed(words, embedding, dtype=None):
    """The lookup the RNN examples run first:
    ``ops.map(lambda ws: ops.map(lambda word: ops.index(ops.slices(embedding, dim=0), word), ws), words)``.

    words: a FractalTensor of integers in any nesting (batch-major [N][L_n] or time-major [L][n_t],
    ragged or not); embedding: [V,H] tensor (or an object with .data).  Returns a FractalTensor with
    the same nesting whose elements are the [1,H] rows, ready for stacked_lstm / stacked_lstm_time_major.
    """
    table = embedding.data if hasattr(embedding, "data") and not isinstance(embedding, torch.Tensor) else embedding
    table = _cuda(table, dtype)
    if table.dim() != 2:
        table = table.reshape(-1, table.shape[-1])
    ids = _cuda(words.data.reshape(-1)).to(torch.int64)
    out = ops.embedding_gather(table.contiguous(), ids.contiguous())
    return FractalTensor(out, words.indices, (1, table.shape[1]))


def project_softmax(hs, prev_softmax_proj):
    """The vocabulary projection behind the recurrent layers: softmax(h @ prev_softmax_proj) for every
    word position (prev_softmax_proj [H, vocab], examples/stacked_rnn/rnn_utils.py:45-50).

    hs: the FractalTensor of [1,H] hidden states a stacked_lstm call returned (any nesting, ragged or
    not); prev_softmax_proj: [H,V] tensor (or an object with .data).  Returns a FractalTensor with the
    same nesting whose elements are the [1,V] fp32 probability rows."""
    P = prev_softmax_proj.data if hasattr(prev_softmax_proj, "data") and not isinstance(prev_softmax_proj, torch.Tensor) \
        else prev_softmax_proj
    h = _cuda(hs.data if not isinstance(hs, torch.Tensor) else hs)
    H = P.shape[0]
    P = _cuda(P, h.dtype).reshape(H, -1).contiguous()
    probs = ops.lstm_project_softmax(h.reshape(-1, H).contiguous(), ops.projection_pack(P), P.shape[1])
    if isinstance(hs, torch.Tensor):
        return probs
    return FractalTensor(probs.contiguous(), hs.indices, (1, P.shape[1]))


def _is_ragged(x):
    if isinstance(x, torch.Tensor):
        return False
    try:
        _nest_dims(x.indices)
        return False
    except ValueError:
        return True


def _packed_weights(Wss, Uss, bss, dtype):
    W, U, b = _cuda(_dense(Wss), dtype), _cuda(_dense(Uss), dtype), _cuda(_dense(bss), dtype)
    D, H = U.shape[0], U.shape[-1]
    Wp, bias_p = ops.lstm_pack_weights(W.contiguous(), U.contiguous(), b.reshape(D, 4, H).contiguous())
    return Wp, bias_p, D, H


def stacked_lstm_time_major(embs, Wss, Uss, bss, dtype=None):
    """The time-major stacked LSTM: fold(depth) of scan(time) of map(active sequences) of lstm_cell.

    embs: [L][n_t] of [1,I], n_t the sequences still running at step t (non-increasing: the batch
    is sorted by decreasing length and sequence n sits at position n of every step it is in).
    Returns the top layer's hidden states with the same nesting, [L][n_t] of [1,H].
    """
    if isinstance(embs, torch.Tensor):
        active = [embs.shape[1]] * embs.shape[0]
        flat = embs.reshape(embs.shape[0] * embs.shape[1], -1)
    else:
        active = [len(step) for step in embs.indices]
        flat = embs.data.reshape(sum(active), -1)
    x = _cuda(flat, dtype).contiguous()
    Wp, bias_p, D, H = _packed_weights(Wss, Uss, bss, x.dtype)
    hs, _ = ops.lstm_stacked_varlen(x, active, Wp, bias_p)
    return FractalTensor(hs[D - 1], [list(range(n)) for n in active], (1, H))


def _stacked_lstm_ragged(embs, Wss, Uss, bss, dtype):
    """Batch-major ragged batch [N][L_n]: sort by decreasing length, transpose into the
    time-major packed layout on the device, run, and put the rows back where they were."""
    lens = [len(seq) for seq in embs.indices]
    if min(lens) <= 0:
        raise ValueError("empty sequence in the batch")
    flat = _cuda(embs.data.reshape(sum(lens), -1), dtype)
    dev = flat.device
    order = sorted(range(len(lens)), key=lambda n: -lens[n])
    start = [0]
    for n in lens:
        start.append(start[-1] + n)
    L = lens[order[0]]
    active = [sum(1 for n in lens if n > t) for t in range(L)]
    # src[k] = position in the batch-major buffer of the k-th row of the time-major one
    src = torch.tensor([start[order[r]] + t for t in range(L) for r in range(active[t])], dtype=torch.long,
                       device=dev)
    Wp, bias_p, D, H = _packed_weights(Wss, Uss, bss, flat.dtype)
    hs, _ = ops.lstm_stacked_varlen(flat.index_select(0, src).contiguous(), active, Wp, bias_p)
    out = torch.empty(sum(lens), H, dtype=hs.dtype, device=dev)
    out.index_copy_(0, src, hs[D - 1])
    return FractalTensor(out, [list(range(n)) for n in lens], (1, H))


def stacked_lstm(embs, Wss, Uss, bss, dtype=None):
    """fold(depth) of map(batch) of scan(time) of lstm_cell, as one depth x time wavefront.

    embs: [N][L] of [1,I] (sequences may differ in length); Wss: [D][4] of [I,H]; Uss: [D][4] of
    [H,H]; bss: [D][4] of [1,H].
    Returns the top layer's hidden states as a FractalTensor [N][L] of [1,H].
    """
    if _is_ragged(embs):
        return _stacked_lstm_ragged(embs, Wss, Uss, bss, dtype)
    x = _cuda(_dense(embs), dtype)
    W, U, b = _cuda(_dense(Wss), dtype), _cuda(_dense(Uss), dtype), _cuda(_dense(bss), dtype)
    N, L = x.shape[0], x.shape[1]
    D, H = U.shape[0], U.shape[-1]
    Wp, bias_p = ops.lstm_pack_weights(W.contiguous(), U.contiguous(), b.reshape(D, 4, H).contiguous())
    xt = x.reshape(N, L, -1).transpose(0, 1).contiguous()  # time-major [L,N,I]
    hs, _ = ops.lstm_stacked(xt, Wp, bias_p)
    top = hs[D - 1].transpose(0, 1).reshape(N, L, 1, H)
    return FractalTensor.from_dense(top, 2)


def dilated_lstm(embs, Wss, Uss, bss, dilations=None, dtype=None):
    """map(batch) of fold(layers) of dilated_map(scan(lstm_cell)), dilation 2**layer by default."""
    x = _cuda(_dense(embs), dtype)
    W, U, b = _cuda(_dense(Wss), dtype), _cuda(_dense(Uss), dtype), _cuda(_dense(bss), dtype)
    N, L = x.shape[0], x.shape[1]
    D, H = U.shape[0], U.shape[-1]
    if dilations is None:
        dilations = [2 ** l for l in range(D)]
    Wp, bias_p = ops.lstm_pack_weights(W.contiguous(), U.contiguous(), b.reshape(D, 4, H).contiguous())
    xt = x.reshape(N, L, H).transpose(0, 1).contiguous()
    hs, _ = ops.lstm_dilated(xt, Wp, dilations, bias_p)
    top = hs[D - 1].transpose(0, 1).reshape(N, L, 1, H)
    return FractalTensor.from_dense(top, 2)


def stacked_grid_rnns(src_encs, trg_encs, stacked_params, dtype=None):
    """Grid RNN over the src x trg grid for a batch of sentence pairs.

    src_encs: [N][B] of [1,H]; trg_encs: [N][A] of [1,H]; stacked_params: a sequence of
    ((i2h_x, h2h_x, bias_x), (i2h_y, h2h_y, bias_y)) per layer (tensors or objects with .data).
    Returns (hx, hy) of the top layer as FractalTensors [N][A][B] of [1,H], where grid
    point (a, b) pairs trg[a] with src[b].
    """
    src = _cuda(_dense(src_encs), dtype)
    trg = _cuda(_dense(trg_encs), dtype)
    N, B = src.shape[0], src.shape[1]
    A = trg.shape[1]
    H = src.shape[-1]
    raw = lambda p: p.data if hasattr(p, "data") and not isinstance(p, torch.Tensor) else p
    stack = lambda d, i: torch.stack([_cuda(raw(layer[d][i]), src.dtype) for layer in stacked_params])
    Wpx = ops.grid_pack_weights(stack(0, 0).contiguous(), stack(0, 1).contiguous())
    Wpy = ops.grid_pack_weights(stack(1, 0).contiguous(), stack(1, 1).contiguous())
    bx = stack(0, 2).reshape(-1, H).float().contiguous()
    by = stack(1, 2).reshape(-1, H).float().contiguous()
    s = src.reshape(N, B, H).transpose(0, 1)  # [B,N,H]
    t = trg.reshape(N, A, H).transpose(0, 1)  # [A,N,H]
    X = s[None].expand(A, B, N, H).contiguous()
    Y = t[:, None].expand(A, B, N, H).contiguous()
    hx, hy = ops.grid_rnn(X, Y, Wpx, Wpy, bx, by)
    D = Wpx.shape[0]
    to_ft = lambda h: FractalTensor.from_dense(h[D - 1].permute(2, 0, 1, 3).reshape(N, A, B, 1, H), 3)
    return to_ft(hx), to_ft(hy)


def flash_attention(qsss, ksss, vsss, scale=1.0, dtype=None, causal=False, window=None, local=None):
    """map(batch) of map(heads) of map(query blocks) of reduce(key/value blocks) of attn_func.

    q/k/v: [B][heads][blocks] of [block, d].  Returns the same nesting.  `causal`: the reduce of
    query block i runs over key/value blocks 0..i, the last one masked above its diagonal; `window`
    (with causal) also drops the keys more than window-1 positions before the query; `local=(left,
    right)` keeps keys i-left..i+right instead.
    """
    q, k, v = (_cuda(_dense(t), dtype) for t in (qsss, ksss, vsss))
    Bsz, heads, nblk, blk, d = q.shape
    flat = lambda t: t.reshape(Bsz, heads, nblk * blk, d).contiguous()
    o = ops.flash_attention(flat(q), flat(k), flat(v), scale=scale, causal=causal, window=window, local=local)
    return FractalTensor.from_dense(o.reshape(Bsz, heads, nblk, blk, d), 3)


def sparse_attention(query_proj, key_proj, value_proj, random_attn, window_size=5, dilation=2, n_global=3,
                     scale=1.0, as_shipped=False, dtype=None):
    """per_head_attn mapped over heads and batch: the last ``ops.map`` of multihead_sparse_attention
    (examples/sparse_attention/sparse_attention.py:109-114), or one head (lines 41-76).

    query_proj / key_proj / value_proj: FractalTensors of [1, d] tokens nested [S] (one head),
    [heads][S] or [B][heads][S]; random_attn: the same nesting of [1, R] integer tensors, S - 2 *
    n_global of them per head.  Returns the attention vectors in the nesting of query_proj.
    `as_shipped=True` runs the softmax dimension the example's ``ops.softmax(x)`` calls really use
    (dimension 0); the default normalises over the keys."""
    q, k, v = (_cuda(_dense(t), dtype) for t in (query_proj, key_proj, value_proj))
    pos = _cuda(_dense(random_attn)).to(torch.int32)
    depth = q.dim() - 2            # element shape is [1, d]
    if depth < 1 or depth > 3:
        raise ValueError("sparse_attention: expected a nesting [S], [heads][S] or [B][heads][S]")
    S, d = q.shape[depth - 1], q.shape[-1]
    lead = tuple(q.shape[:depth - 1])
    heads_total = 1
    for n in lead:
        heads_total *= n
    flat = lambda t: t.reshape(1, heads_total, S, d).contiguous()
    o = ops.sparse_attention(flat(q), flat(k), flat(v), pos.reshape(1, heads_total, S - 2 * n_global, -1).contiguous(),
                             window_size=window_size, dilation=dilation, n_global=n_global, scale=scale,
                             as_shipped=as_shipped)
    return FractalTensor.from_dense(o.reshape(*lead, S, 1, d), depth)


def _tensor_of(x):
    return x.data if hasattr(x, "data") and not isinstance(x, torch.Tensor) else x


def _pad_time_major(x, dtype):
    """Batch-major ragged FractalTensor [N][L_n] of [1,H] -> ([Lmax, N, H] zero-padded, lens, row index)."""
    lens = [len(seq) for seq in x.indices]
    if not lens or min(lens) <= 0:
        raise ValueError("empty batch or empty sequence")
    flat = _cuda(x.data.reshape(sum(lens), -1), dtype)
    N, L, H = len(lens), max(lens), flat.shape[1]
    # position in the padded [L, N] grid of every row of the batch-major buffer
    idx = torch.tensor([t * N + n for n in range(N) for t in range(lens[n])], dtype=torch.long, device=flat.device)
    padded = torch.zeros(L * N, H, dtype=flat.dtype, device=flat.device)
    padded.index_copy_(0, idx, flat)
    return padded.reshape(L, N, H), lens, idx


def rnn_attention(src_embs, trg_embs, src_params, trg_params, attn_params, dtype=None):
    """The attention RNN behind the word lookups (examples/rnn_attention/rnn_attention.py:86-110):
    ``src_enc_outs = map(scan(cell))`` over the source sequences, then ``map(attn_layer)`` over the
    (encoder states, target sequence) pairs.

    src_embs, trg_embs: FractalTensors [N][L_n] of [1,H] rows (ragged or not, any order);
    src_params, trg_params: (W [H,H], U [H,H], b [1,H]) as CellParams; attn_params: (encoder_proj
    [H,1], decoder_proj [H,1]).  Returns the attention vectors with the nesting of trg_embs."""
    src, src_lens, _ = _pad_time_major(src_embs, dtype)
    trg, trg_lens, trg_idx = _pad_time_major(trg_embs, dtype)
    if len(src_lens) != len(trg_lens):
        raise ValueError("rnn_attention: source and target batches differ in size")
    dt, dev = src.dtype, src.device
    H = src.shape[2]
    par = lambda t: _cuda(_tensor_of(t), dt).contiguous()
    Ws, Us, bs = (par(t) for t in src_params)
    Wt, Ut, bt = (par(t) for t in trg_params)
    enc_proj, dec_proj = (par(t).reshape(H) for t in attn_params)
    lens = torch.tensor(src_lens, dtype=torch.int32, device=dev)
    _, out = ops.rnn_attention(src, trg.to(dt), ops.rnn_pack_weights(Ws, Us), ops.rnn_pack_weights(Wt, Ut),
                               bs.reshape(H).float().contiguous(), bt.reshape(H).float().contiguous(), enc_proj,
                               dec_proj, lens)
    rows = out.reshape(-1, H).index_select(0, trg_idx)
    return FractalTensor(rows.contiguous(), [list(range(n)) for n in trg_lens], (1, H))
