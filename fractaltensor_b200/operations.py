"""Second-order array combinators with the reference's signatures, dispatching whole programs.

The reference's frontend runs ``ops.map / scan / fold / zip`` eagerly, one Python call per
element (kaleido/frontend/operations/fractaltensor/functional/aggregate.py:28-112,
apply_to_each.py:28-46, access.py:36-61).  Here a program written with the same combinators is
*traced*: the outermost combinator that receives real FractalTensors runs the user's functions
once on symbolic stand-ins, obtains the nest of combinators and the cell arithmetic as a tree,
and compares it with the trees of the programs the library has fused kernels for.  On a match
the whole nest runs as one wavefront on the GPU; anything else raises ``NotImplementedError``
(there is no element-by-element fallback).

Recognised so far: the stacked LSTM, batch-major (examples/stacked_rnn/stacked_lstm1.py:12-76)
and time-major over a length-sorted ragged batch (examples/stacked_rnn/stacked_rnn.py:12-79), and
blockwise attention with the online-softmax carry (examples/flash_attention/flash_attention.py:14-88,
carry in (max, sum, out) order, optionally with the scores multiplied by a Python float), and the
stacked dilated LSTM (examples/dilated_rnn/dilated_rnn.py:16-41, dilation 2**layer), and the stacked
grid RNN (examples/grid_rnn/grid_rnn.py:42-146: ``ops.product`` of the two sentences, two nested
scans, ``ops.cat`` of the two incoming states, a tanh cell per direction; ``stacked_params`` a
Python sequence of ((i2h, h2h, bias), (i2h, h2h, bias)) per layer; the call returns the top layer's
(h_x, h_y) grids).

    from fractaltensor_b200 import operations as ops
    out = ops.fold(lambda s, param: lstm_layer(s, *param), ops.zip(Wss, Uss, bss), initializer=embs)
"""
import builtins

import torch

from . import frontend

__all__ = ["map", "scan", "fold", "reduce", "zip", "enumerate", "dilated_map", "product", "repeat", "zeros", "full", "cat",
           "sigmoid", "tanh", "exp", "max", "sum", "maximum"]


# ----------------------------------------------------------------- symbolic values
def _canon(op, a, b):
    """Commutative operands in a fixed order, so that x*y and y*x trace to the same tree."""
    return (op,) + tuple(sorted((a, b), key=repr))


class SymTensor(object):
    """Stand-in for a Tensor while a program is traced: records the arithmetic applied to it."""

    def __init__(self, expr):
        self.expr = expr

    def __matmul__(self, other):
        return SymTensor(("matmul", self.expr, _expr(other)))

    def __add__(self, other):
        return SymTensor(_canon("add", self.expr, _expr(other)))

    __radd__ = __add__

    def __mul__(self, other):
        if isinstance(other, (int, float)):
            return SymTensor(("scale", self.expr, float(other)))
        return SymTensor(_canon("mul", self.expr, _expr(other)))

    __rmul__ = __mul__

    def __sub__(self, other):
        return SymTensor(("sub", self.expr, _expr(other)))

    def __truediv__(self, other):
        return SymTensor(("div", self.expr, _expr(other)))

    @property
    def T(self):
        return SymTensor(("transpose", self.expr))


def _expr(v):
    if isinstance(v, SymTensor):
        return v.expr
    raise NotImplementedError("only traced tensors can be combined inside a traced program, got %s" % type(v).__name__)


_LEN_BASE = 1 << 40
_len_codes = {}  # tag of a traced sequence -> the integer its len() answered with


def _length_of(n):
    """The symbolic length an integer from len(traced sequence) stands for; other values as they are."""
    if isinstance(n, int) and n >= _LEN_BASE:
        for tag, code in _len_codes.items():
            if code == n:
                return ("len", tag)
        raise NotImplementedError("arithmetic on the length of a traced sequence")
    return n


class SymSeq(object):
    """Stand-in for a FractalTensor: either unrolled (``items``: a short static list, e.g. the four
    gates of a layer) or one representative element plus a tag that says where it comes from."""

    def __init__(self, elem=None, items=None, tag=None):
        self.elem, self.items, self.tag = elem, items, tag

    @property
    def length(self):
        return len(self.items) if self.items is not None else ("len", self.tag)

    def __len__(self):
        """len() must return an int: a traced sequence answers with a number that stands for its
        (symbolic) length, which repeat() turns back into the sequence it was asked of."""
        if self.items is not None:
            return len(self.items)
        if self.tag not in _len_codes:
            _len_codes[self.tag] = _LEN_BASE + len(_len_codes)
        return _len_codes[self.tag]

    def __iter__(self):
        if self.items is None:
            raise NotImplementedError("a traced sequence cannot be iterated or unpacked")
        return iter(self.items)

    def __getitem__(self, i):
        if self.items is not None:
            got = self.items[i]
            return SymSeq(items=got) if isinstance(i, slice) else got
        if isinstance(i, slice):
            if i.start not in (None, 0) or i.step is not None:
                raise NotImplementedError("only prefixes of a traced sequence can be sliced")
            return SymSeq(elem=self.elem, tag=("prefix", self.tag, i.stop))
        return self.elem  # any element of a traced sequence stands for all of them


def _desc(v):
    """Canonical, comparable description of a traced value."""
    if isinstance(v, SymTensor):
        return v.expr
    if isinstance(v, SymSeq):
        if v.items is not None:
            return ("list",) + tuple(_desc(x) for x in v.items)
        return ("seq", v.tag)
    if isinstance(v, tuple):
        return ("tuple",) + tuple(_desc(x) for x in v)
    raise NotImplementedError("cannot trace a value of type %s" % type(v).__name__)


def _is_sym(v):
    return isinstance(v, (SymTensor, SymSeq)) or (isinstance(v, tuple) and len(v) > 0 and builtins.all(_is_sym(x) for x in v))


def _split(results, make):
    """A traced function that returns a tuple yields a tuple of sequences, like the reference."""
    if isinstance(results, tuple):
        return tuple(make(results[j], j) for j in range(len(results)))
    return make(results, 0)


# ------------------------------------------------------------------- combinators
class SymInt(object):
    """Stand-in for the position that ops.enumerate hands to the folded function."""

    def __init__(self, expr):
        self.expr = expr

    def __rpow__(self, base):
        return SymInt(("pow", base, self.expr))


class _Enumerated(object):
    """enumerate of real FractalTensors, kept until the enclosing combinator dispatches."""

    def __init__(self, xs):
        self.xs = xs


def enumerate(*xs):
    if builtins.any(isinstance(x, SymSeq) for x in xs):
        raise NotImplementedError("enumerate of traced sequences")
    return _Enumerated(xs)


_seen = {}  # real parameter sets met inside the program being traced


class _Zipped(object):
    """zip of real FractalTensors, kept as is until the enclosing combinator dispatches."""

    def __init__(self, xs):
        self.xs = xs


def zip(*xs):
    if builtins.all(isinstance(x, SymSeq) for x in xs):
        if builtins.all(x.items is not None for x in xs):
            n = len(xs[0].items)
            if builtins.any(len(x.items) != n for x in xs):
                raise ValueError("zip of sequences of different lengths")
            return SymSeq(items=[tuple(x.items[k] for x in xs) for k in range(n)])
        if builtins.any(x.items is not None for x in xs):
            raise NotImplementedError("zip of an unrolled and a traced sequence")
        return SymSeq(elem=tuple(x.elem for x in xs), tag=("zip",) + tuple(x.tag for x in xs))
    if builtins.any(isinstance(x, SymSeq) for x in xs):
        raise NotImplementedError("zip of traced and real sequences")
    return _Zipped(xs)


def map(func, xs, **kwargs):
    if kwargs:
        raise NotImplementedError("map: keyword arguments are not supported")
    if isinstance(xs, _Zipped):
        return _dispatch_grid(func, xs) if len(xs.xs) == 2 else _dispatch_attention(func, xs)
    if not isinstance(xs, SymSeq) and hasattr(xs, "indices") and hasattr(xs, "data"):
        return _dispatch_dilated(func, xs)
    if not isinstance(xs, SymSeq):
        raise NotImplementedError("map over real data is only dispatched as part of a recognised program")
    if xs.items is not None:
        results = [func(it) for it in xs.items]
        if isinstance(results[0], tuple):
            return tuple(SymSeq(items=[r[j] for r in results]) for j in range(len(results[0])))
        return SymSeq(items=results)
    body = func(xs.elem)
    bdesc = _desc(body)
    return _split(body, lambda r, j: SymSeq(elem=r, tag=("map", xs.tag, bdesc, j)))


def scan(func, xs, initializer=None, **kwargs):
    if kwargs:
        raise NotImplementedError("scan: keyword arguments are not supported")
    if not isinstance(xs, SymSeq) or xs.items is not None:
        raise NotImplementedError("scan over real data is only dispatched as part of a recognised program")
    if initializer is None:
        raise NotImplementedError("scan without an initializer")
    init = initializer if isinstance(initializer, tuple) else (initializer,)

    def state_like(v, j):
        tag = ("state", xs.tag, j)
        if isinstance(v, SymSeq):
            return SymSeq(elem=SymTensor(("elem", tag)), tag=tag)
        return SymTensor(tag)

    state = tuple(state_like(v, j) for j, v in builtins.enumerate(init))
    body = func(state if isinstance(initializer, tuple) else state[0], xs.elem)
    idesc, bdesc = _desc(tuple(init)), _desc(body)
    return _split(body, lambda r, j: SymSeq(elem=r, tag=("scan", xs.tag, idesc, bdesc, j)))


def dilated_map(func, xs, dilation=1, **kwargs):
    """func applied to each of the `dilation` interleaved sub-sequences of xs, results merged back."""
    if kwargs:
        raise NotImplementedError("dilated_map: keyword arguments are not supported")
    if not isinstance(xs, SymSeq) or xs.items is not None:
        raise NotImplementedError("dilated_map over real data is only dispatched as part of a recognised program")
    d = dilation.expr if isinstance(dilation, SymInt) else int(dilation)
    sub = SymSeq(elem=xs.elem, tag=("every", d, xs.tag))
    body = func(sub)
    bdesc = _desc(body)
    return _split(body, lambda r, j: SymSeq(elem=r.elem if isinstance(r, SymSeq) else r,
                                            tag=("dilated_map", xs.tag, d, bdesc, j)))


def repeat(x, n):
    return SymSeq(elem=x, tag=("repeat", _desc(x), _length_of(n)))


def product(xs, ys):
    """Cartesian product as two grids: xss[i][j] = xs[j], yss[i][j] = ys[i]
    (kaleido/frontend/operations/fractaltensor/access.py:207-247)."""
    if not (isinstance(xs, SymSeq) and isinstance(ys, SymSeq)) or xs.items is not None or ys.items is not None:
        raise NotImplementedError("product over real data is only dispatched as part of a recognised program")
    xss = repeat(xs, ys.length)
    yss = SymSeq(elem=repeat(ys.elem, xs.length), tag=("rows", ys.tag, xs.length))
    return xss, yss


def cat(tensors, dim=0):
    return SymTensor(("cat", int(dim)) + tuple(_expr(t) for t in tensors))


def zeros(shape, device=None, dtype=None):
    return SymTensor(("zeros",))


def full(shape, fill_value, device=None, dtype=None):
    return SymTensor(("full", "lowest" if fill_value <= -3e38 else float(fill_value)))


def exp(x):
    return SymTensor(("exp", _expr(x)))


def maximum(x, y):
    return SymTensor(_canon("maximum", _expr(x), _expr(y)))


def max(x, dim=-1, keepdim=False):
    return SymTensor(("rowmax", _expr(x), dim, bool(keepdim)))


def sum(x, dim=-1, keepdim=False):
    return SymTensor(("rowsum", _expr(x), dim, bool(keepdim)))


def reduce(func, xs, initializer=None, **kwargs):
    """Like scan, but only the last state comes back (a tuple of tensors)."""
    if kwargs:
        raise NotImplementedError("reduce: keyword arguments are not supported")
    if not isinstance(xs, SymSeq) or xs.items is not None or initializer is None:
        raise NotImplementedError("reduce over real data is only dispatched as part of a recognised program")
    init = initializer if isinstance(initializer, tuple) else (initializer,)
    state = tuple(SymTensor(("state", xs.tag, j)) for j in range(len(init)))
    body = func(state if isinstance(initializer, tuple) else state[0], xs.elem)
    idesc, bdesc = _desc(tuple(init)), _desc(body)
    return _split(body, lambda r, j: SymTensor(("reduce", xs.tag, idesc, bdesc, j)))


def sigmoid(x):
    return SymTensor(("sigmoid", _expr(x)))


def tanh(x):
    return SymTensor(("tanh", _expr(x)))


# ------------------------------------------------------------ recognised programs
def _gate(w, u, b, x, s):
    return x @ w + s @ u + b


def _cell(h_prev, c_prev, x, ws, us, bs):
    pre = map(lambda p: _gate(*p, x, h_prev), zip(ws, us, bs))
    g = map(sigmoid, pre[:3])
    c = g[1] * c_prev + g[0] * tanh(pre[3])
    return g[2] * tanh(c), c


def _program_batch_major(embs, params):
    """fold(depth) of map(batch) of scan(time): stacked_lstm1.py."""
    def layer(xss, ws, us, bs):
        hss, _ = map(lambda xs: scan(lambda st, x: _cell(*st, x, ws, us, bs), xs, initializer=(zeros(()), zeros(()))), xss)
        return hss

    return layer(embs, *params)


def _program_time_major(embs, params):
    """fold(depth) of scan(time) of map(sequences still running): stacked_rnn.py."""
    def step(hs_prev, cs_prev, xs, ws, us, bs):
        return map(lambda t: _cell(*t, ws, us, bs), zip(hs_prev[0:xs.length], cs_prev[0:xs.length], xs))

    def layer(xss, ws, us, bs):
        init = repeat(zeros(()), xss[0].length)
        hss, _ = scan(lambda st, xs: step(*st, xs, ws, us, bs), xss, initializer=(init, init))
        return hss

    return layer(embs, *params)


def _program_attention(batch, scale):
    """map(batch) of map(heads) of map(query blocks) of reduce(key/value blocks): flash_attention.py."""
    def step(m_prev, l_prev, o_prev, q, k, v):
        w = q @ k.T
        if scale is not None:
            w = w * scale
        m_cur = max(w, dim=-1, keepdim=True)
        e = exp(w - m_cur)
        ev = e @ v
        l_cur = sum(e, dim=-1, keepdim=True)
        m_new = maximum(m_cur, m_prev)
        r_prev, r_cur = exp(m_prev - m_new), exp(m_cur - m_new)
        l_new = r_prev * l_prev + r_cur * l_cur
        return m_new, l_new, (o_prev * l_prev * r_prev + r_cur * ev) / l_new

    def block(q, ks, vs):
        init = (full((), -3.5e38), zeros(()), zeros(()))
        _, _, o = reduce(lambda st, kv: step(*st, q, *kv), zip(ks, vs), initializer=init)
        return o

    return map(lambda xss: map(lambda xs: map(lambda q: block(q, xs[1], xs[2]), xs[0]), zip(*xss)), batch)


def _deep_input(name, depth):
    tag = ("input", name)
    def build(t, d):
        return SymTensor(("elem", t)) if d == 0 else SymSeq(tag=t, elem=build(("elem", t), d - 1))
    return build(tag, depth)


def _find_scales(tree, out):
    if isinstance(tree, tuple):
        if len(tree) == 3 and tree[0] == "scale":
            out.add(tree[2])
        for x in tree:
            _find_scales(x, out)
    return out


def _dispatch_attention(func, zipped):
    def depth(ft):
        d, x = 0, getattr(ft, "indices", None)
        while isinstance(x, list):
            d, x = d + 1, (x[0] if x else None)
        return d

    if len(zipped.xs) != 3 or builtins.any(depth(x) != 3 for x in zipped.xs):
        raise NotImplementedError("map over real data: expected ops.zip(qsss, ksss, vsss) of depth-3 FractalTensors")

    def batch():
        return zip(*[_deep_input(n, 3) for n in ("q", "k", "v")])
    _len_codes.clear()
    traced = _desc(map(func, batch()))
    scales = _find_scales(traced, set())
    if len(scales) > 1:
        raise NotImplementedError("more than one constant factor in the program")
    scale = scales.pop() if scales else None
    if traced == _desc(_program_attention(batch(), scale)):
        q, k, v = zipped.xs
        return frontend.flash_attention(q, k, v, scale=1.0 if scale is None else scale)
    raise NotImplementedError("this program is not one the library has a fused kernel for, and there is no "
                              "element-by-element fallback")


def _program_dilated(embs, enumerated):
    """map(batch) of fold(layers) of dilated_map(scan(time)), dilation 2**layer: dilated_rnn.py."""
    def layer(state, position, ws, us, bs):
        h, _ = dilated_map(lambda xs: scan(lambda st, x: _cell(*st, x, ws, us, bs), xs, initializer=(zeros(()), zeros(()))),
                           state, dilation=2 ** position)
        return h

    return map(lambda xs: fold(lambda s, p: layer(s, *p), enumerated, initializer=xs), embs)


def _dispatch_dilated(func, embs):
    def symbolic():
        return _symbolic_inputs(3, 4)[0]

    _seen.clear()
    _len_codes.clear()
    traced = _desc(map(func, symbolic()))
    params = _seen.pop("enumerated", None)
    if params is not None and traced == _desc(_program_dilated(symbolic(), params)):
        Wss, Uss, bss = params.xs
        return frontend.dilated_lstm(embs, Wss, Uss, bss)
    raise NotImplementedError("this program is not one the library has a fused kernel for, and there is no "
                              "element-by-element fallback")


def _program_grid(pairs, stacked_params):
    """map(sentence pairs) of fold(depth) of scan(rows) of scan(columns) of the two-direction tanh
    cell on the src x trg grid: grid_rnn.py."""
    def cell(own, both, i2h, h2h, bias):
        return tanh(both @ i2h + own @ h2h + bias)

    def point(carry, cur, px, py):
        from_above, (x, y) = cur
        both = cat([from_above, carry[1]], dim=1)
        return cell(x, both, *px), cell(y, both, *py)

    def row(carry, cur, px, py):
        z = zeros(())
        return scan(lambda c, p: point(c, p, px, py), zip(carry[0], zip(cur[0], cur[1])), initializer=(z, z))

    def layer(grid, px, py):
        z = repeat(zeros(()), len(grid[0][0]))
        hx, hy = scan(lambda c, r: row(c, r, px, py), grid, initializer=(z, z))
        return zip(hx, hy)

    def pair(src, trg):
        xss, yss = product(src, trg)
        return fold(lambda g, p: layer(g, *p), stacked_params, initializer=zip(xss, yss))

    return map(lambda st: pair(st[0], st[1]), pairs)


def _dispatch_grid(func, zipped):
    def depth(ft):
        d, x = 0, getattr(ft, "indices", None)
        while isinstance(x, list):
            d, x = d + 1, (x[0] if x else None)
        return d

    if builtins.any(depth(x) != 2 for x in zipped.xs):
        raise NotImplementedError("map over real data: expected ops.zip(src_encs, trg_encs) of depth-2 FractalTensors")

    def pairs():
        return zip(_deep_input("src", 2), _deep_input("trg", 2))

    _seen.clear()
    _len_codes.clear()
    traced = _desc(map(func, pairs()))
    params = _seen.pop("grid_params", None)
    if params is not None and traced == _desc(_program_grid(pairs(), params)):
        src, trg = zipped.xs
        return frontend.stacked_grid_rnns(src, trg, params)
    raise NotImplementedError("this program is not one the library has a fused kernel for, and there is no "
                              "element-by-element fallback")


def _like(v, tag):
    """A fresh stand-in with the structure of v."""
    if isinstance(v, tuple):
        return tuple(_like(x, (tag, j)) for j, x in builtins.enumerate(v))
    if isinstance(v, SymSeq):
        return SymSeq(elem=_like(v.elem, ("elem", tag)), tag=tag)
    return SymTensor(tag)


def _is_grid_params(xs):
    def is_cell(c):
        return isinstance(c, (tuple, list)) and len(c) == 3

    return (isinstance(xs, (tuple, list)) and len(xs) > 0 and
            builtins.all(isinstance(b, (tuple, list)) and len(b) == 2 and is_cell(b[0]) and is_cell(b[1]) for b in xs))


def _symbolic_inputs(n_params, gates):
    seq = ("input", "state")
    inner = ("elem", seq)
    embs = SymSeq(tag=seq, elem=SymSeq(tag=inner, elem=SymTensor(("elem", inner))))
    params = tuple(SymSeq(items=[SymTensor(("param", p, k)) for k in range(gates)]) for p in range(n_params))
    return embs, params


def _inner_length(ft):
    idx = ft.indices
    return len(idx[0]) if idx and isinstance(idx[0], list) else None


def fold(func, xs, initializer=None, **kwargs):
    """``ops.fold(lambda s, param: layer(s, *param), ops.zip(Wss, Uss, bss), initializer=embs)``."""
    if kwargs:
        raise NotImplementedError("fold: keyword arguments are not supported")
    if isinstance(xs, _Enumerated) and isinstance(initializer, SymSeq):
        # Inside a traced program: fold over (position, one layer's parameters) of real parameters.
        if len(xs.xs) != 3 or builtins.any(_inner_length(p) != 4 for p in xs.xs):
            raise NotImplementedError("fold: expected ops.enumerate(Wss, Uss, bss) of [depth][4 gates] parameters")
        _seen["enumerated"] = xs
        state = SymSeq(elem=initializer.elem, tag=("state", "fold"))
        elem = (SymInt("position"),) + _symbolic_inputs(3, 4)[1]
        body = func(state, elem)
        return SymSeq(elem=body.elem, tag=("fold", _desc(initializer), _desc(body)))
    if _is_grid_params(xs) and isinstance(initializer, SymSeq):
        # Inside a traced program: fold over the layers' (x-direction, y-direction) cell parameters.
        _seen["grid_params"] = xs
        state = _like(initializer, ("state", "fold"))
        elem = tuple(tuple(SymTensor(("param", d, k)) for k in range(3)) for d in range(2))
        body = func(state, elem)
        if not isinstance(body, SymSeq):
            raise NotImplementedError("fold: the folded function must return a sequence")
        return SymSeq(elem=body.elem, tag=("fold", _desc(initializer), _desc(body)))
    if isinstance(xs, SymSeq) or _is_sym(initializer):
        raise NotImplementedError("a fold inside a traced program is not recognised")
    if not isinstance(xs, _Zipped) or len(xs.xs) != 3 or initializer is None:
        raise NotImplementedError("fold: expected ops.zip(Wss, Uss, bss) and an initializer (the stacked LSTM)")
    Wss, Uss, bss = xs.xs
    if builtins.any(_inner_length(p) != 4 for p in (Wss, Uss, bss)):
        raise NotImplementedError("fold: the parameters are not [depth][4 gates] FractalTensors")
    embs_sym, params_sym = _symbolic_inputs(3, 4)
    _len_codes.clear()
    traced = _desc(func(embs_sym, params_sym))
    if traced == _desc(_program_batch_major(*_symbolic_inputs(3, 4))):
        return frontend.stacked_lstm(initializer, Wss, Uss, bss)
    if traced == _desc(_program_time_major(*_symbolic_inputs(3, 4))):
        return frontend.stacked_lstm_time_major(initializer, Wss, Uss, bss)
    raise NotImplementedError("this program is not one the library has a fused kernel for, and there is no "
                              "element-by-element fallback")
