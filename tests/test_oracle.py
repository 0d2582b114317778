"""The dense oracle against the golden vectors produced by the reference's own
frontend (tests/golden/generate.py) and against closed forms."""
import math
import os

import numpy as np
import torch

from oracle import dense


def _load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name))
    return {k: (torch.from_numpy(z[k]) if z[k].ndim > 0 else z[k].item()) for k in z.files}


def test_stacked_lstm_small_matches_reference_frontend(golden_dir):
    g = _load(golden_dir, "stacked_lstm_small.npz")
    hs, _ = dense.stacked_lstm_dense(g["x"], g["W"], g["U"], g["b"])
    assert torch.allclose(hs[-1], g["top"], rtol=1e-5, atol=1e-6)
    assert (hs[-1] - g["top"]).abs().max().item() <= 1e-6


def test_stacked_lstm_config1_matches_reference_frontend(golden_dir):
    """benchmark config 1 at full size (D4, H256, N32, L64, seed 0): the fixture holds
    two samples of the frontend's output; samples are independent."""
    g = _load(golden_dir, "stacked_lstm_config1_samples.npz")
    x, W, U, _ = dense.make_lstm_inputs(4, 64, 32, 256, 256, 0, 1.0 / 16)
    idx = g["samples"].long()
    # in float64: the fp32 evaluation on a multi-threaded host is not reproducible to this bound
    hs, _ = dense.stacked_lstm_dense(x[:, idx].double(), W.double(), U.double())
    err = (hs[-1] - g["top"]).abs().max().item()
    assert err <= 1e-5 * g["top"].abs().max().item(), err


def test_stacked_lstm_varlen_matches_reference_frontend(golden_dir):
    """Length-sorted ragged batch through the reference's time-major program."""
    g = _load(golden_dir, "stacked_lstm_varlen_small.npz")
    hs, _ = dense.stacked_lstm_varlen_dense(g["x"], g["active_rows"].tolist(), g["W"], g["U"], g["b"])
    assert (hs[-1] - g["top"]).abs().max().item() <= 1e-6


def test_stacked_lstm_varlen_equals_per_sequence_runs():
    """Each sequence of the ragged batch sees only its own steps: running it alone, as a
    rectangular batch of one, gives the same rows and the same final cell state."""
    D, L, N, H = 2, 6, 4, 8
    active = dense.make_active_rows(L, N, 5)
    T = sum(active)
    x, W, U, b = dense.make_lstm_inputs(D, T, 1, H, H, 5, 0.3, bias=True)
    x = x.reshape(T, H)
    hs, cs = dense.stacked_lstm_varlen_dense(x, active, W, U, b)
    off = np.concatenate([[0], np.cumsum(active)])
    for n in range(N):
        steps = [t for t in range(L) if active[t] > n]
        rows = [int(off[t]) + n for t in steps]
        h1, c1 = dense.stacked_lstm_dense(x[rows][:, None], W, U, b)
        assert torch.allclose(hs[:, rows], h1[:, :, 0], atol=1e-6)
        assert torch.allclose(cs[:, n], c1[:, 0], atol=1e-6)
    # equal lengths: the rectangular program
    hs2, cs2 = dense.stacked_lstm_varlen_dense(x[:L * 2], [2] * L, W, U, b)
    h3, c3 = dense.stacked_lstm_dense(x[:L * 2].reshape(L, 2, H), W, U, b)
    assert torch.equal(hs2.reshape(D, L, 2, H), h3) and torch.equal(cs2, c3)


def test_dilated_lstm_matches_reference_frontend(golden_dir):
    g = _load(golden_dir, "dilated_lstm_small.npz")
    hs = dense.dilated_lstm_dense(g["x"], g["W"], g["U"], g["dilations"].tolist())
    assert (hs[-1] - g["top"]).abs().max().item() <= 1e-6


def test_grid_rnn_matches_reference_frontend(golden_dir):
    g = _load(golden_dir, "grid_rnn_small.npz")
    hx, hy = dense.grid_rnn_dense(g["X"], g["Y"], g["i2h_x"], g["h2h_x"], g["b_x"], g["i2h_y"], g["h2h_y"], g["b_y"])
    assert (hx[-1] - g["hx_top"]).abs().max().item() <= 1e-6
    assert (hy[-1] - g["hy_top"]).abs().max().item() <= 1e-6


def test_flash_attention_matches_reference_frontend(golden_dir):
    g = _load(golden_dir, "flash_attention_small.npz")
    o = dense.flash_attention_dense(g["q"], g["k"], g["v"], scale=g["scale"], block=int(g["block"]))
    assert (o - g["o"]).abs().max().item() <= 2e-6
    # and the carry equals the closed form
    ref = dense.attention_plain(g["q"], g["k"], g["v"], scale=g["scale"])
    assert (o - ref).abs().max().item() <= 2e-6


def test_causal_attention_blockwise_equals_closed_form():
    q, k, v = dense.make_attention_inputs(1, 2, 128, 16, 7, dtype=torch.float32)
    ref = dense.attention_plain(q.double(), k.double(), v.double(), scale=0.25, causal=True)
    for block in (16, 32, 128):
        o = dense.flash_attention_causal_dense(q.double(), k.double(), v.double(), scale=0.25, block=block)
        assert (o - ref).abs().max().item() <= 1e-12
    # row 0 attends to key 0 only
    assert torch.equal(ref[:, :, 0], v.double()[:, :, 0])
    # a window of one key: every query returns its own value; a window of S keys: plain causal
    one = dense.attention_plain(q.double(), k.double(), v.double(), scale=0.25, causal=True, window=1)
    assert (one - v.double()).abs().max().item() <= 1e-12
    full = dense.attention_plain(q.double(), k.double(), v.double(), scale=0.25, causal=True, window=128)
    assert torch.equal(full, ref)
    # two-sided windows: (S, 0) is causal, (S, S) is unmasked, (w-1, 0) is the one-sided window w
    qd, kd, vd = q.double(), k.double(), v.double()
    assert torch.equal(dense.attention_plain(qd, kd, vd, scale=0.25, local=(128, 0)), ref)
    assert torch.equal(dense.attention_plain(qd, kd, vd, scale=0.25, local=(128, 128)),
                       dense.attention_plain(qd, kd, vd, scale=0.25))
    assert torch.equal(dense.attention_plain(qd, kd, vd, scale=0.25, local=(6, 0)),
                       dense.attention_plain(qd, kd, vd, scale=0.25, causal=True, window=7))


def test_flash_attention_block_size_does_not_matter():
    q, k, v = dense.make_attention_inputs(1, 2, 128, 16, 7, dtype=torch.float32)
    a = dense.flash_attention_dense(q, k, v, scale=0.25, block=32)
    b = dense.flash_attention_dense(q, k, v, scale=0.25, block=128)
    assert (a - b).abs().max().item() <= 2e-6


def test_b2b_rounds_the_intermediate():
    """P = A.B is rounded to fp16 before the second product (cutlass_wmma.h:512-517)."""
    A, B, C = dense.make_b2b_inputs(2, 64, 128, 128, 128, 1)
    out = dense.b2b_gemm_dense(A, B, C)
    assert out.dtype == torch.float16 and tuple(out.shape) == (2, 64, 128)
    P = (A.double() @ B.double().transpose(-1, -2)).half()
    want = (P.double() @ C.double().transpose(-1, -2)).half()
    assert (out.float() - want.float()).abs().max().item() <= 2e-3
    unrounded = (A.double() @ B.double().transpose(-1, -2) @ C.double().transpose(-1, -2))
    assert (out.double() - unrounded).abs().max().item() > 0


def test_lstm_zero_weights_closed_form():
    """With zero weights every gate is sigmoid(0)=0.5 / tanh(0)=0: c and h stay 0."""
    x = torch.randn(3, 2, 8)
    W = torch.zeros(2, 4, 8, 8)
    U = torch.zeros(2, 4, 8, 8)
    hs, c = dense.stacked_lstm_dense(x, W, U)
    assert hs.abs().max().item() == 0 and c.abs().max().item() == 0


def test_dilation_one_equals_stacked():
    x, W, U, _ = dense.make_lstm_inputs(2, 7, 3, 8, 8, 5, 0.3)
    a, _ = dense.stacked_lstm_dense(x, W, U)
    b = dense.dilated_lstm_dense(x, W, U, [1, 1])
    assert torch.equal(a, b)


def test_seeded_inputs_are_deterministic():
    a = dense.make_lstm_inputs(1, 2, 2, 4, 4, 3, 1 / 32)[0]
    b = dense.make_lstm_inputs(1, 2, 2, 4, 4, 3, 1 / 32)[0]
    assert torch.equal(a, b)
    q1 = dense.make_attention_inputs(1, 1, 4, 4, 2)[0]
    q2 = dense.make_attention_inputs(1, 1, 4, 4, 2)[0]
    assert torch.equal(q1, q2)
    assert abs(dense.make_b2b_inputs(1, 256, 128, 128, 128, 1)[0].float().std().item() - 1 / math.sqrt(128)) < 0.01


def test_online_softmax_is_softmax_with_a_clamp():
    """The reference checks its online softmax against its plain softmax (and rows against 1):
    the same here, plus the clamp at x - max = -64 that only the online kernel has."""
    g = torch.Generator().manual_seed(9)
    for rows, width in ((2, 7), (2, 517), (2, 1027)):  # the reference test's shapes
        x = torch.randn(rows, width, generator=g)
        y = dense.online_softmax_dense(x)
        assert torch.allclose(y, torch.softmax(x, dim=1), atol=1e-7)
        assert torch.allclose(y.sum(dim=1), torch.ones(rows), atol=1e-5)
    x = torch.tensor([[0.0, -100.0, -64.0]])
    y = dense.online_softmax_dense(x)
    d = 1.0 + math.exp(-100.0) + math.exp(-64.0)
    assert abs(y[0, 1].item() - math.exp(-64.0) / d) < 1e-35 and y[0, 1].item() > 0


def test_embedding_lookup_matches_reference_frontend(golden_dir):
    """ops.index(ops.slices(embedding, dim=0), word) mapped over a ragged batch of word sequences."""
    g = _load(golden_dir, "embedding_small.npz")
    rows = dense.embedding_gather_dense(g["table"], g["ids"])
    assert torch.equal(rows, g["rows"])


def test_projection_softmax_matches_reference_frontend(golden_dir):
    """softmax(h @ prev_softmax_proj) per word position, as the reference's Tensor @ and ops.softmax
    compute it on a ragged batch of hidden states."""
    g = _load(golden_dir, "projection_small.npz")
    out = dense.project_softmax_dense(g["h"], g["proj"])
    assert out.shape == g["probs"].shape
    assert (out - g["probs"]).abs().max().item() <= 1e-6
    assert (out.sum(dim=1) - 1).abs().max().item() <= 1e-5


def test_sparse_attention_matches_reference_frontend(golden_dir):
    """per_head_attn of the sparse attention example run through the reference's own shifted_slide,
    filter, join, split and softmax (window 5, dilation 2, 3 random keys, 3 + 3 global tokens).  The
    fixture holds what that program returns, which normalises dimension 0 (as_shipped)."""
    g = _load(golden_dir, "sparse_attention_small.npz")
    ws, dil = int(g["window_size"]), int(g["dilation"])
    out = dense.sparse_attention_dense(g["q"], g["k"], g["v"], g["rand_pos"], ws, dil, as_shipped=True)
    assert out.shape == g["out"].shape
    assert (out - g["out"]).abs().max().item() <= 1e-6
    # the attention the example describes: a convex combination of the gathered values per token
    att = dense.sparse_attention_dense(g["q"], g["k"], g["v"], g["rand_pos"], ws, dil)
    assert att.min().item() >= g["v"].min().item() - 1e-6 and att.max().item() <= g["v"].max().item() + 1e-6
    # windowed tokens of the shipped form are plain sums of window + R value rows
    S = g["q"].shape[0]
    i, half = 5, (ws - 1) * dil // 2
    rows = [x + S - 1 if x < 0 else (x - S if x >= S else x) for x in range(i - half, i + half + 1, dil)]
    rows += g["rand_pos"][i - 3].tolist()
    assert torch.allclose(g["out"][i], g["v"][rows].sum(dim=0), atol=1e-5)


def test_rnn_attention_matches_reference_frontend(golden_dir):
    """The attention RNN (tanh encoder scan, attention scan over the targets) run through the
    reference's own scan / map / reduce / softmax / scale / add on ragged batches."""
    g = _load(golden_dir, "rnn_attention_small.npz")
    enc, out = dense.rnn_attention_dense(g["src"], g["trg"], g["src_lens"], g["trg_lens"], g["Ws"], g["Us"], g["bs"],
                                         g["Wt"], g["Ut"], g["bt"], g["enc_proj"], g["dec_proj"])
    assert enc.shape == g["enc"].shape and out.shape == g["out"].shape
    assert (enc - g["enc"]).abs().max().item() <= 1e-6
    assert (out - g["out"]).abs().max().item() <= 1e-6
