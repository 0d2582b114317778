"""GPU parity of the token-level sparse attention (dilated window + random + global keys) with the
oracle and with the fixture the reference's frontend produced
(examples/sparse_attention/sparse_attention.py:24-76)."""
import os

import numpy as np
import pytest
import torch

from oracle import dense

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from fractaltensor_b200 import ops as _ops
    return _ops


def _load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name))
    return {k: (torch.from_numpy(z[k]) if z[k].ndim > 0 else z[k].item()) for k in z.files}


def _inputs(B, heads, S, d, ng, R, seed, dt):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.rand(B, heads, S, d, generator=g).to(dt) for _ in range(3))
    pos = torch.randint(0, S, (B, heads, S - 2 * ng, max(R, 1)), generator=g, dtype=torch.int32)[..., :R].contiguous()
    return q, k, v, pos


def test_sparse_attention_golden(ops, golden_dir):
    """What the reference's frontend returns for per_head_attn (softmax over dimension 0, as shipped)."""
    g = _load(golden_dir, "sparse_attention_small.npz")
    ws, dil = int(g["window_size"]), int(g["dilation"])
    q, k, v = (g[n][None, None].contiguous().cuda() for n in ("q", "k", "v"))
    pos = g["rand_pos"].to(torch.int32)[None, None].contiguous().cuda()
    out = ops.sparse_attention(q, k, v, pos, ws, dil, as_shipped=True)
    ops.check_status()
    assert (out[0, 0].cpu() - g["out"]).abs().max().item() <= 1e-5
    # the attention the example describes, against the oracle
    att = ops.sparse_attention(q, k, v, pos, ws, dil)
    ref = dense.sparse_attention_dense(g["q"].double(), g["k"].double(), g["v"].double(), g["rand_pos"], ws, dil)
    assert (att[0, 0].cpu().double() - ref).abs().max().item() <= 1e-5


def test_sparse_attention_frontend_nestings(ops, golden_dir):
    """The model-level signature: FractalTensors of [1, d] tokens, one head or [B][heads][S]."""
    from fractaltensor_b200 import frontend
    g = _load(golden_dir, "sparse_attention_small.npz")
    ws, dil = int(g["window_size"]), int(g["dilation"])
    S, d = g["q"].shape
    ft = lambda t, depth: frontend.FractalTensor.from_dense(t.cuda(), depth)
    one = frontend.sparse_attention(ft(g["q"][:, None], 1), ft(g["k"][:, None], 1), ft(g["v"][:, None], 1),
                                    ft(g["rand_pos"][:, None], 1), ws, dil, as_shipped=True)
    assert len(one) == S and one.element_shape == (1, d)
    assert (one.to_dense()[:, 0].cpu() - g["out"]).abs().max().item() <= 1e-5
    B, heads = 2, 3
    q, k, v, pos = _inputs(B, heads, S, d, 3, 3, 5, torch.float32)
    many = frontend.sparse_attention(ft(q[:, :, :, None], 3), ft(k[:, :, :, None], 3), ft(v[:, :, :, None], 3),
                                     ft(pos[:, :, :, None], 3), ws, dil)
    ops.check_status()
    assert many.depth == 3 and many.element_shape == (1, d)
    ref = dense.sparse_attention_dense(q.double(), k.double(), v.double(), pos, ws, dil)
    assert (many.to_dense()[:, :, :, 0].cpu().double() - ref).abs().max().item() <= 1e-5


CASES = [
    # B, heads, S, d, window, dilation, n_global, R
    (1, 1, 16, 64, 5, 2, 3, 3),      # the example's own sizes
    (2, 4, 64, 64, 5, 2, 3, 3),
    (1, 2, 33, 32, 1, 1, 0, 0),      # a window of the token itself, nothing else
    (1, 2, 40, 128, 7, 3, 1, 5),
    (2, 1, 50, 256, 3, 1, 4, 0),     # no random keys
    (1, 3, 128, 64, 31, 2, 16, 33),  # 64 keys per windowed token, 32 global keys
    (1, 1, 12, 64, 5, 2, 6, 2),      # every token is global
    (1, 2, 70, 64, 9, 4, 32, 1),     # 64 global keys: two per lane
    (2, 3, 300, 64, 5, 2, 3, 3),     # the example's key counts: interior tiles by the kernel built for them
    (1, 2, 300, 128, 5, 3, 2, 3),    # the same with dilation 3 and 128 elements per head
    (1, 2, 1000, 32, 5, 1, 0, 3),    # no global tokens, dilation 1
    (1, 1, 200, 256, 5, 2, 30, 3),   # 60 global keys, 256 elements per head
]


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shipped", [False, True])
@pytest.mark.parametrize("case", CASES)
def test_sparse_attention_matches_oracle(ops, dt, shipped, case):
    B, heads, S, d, ws, dil, ng, R = case
    q, k, v, pos = _inputs(B, heads, S, d, ng, R, S * 7 + d + R, dt)
    scale = 1.0 if shipped else 0.25
    out = ops.sparse_attention(q.cuda(), k.cuda(), v.cuda(), pos.cuda() if R else None, ws, dil, ng, scale=scale,
                               as_shipped=shipped)
    ops.check_status()
    ref = dense.sparse_attention_dense(q.double() * scale, k.double(), v.double(),
                                       pos if R else torch.zeros(B, heads, S - 2 * ng, 0, dtype=torch.int32), ws, dil,
                                       ng, as_shipped=shipped)
    # fp32 arithmetic everywhere; 16-bit types round the stored output once (2^-11 / 2^-8 relative)
    rel = {torch.float32: 2e-6, torch.float16: 6e-4, torch.bfloat16: 5e-3}[dt]
    err = (out.cpu().double() - ref).abs().max().item()
    assert err <= rel * max(1.0, ref.abs().max().item()), err


def test_sparse_attention_full_size(ops):
    """The sizes the example names for real use (sequence 4096, 16 heads of 64, batch 2), fp32, every
    token compared with the oracle; and the shipped form against a plain gather-and-sum."""
    B, heads, S, d, ws, dil, ng, R = 2, 16, 4096, 64, 5, 2, 3, 3
    q, k, v, pos = _inputs(B, heads, S, d, ng, R, 77, torch.float32)
    out = ops.sparse_attention(q.cuda(), k.cuda(), v.cuda(), pos.cuda(), ws, dil, ng, scale=0.125)
    ops.check_status()
    ref = dense.sparse_attention_dense(q * 0.125, k, v, pos, ws, dil, ng)
    assert (out.cpu() - ref).abs().max().item() <= 2e-5
    shipped = ops.sparse_attention(q.cuda(), k.cuda(), v.cuda(), pos.cuda(), ws, dil, ng, as_shipped=True)
    half = (ws - 1) * dil // 2
    i = torch.arange(ng, S - ng)
    win = i[:, None] - half + torch.arange(ws)[None, :] * dil
    win = torch.where(win < 0, win + S - 1, torch.where(win >= S, win - S, win))
    idx = torch.cat([win.expand(B, heads, -1, -1), pos.long()], dim=-1)            # [B, heads, S - 6, ws + R]
    total = torch.zeros(B, heads, S - 2 * ng, d)
    for j in range(ws + R):
        total += torch.gather(v, 2, idx[..., j, None].expand(-1, -1, -1, d))
    assert (shipped[:, :, ng:S - ng].cpu() - total).abs().max().item() <= 1e-5


def test_sparse_attention_bad_position_sets_status(ops):
    q, k, v, pos = _inputs(1, 1, 16, 64, 3, 3, 3, torch.float32)
    pos[0, 0, 4, 1] = 16
    out = ops.sparse_attention(q.cuda(), k.cuda(), v.cuda(), pos.cuda())
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    from fractaltensor_b200._lib import FtbError
    with pytest.raises(FtbError) as e:
        ops.check_status()
    assert e.value.code == 22
    ops.check_status()  # the word was cleared by the failed check


def test_sparse_attention_rejects_host_tensors(ops):
    q, k, v, pos = _inputs(1, 1, 16, 64, 3, 3, 3, torch.float32)
    with pytest.raises(RuntimeError):
        ops.sparse_attention(q, k, v, pos)
    with pytest.raises(ValueError):
        ops.sparse_attention(q.cuda(), k.cuda(), v.cuda(), pos.cuda().long())


def test_sparse_attention_empty_batch_and_single_tile_edges(ops):
    """No heads at all is a no-op; a sequence of exactly one tile with every kind of token in it."""
    q = torch.empty(0, 4, 64, 64, device="cuda")
    pos = torch.empty(0, 4, 58, 3, dtype=torch.int32, device="cuda")
    out = ops.sparse_attention(q, q.clone(), q.clone(), pos)
    ops.check_status()
    assert out.shape == q.shape
    q, k, v, pos = _inputs(3, 2, 64, 64, 3, 3, 9, torch.float32)
    out = ops.sparse_attention(q.cuda(), k.cuda(), v.cuda(), pos.cuda())
    ops.check_status()
    ref = dense.sparse_attention_dense(q.double(), k.double(), v.double(), pos)
    assert (out.cpu().double() - ref).abs().max().item() <= 2e-6 * max(1.0, ref.abs().max().item())
