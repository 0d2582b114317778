"""GPU parity of the attention RNN (examples/rnn_attention/rnn_attention.py:40-110) with the oracle
and with the fixture the reference's frontend produced."""
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


def _ragged(flat, lens):
    from fractaltensor_b200 import frontend
    return frontend.FractalTensor(flat.cuda(), [list(range(int(n))) for n in lens], (1, flat.shape[1]))


def _params(H, seed, bound):
    g = torch.Generator().manual_seed(seed)
    uni = lambda *s: (torch.rand(*s, generator=g) * 2 - 1) * bound
    return dict(Ws=uni(H, H), Us=uni(H, H), bs=uni(1, H), Wt=uni(H, H), Ut=uni(H, H), bt=uni(1, H),
                enc_proj=torch.rand(H, 1, generator=g), dec_proj=torch.rand(H, 1, generator=g)), g


def test_rnn_attention_golden(ops, golden_dir):
    """The reference frontend's own result on ragged batches (H = 16 there; the kernels take multiples
    of 64, so the fixture's parameters are embedded in H = 64 with zeros, which leaves the first 16
    columns of every state unchanged)."""
    from fractaltensor_b200 import frontend
    g = _load(golden_dir, "rnn_attention_small.npz")
    h, H = g["src"].shape[1], 64
    pad_m = lambda m: torch.nn.functional.pad(m, (0, H - m.shape[1], 0, H - m.shape[0]))
    pad_r = lambda m: torch.nn.functional.pad(m, (0, H - m.shape[1]))
    pad_c = lambda m: torch.nn.functional.pad(m, (0, 0, 0, H - m.shape[0]))
    # padded units: zero weights and zero bias -> tanh(0) = 0 everywhere, and zero projection rows
    src, trg = _ragged(pad_r(g["src"]), g["src_lens"]), _ragged(pad_r(g["trg"]), g["trg_lens"])
    out = frontend.rnn_attention(src, trg, (pad_m(g["Ws"]).cuda(), pad_m(g["Us"]).cuda(), pad_r(g["bs"]).cuda()),
                                 (pad_m(g["Wt"]).cuda(), pad_m(g["Ut"]).cuda(), pad_r(g["bt"]).cuda()),
                                 (pad_c(g["enc_proj"]).cuda(), pad_c(g["dec_proj"]).cuda()))
    ops.check_status()
    assert [len(i) for i in out.indices] == g["trg_lens"].tolist() and out.element_shape == (1, H)
    got = out.data.reshape(-1, H).cpu()
    assert (got[:, :h] - g["out"]).abs().max().item() <= 1e-5
    assert got[:, h:].abs().max().item() == 0


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("H,src_lens,trg_lens", [
    (64, [5, 3, 7], [4, 6, 2]),
    (128, [9] * 4, [5] * 4),                       # rectangular
    (256, list(range(1, 41)), list(range(40, 0, -1))),  # 40 sequences, lengths 1..40
    (512, [30, 17, 50, 50, 2, 41, 8], [20, 33, 5, 12, 40, 1, 9]),  # the example's hidden size and batch
])
def test_rnn_attention_matches_oracle(ops, dt, H, src_lens, trg_lens):
    from fractaltensor_b200 import frontend
    p, g = _params(H, H + len(src_lens), 1.0 / (H ** 0.5))
    src = torch.randn(sum(src_lens), H, generator=g).to(dt)
    trg = torch.randn(sum(trg_lens), H, generator=g).to(dt)
    pq = {k: v.to(dt) for k, v in p.items()}
    out = frontend.rnn_attention(_ragged(src, src_lens), _ragged(trg, trg_lens),
                                 (pq["Ws"].cuda(), pq["Us"].cuda(), pq["bs"].cuda()),
                                 (pq["Wt"].cuda(), pq["Ut"].cuda(), pq["bt"].cuda()),
                                 (pq["enc_proj"].cuda(), pq["dec_proj"].cuda()))
    ops.check_status()
    d64 = {k: v.double() for k, v in pq.items()}
    _, ref = dense.rnn_attention_dense(src.double(), trg.double(), src_lens, trg_lens, d64["Ws"], d64["Us"], d64["bs"],
                                       d64["Wt"], d64["Ut"], d64["bt"], d64["enc_proj"], d64["dec_proj"])
    got = out.data.reshape(-1, H).cpu().double()
    err = (got - ref).abs().max().item()
    if dt == torch.float32:
        assert err <= 1e-5 * max(1.0, ref.abs().max().item()), err
    else:
        assert err <= 2e-2, err


def test_rnn_attention_dense_entry(ops):
    """The tensor-level entry on a rectangular time-major batch without lengths, encoder states included."""
    H, Ls, Lt, N = 128, 12, 7, 130
    p, g = _params(H, 5, 1.0 / (H ** 0.5))
    dt = torch.bfloat16
    src, trg = torch.randn(Ls, N, H, generator=g).to(dt), torch.randn(Lt, N, H, generator=g).to(dt)
    pq = {k: v.to(dt) for k, v in p.items()}
    enc, out = ops.rnn_attention(src.cuda(), trg.cuda(), ops.rnn_pack_weights(pq["Ws"].cuda(), pq["Us"].cuda()),
                                 ops.rnn_pack_weights(pq["Wt"].cuda(), pq["Ut"].cuda()),
                                 pq["bs"].reshape(H).float().cuda(), pq["bt"].reshape(H).float().cuda(),
                                 pq["enc_proj"].reshape(H).cuda(), pq["dec_proj"].reshape(H).cuda())
    ops.check_status()
    d64 = {k: v.double() for k, v in pq.items()}
    for n in (0, 64, 129):
        e_ref, o_ref = dense.rnn_attention_dense(src[:, n].double(), trg[:, n].double(), [Ls], [Lt], d64["Ws"], d64["Us"],
                                                 d64["bs"], d64["Wt"], d64["Ut"], d64["bt"], d64["enc_proj"],
                                                 d64["dec_proj"])
        assert (enc[:, n].cpu().double() - e_ref).abs().max().item() <= 2e-2
        assert (out[:, n].cpu().double() - o_ref).abs().max().item() <= 2e-2


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_rnn_attention_smallest_shapes(ops, dt):
    """One sequence, one source and one target position; and a batch that is not a multiple of any tile."""
    from fractaltensor_b200 import frontend
    for src_lens, trg_lens in (([1], [1]), ([1, 2, 1], [2, 1, 3])):
        H = 64
        p, g = _params(H, 3 + len(src_lens), 1.0 / (H ** 0.5))
        src = torch.randn(sum(src_lens), H, generator=g).to(dt)
        trg = torch.randn(sum(trg_lens), H, generator=g).to(dt)
        pq = {k: v.to(dt) for k, v in p.items()}
        out = frontend.rnn_attention(_ragged(src, src_lens), _ragged(trg, trg_lens),
                                     (pq["Ws"].cuda(), pq["Us"].cuda(), pq["bs"].cuda()),
                                     (pq["Wt"].cuda(), pq["Ut"].cuda(), pq["bt"].cuda()),
                                     (pq["enc_proj"].cuda(), pq["dec_proj"].cuda()))
        ops.check_status()
        d64 = {k: v.double() for k, v in pq.items()}
        _, ref = dense.rnn_attention_dense(src.double(), trg.double(), src_lens, trg_lens, d64["Ws"], d64["Us"],
                                           d64["bs"], d64["Wt"], d64["Ut"], d64["bt"], d64["enc_proj"], d64["dec_proj"])
        err = (out.data.reshape(-1, H).cpu().double() - ref).abs().max().item()
        assert err <= (1e-5 if dt == torch.float32 else 2e-2), err
        # with a single source position the attention vector is that encoder state, whatever the scores
        if src_lens == [1]:
            enc1 = torch.tanh(src.double() @ d64["Ws"] + d64["bs"])
            assert (out.data.reshape(-1, H).cpu().double() - enc1).abs().max().item() <= (1e-5 if dt == torch.float32 else 2e-2)
