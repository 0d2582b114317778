"""Host-side logic that needs no GPU: FractalTensor views, batch sharding, and
the two-rank gather over gloo."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fractaltensor_b200 import frontend, sharding


def test_fractaltensor_dense_roundtrip():
    t = torch.arange(2 * 3 * 4.0).reshape(2, 3, 1, 4)
    ft = frontend.FractalTensor.from_dense(t, 2)
    assert ft.depth == 2 and len(ft) == 2 and ft.element_shape == (1, 4)
    assert ft.indices == [[0, 1, 2], [0, 1, 2]]
    assert torch.equal(ft.to_dense(), t)


def test_ragged_nesting_is_rejected():
    ft = frontend.FractalTensor(torch.zeros(5 * 4), [[0, 1, 2], [0, 1]], (1, 4))
    with pytest.raises(ValueError, match="ragged"):
        ft.to_dense()


def test_ragged_batches_are_routed_not_densified():
    """The stacked LSTM takes ragged batches; with CPU data the call must stop at the device
    check (no CPU path), not at the nesting check."""
    x = frontend.FractalTensor(torch.zeros(5 * 64), [[0, 1, 2], [0, 1]], (1, 64))
    w = frontend.FractalTensor.from_dense(torch.zeros(1, 4, 64, 64), 2)
    b = frontend.FractalTensor.from_dense(torch.zeros(1, 4, 1, 64), 2)
    with pytest.raises(RuntimeError, match="no CPU path"):
        frontend.stacked_lstm(x, w, w, b)
    with pytest.raises(RuntimeError, match="no CPU path"):
        frontend.stacked_lstm_time_major(x, w, w, b)
    with pytest.raises(ValueError, match="ragged"):
        frontend.dilated_lstm(x, w, w, b)


def test_cpu_tensors_are_rejected_not_computed():
    x = frontend.FractalTensor.from_dense(torch.zeros(2, 3, 1, 64), 2)
    w = frontend.FractalTensor.from_dense(torch.zeros(1, 4, 64, 64), 2)
    b = frontend.FractalTensor.from_dense(torch.zeros(1, 4, 1, 64), 2)
    with pytest.raises(RuntimeError, match="no CPU path"):
        frontend.stacked_lstm(x, w, w, b)
    from fractaltensor_b200 import ops
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.gemm_nt(torch.zeros(128, 64), torch.zeros(128, 64))


@pytest.mark.parametrize("n,world", [(256, 1), (256, 2), (256, 8), (10, 4), (3, 4)])
def test_shard_range_partitions_the_batch(n, world):
    spans = [sharding.shard_range(n, r, world) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == n
    for (a, b), (c, d) in zip(spans, spans[1:]):
        assert b == c and b - a >= d - c >= b - a - 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, n, dim, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    full_shape = [4, 4, 4]
    full_shape[dim] = n
    full = torch.arange(float(torch.tensor(full_shape).prod())).reshape(full_shape)
    local = sharding.shard_batch(full, dim, rank, world) * 1.0
    out = sharding.gather_batch(local, dim, n, None)
    q.put((rank, bool(torch.equal(out, full))))
    dist.destroy_process_group()


@pytest.mark.parametrize("n,dim", [(8, 0), (7, 1)])
def test_two_rank_shard_and_gather_gloo(n, dim):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, n, dim, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, True), (1, True)]


# ----------------------------------------------------- program tracing and dispatch
def test_programs_are_recognised_and_routed(monkeypatch):
    from fractaltensor_b200 import operations as ops
    calls = []
    monkeypatch.setattr(frontend, "stacked_lstm", lambda *a: calls.append("batch") or "B")
    monkeypatch.setattr(frontend, "stacked_lstm_time_major", lambda *a: calls.append("time") or "T")
    embs = frontend.FractalTensor.from_dense(torch.zeros(2, 3, 1, 64), 2)
    w = frontend.FractalTensor.from_dense(torch.zeros(2, 4, 64, 64), 2)
    b = frontend.FractalTensor.from_dense(torch.zeros(2, 4, 1, 64), 2)
    from programs import user_programs
    batch_major, time_major, wrong_gates = user_programs(ops)
    assert batch_major(embs, w, w, b) == "B"
    assert time_major(embs, w, w, b) == "T"
    assert calls == ["batch", "time"]
    with pytest.raises(NotImplementedError, match="fused kernel"):
        wrong_gates(embs, w, w, b)
    assert calls == ["batch", "time"]
    three_gates = frontend.FractalTensor.from_dense(torch.zeros(2, 3, 64, 64), 2)
    with pytest.raises(NotImplementedError):
        batch_major(embs, three_gates, three_gates, b)


def test_attention_program_is_recognised_with_its_scale(monkeypatch):
    from fractaltensor_b200 import operations as ops
    from programs import attention_program
    seen = []
    monkeypatch.setattr(frontend, "flash_attention", lambda q, k, v, scale=1.0: seen.append(scale) or "A")
    t = frontend.FractalTensor.from_dense(torch.zeros(1, 2, 2, 64, 128), 3)
    assert attention_program(ops, 64, 128)(t, t, t) == "A"
    assert attention_program(ops, 64, 128, scale=0.125)(t, t, t) == "A"
    assert seen == [1.0, 0.125]
    shallow = frontend.FractalTensor.from_dense(torch.zeros(2, 2, 64, 128), 2)
    with pytest.raises(NotImplementedError):
        attention_program(ops, 64, 128)(shallow, shallow, shallow)


def test_dilated_program_is_recognised(monkeypatch):
    from fractaltensor_b200 import operations as ops
    from programs import dilated_program
    got = []
    monkeypatch.setattr(frontend, "dilated_lstm", lambda embs, W, U, b: got.append((W, U, b)) or "D")
    embs = frontend.FractalTensor.from_dense(torch.zeros(2, 8, 1, 64), 2)
    w = frontend.FractalTensor.from_dense(torch.zeros(3, 4, 64, 64), 2)
    u = frontend.FractalTensor.from_dense(torch.zeros(3, 4, 64, 64), 2)
    b = frontend.FractalTensor.from_dense(torch.zeros(3, 4, 1, 64), 2)
    assert dilated_program(ops)(embs, w, u, b) == "D"
    assert got[0][0] is w and got[0][1] is u and got[0][2] is b
    # a plain map over real data with some other body is not a known program
    with pytest.raises(NotImplementedError):
        ops.map(lambda xs: ops.map(lambda x: ops.tanh(x), xs), embs)


def test_grid_program_is_recognised(monkeypatch):
    from fractaltensor_b200 import operations as ops
    from programs import grid_program
    got = []
    monkeypatch.setattr(frontend, "stacked_grid_rnns", lambda s, t, p: got.append((s, t, p)) or "G")
    src = frontend.FractalTensor.from_dense(torch.zeros(2, 5, 1, 64), 2)
    trg = frontend.FractalTensor.from_dense(torch.zeros(2, 4, 1, 64), 2)
    cell = lambda: (torch.zeros(128, 64), torch.zeros(64, 64), torch.zeros(1, 64))
    params = [(cell(), cell()) for _ in range(3)]
    model, wrong_state = grid_program(ops, 64)
    assert model(src, trg, params) == "G"
    assert got[0][0] is src and got[0][1] is trg and got[0][2] is params
    with pytest.raises(NotImplementedError):
        wrong_state(src, trg, params)
    # initial column state sized by the number of rows instead of the row length: another program
    def wrong_len(src_encs, trg_encs, stacked_params):
        def layer(state, p):
            z = ops.repeat(ops.zeros(shape=(1, 64)), len(state))
            ys1, ys2 = ops.scan(lambda s, x: s, state, initializer=(z, z))
            return ops.zip(ys1, ys2)
        return ops.map(lambda x: ops.fold(layer, stacked_params, initializer=ops.zip(*ops.product(*x))),
                       ops.zip(src_encs, trg_encs))
    with pytest.raises(NotImplementedError):
        wrong_len(src, trg, params)


def test_element_type_singletons():
    from fractaltensor_b200 import types as T
    assert T.internal_type_to_torch_type(T.float32) is torch.float32
    assert T.internal_type_to_torch_type(T.float16) is torch.float16
    assert T.internal_type_to_torch_type(T.bfloat16) is torch.bfloat16
    for name, want in (("float", T.float32), ("half", T.float16), ("bfloat16", T.bfloat16), ("int", T.int32)):
        assert T.str_to_internal_type(name) is want
    for t in (torch.float16, torch.bfloat16, torch.float32, torch.int32, torch.int64):
        assert T.internal_type_to_torch_type(T.torch_type_to_internal_type(t)) is t
    assert not T.float16.is_equal_type(T.bfloat16) and T.float16.is_equal_type(T.Real(16))
    assert T.float16.byte == 16 and T.bfloat16.max > T.float16.max
    assert T.pytype_to_internal_type(1) is T.int64 and T.pytype_to_internal_type(1.0) is T.float32
    with pytest.raises(NotImplementedError):
        T.str_to_internal_type("complex")
    with pytest.raises(ValueError):
        T.Real(32, brain=True)


def test_fractal_tensor_element_type():
    from fractaltensor_b200 import types as T
    ft = frontend.FractalTensor.from_dense(torch.zeros(2, 3, 1, 8), 2)
    assert ft.element_type is T.float32
    half = ft.astype(T.bfloat16)
    assert half.element_type is T.bfloat16 and half.indices == ft.indices and half.element_shape == (1, 8)
    assert ft.astype(torch.float16).element_type is T.float16


REFERENCE_ROOT = os.environ.get("FTB_REFERENCE_ROOT", "/root/reference")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE_ROOT, "kaleido")),
                    reason="the reference tree is not mounted on this machine")
def test_reference_fractaltensor_objects_are_accepted_as_they_are():
    """The reference's own kaleido.FractalTensor objects (built with the loader of
    tests/golden/generate.py, which imports the reference frontend from its tree) go straight into
    the model-level entry points: their flat buffer and nesting are read into the dense view the
    kernels take, and the call then stops at the device check because the data lives on the CPU."""
    sys_path = list(__import__("sys").path)
    try:
        from golden import generate
        kaleido, _ = generate.load_reference_frontend(REFERENCE_ROOT)
        from kaleido import FractalTensor, FractalTensorStorage, TensorStorage
    finally:
        __import__("sys").path[:] = sys_path

    def ft(data, shape, indices):
        depth = 1 if not isinstance(indices[0], list) else 2
        st = TensorStorage(list(shape), kaleido.float32, device="cpu")
        x = FractalTensor(FractalTensorStorage(st) if depth == 2 else st)
        x.indices = indices
        x.data = data.clone()
        return x

    D, L, N, H = 2, 5, 3, 64
    g = torch.Generator().manual_seed(1)
    x = torch.randn(N, L, 1, H, generator=g)
    W = torch.randn(D, 4, H, H, generator=g)
    b = torch.randn(D, 4, 1, H, generator=g)
    embs = ft(x.reshape(N * L, 1, H), (1, H), [list(range(L)) for _ in range(N)])
    Wss = ft(W.reshape(D * 4, H, H), (H, H), [list(range(4)) for _ in range(D)])
    bss = ft(b.reshape(D * 4, 1, H), (1, H), [list(range(4)) for _ in range(D)])
    assert type(embs).__module__.startswith("kaleido.")
    # the dense views the entry points compute from the reference objects
    assert torch.equal(frontend._dense(embs), x)
    assert torch.equal(frontend._dense(Wss), W)
    assert torch.equal(frontend._dense(bss), b)
    assert not frontend._is_ragged(embs)
    for fn in (frontend.stacked_lstm, frontend.stacked_lstm_time_major, frontend.dilated_lstm):
        with pytest.raises(RuntimeError, match="no CPU path"):
            fn(embs, Wss, Wss, bss)
    # a ragged reference object is routed to the variable-length entry, not densified
    ragged = ft(x.reshape(N * L, 1, H)[:12], (1, H), [list(range(5)), list(range(4)), list(range(3))])
    assert frontend._is_ragged(ragged)
    with pytest.raises(RuntimeError, match="no CPU path"):
        frontend.stacked_lstm(ragged, Wss, Wss, bss)
