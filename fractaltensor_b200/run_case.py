"""Runs one operator of the hot path once (or a few times) on seeded synthetic inputs.

    python -m fractaltensor_b200.run_case lstm --D 16 --L 20 --N 256 --H 1024 --dtype bf16 --iters 2
    python -m fractaltensor_b200.run_case lstm --D 16 --L 20 --N 32 --H 1024      # a batch shard: the small-batch kernel
    python -m fractaltensor_b200.run_case dilated --D 6 --L 128 --N 256 --H 256 --dtype fp16
    python -m fractaltensor_b200.run_case grid --D 1 --A 32 --N 64 --H 256 --dtype fp16
    python -m fractaltensor_b200.run_case varlen --D 16 --L 100 --N 256 --H 1024 --min-len 20
    python -m fractaltensor_b200.run_case b2b --batch 16 --M 16384
    python -m fractaltensor_b200.run_case attn --B 4 --heads 16 --S 2048
    python -m fractaltensor_b200.run_case sparse_attn --B 2 --heads 16 --S 4096 --dtype fp32

A small, fixed workload to put under a profiler or to time by hand; prints the
average time per call measured with CUDA events.
"""
import argparse
import math

import torch

from . import ops

DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["lstm", "varlen", "dilated", "grid", "b2b", "attn", "softmax", "sparse_attn"])
    ap.add_argument("--D", type=int, default=16)
    ap.add_argument("--L", type=int, default=20)
    ap.add_argument("--N", type=int, default=256)
    ap.add_argument("--H", type=int, default=1024)
    ap.add_argument("--A", type=int, default=32)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--B", type=int, default=16)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--S", type=int, default=2048)
    ap.add_argument("--dtype", default="bf16", choices=sorted(DT))
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--layers-per-group", type=int, default=0)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--schedule", type=int, default=0)
    ap.add_argument("--pair", type=int, default=0)
    ap.add_argument("--resident", type=int, default=0, help="lstm, small-batch kernel: recurrent weight blocks kept in TMEM")
    ap.add_argument("--min-len", type=int, default=1, help="varlen: lengths are uniform in [min-len, L]")
    ap.add_argument("--causal", action="store_true", help="attn: keys 0..i for query i")
    ap.add_argument("--window", type=int, default=None, help="attn with --causal: keys i-window+1..i")
    ap.add_argument("--local", type=int, nargs=2, default=None, help="attn: keys i-LEFT..i+RIGHT")
    ap.add_argument("--head-dim", type=int, default=64, help="sparse_attn: elements per head")
    ap.add_argument("--as-shipped", action="store_true", help="sparse_attn: the softmax dimension of the shipped example")
    ap.add_argument("--graph", action="store_true",
                    help="capture one call in a CUDA graph and time replays (schedules with one launch per level)")
    a = ap.parse_args()
    dt, dev = DT[a.dtype], torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    uni = lambda bound, *s: (torch.rand(*s, device=dev, generator=g) * 2 - 1) * bound

    if a.case == "lstm":
        x = rnd(a.L, a.N, a.H).to(dt)
        Wp, _ = ops.lstm_pack_weights(uni(1 / 32, a.D, 4, a.H, a.H).to(dt), uni(1 / 32, a.D, 4, a.H, a.H).to(dt))
        hs = torch.empty(a.D, a.L, a.N, a.H, dtype=dt, device=dev)
        c = torch.empty(a.D, a.N, a.H, device=dev)
        fn = lambda: ops.lstm_stacked(x, Wp, None, hs, c, layers_per_group=a.layers_per_group, bn=a.bn,
                                      schedule=a.schedule, pair=a.pair, resident=a.resident)
    elif a.case == "varlen":
        lens = torch.randint(a.min_len, a.L + 1, (a.N,), generator=torch.Generator().manual_seed(0))
        lens[0] = a.L
        active = [int((lens > t).sum()) for t in range(a.L)]
        T = sum(active)
        x = rnd(T, a.H).to(dt)
        Wp, _ = ops.lstm_pack_weights(uni(1 / 32, a.D, 4, a.H, a.H).to(dt), uni(1 / 32, a.D, 4, a.H, a.H).to(dt))
        hs = torch.empty(a.D, T, a.H, dtype=dt, device=dev)
        c = torch.empty(a.D, a.N, a.H, device=dev)
        print("varlen: %d of %d rows active (%.1f%%)" % (T, a.L * a.N, 100.0 * T / (a.L * a.N)))
        fn = lambda: ops.lstm_stacked_varlen(x, active, Wp, None, hs, c, layers_per_group=a.layers_per_group,
                                             bn=a.bn, schedule=a.schedule, pair=a.pair)
    elif a.case == "dilated":
        x = rnd(a.L, a.N, a.H).to(dt)
        Wp, _ = ops.lstm_pack_weights(uni(1 / 16, a.D, 4, a.H, a.H).to(dt), uni(1 / 16, a.D, 4, a.H, a.H).to(dt))
        dil = [2 ** l for l in range(a.D)]
        fn = lambda: ops.lstm_dilated(x, Wp, dil, bn=a.bn, schedule=a.schedule)
    elif a.case == "grid":
        X, Y = rnd(a.A, a.A, a.N, a.H).to(dt), rnd(a.A, a.A, a.N, a.H).to(dt)
        Wpx = ops.grid_pack_weights(uni(1 / 16, a.D, 2 * a.H, a.H).to(dt), uni(1 / 16, a.D, a.H, a.H).to(dt))
        Wpy = ops.grid_pack_weights(uni(1 / 16, a.D, 2 * a.H, a.H).to(dt), uni(1 / 16, a.D, a.H, a.H).to(dt))
        fn = lambda: ops.grid_rnn(X, Y, Wpx, Wpy, schedule=a.schedule)
    elif a.case == "b2b":
        s = 1 / math.sqrt(128)
        A_, B_, C_ = (rnd(a.batch, a.M, 128) * s).to(dt), (rnd(a.batch, 128, 128) * s).to(dt), (rnd(a.batch, 128, 128) * s).to(dt)
        # three buffer sets used in turn (each 135 MB > L2), so no call finds its operands cached
        sets = [(A_.clone(), B_.clone(), C_.clone(), torch.empty_like(A_)) for _ in range(3)]
        turn = [0]

        def fn():
            turn[0] = (turn[0] + 1) % 3
            return ops.b2b_gemm(*sets[turn[0]])
    elif a.case == "softmax":
        # rows x width fp32; three input/output pairs in turn when a pair is smaller than 2 x L2
        xs = [rnd(a.M, a.H) for _ in range(3)]
        ys = [torch.empty_like(xs[0]) for _ in range(3)]
        turn = [0]

        def fn():
            turn[0] = (turn[0] + 1) % 3
            return ops.online_softmax(xs[turn[0]], ys[turn[0]])
    elif a.case == "sparse_attn":
        # window 5, dilation 2, 3 random keys, 3 + 3 global tokens as in the example; three q/k/v/o sets in turn
        sets = [[rnd(a.B, a.heads, a.S, a.head_dim).to(dt) for _ in range(3)] for _ in range(3)]
        outs = [torch.empty_like(s_[0]) for s_ in sets]
        pos = torch.randint(0, a.S, (a.B, a.heads, a.S - 6, 3), device=dev, generator=g, dtype=torch.int32)
        turn = [0]

        def fn():
            turn[0] = (turn[0] + 1) % 3
            q, k, v = sets[turn[0]]
            return ops.sparse_attention(q, k, v, pos, 5, 2, 3, scale=1 / math.sqrt(a.head_dim),
                                        as_shipped=a.as_shipped, out=outs[turn[0]])
    else:
        q, k, v = (rnd(a.B, a.heads, a.S, 128).to(dt) for _ in range(3))
        out = torch.empty_like(q)
        fn = lambda: ops.flash_attention(q, k, v, scale=1 / math.sqrt(128), out=out, causal=a.causal, window=a.window, local=a.local)

    for _ in range(a.warmup):
        fn()
    torch.cuda.synchronize()
    if a.graph:
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()  # warm the side stream (workspace, lazy initialisation) before capturing
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(graph):
            fn()
        fn = graph.replay
        fn()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ops.check_status()
    ms = e0.elapsed_time(e1) / a.iters
    print("%s: %.3f ms per call (%.1f us)" % (a.case, ms, ms * 1e3))


if __name__ == "__main__":
    main()
