"""Headline benchmark: stacked LSTM forward, benchmark config 4 (depth 16, hidden 1024,
batch 256, 100 steps, bf16 with fp32 cell state), metric samples*steps/s.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # CPU arm: the oracle port on host cores

One "step" is one full forward pass of the wavefront over the batch of synthetic input.
With N GPUs the batch of 256 is split into contiguous shards of 256/N sequences (strong
scaling: the total work is fixed), weights are replicated, nothing is exchanged inside the
recurrence, and one all-gather of the top layer's output shards per step is inside the timed
region.  A second measurement with 256 sequences on every GPU (weak scaling) is reported under
its own key.  Prints one JSON line on rank 0.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(D=16, L=100, N=256, I=1024, H=1024, seed=3, w_bound=1.0 / 32)
METRIC = "lstm_samples_steps_per_s_h1024_d16"
UNIT = "samples*steps/s"
FLOPS_PER_SAMPLE_STEP = CFG["D"] * 2 * 4 * CFG["H"] * (CFG["I"] + CFG["H"])  # all layers
# DRAM bytes (read + write) of one launch of the dominant kernel at the 1-GPU workload, from a
# one-pass ncu capture of this command (717.7 MB read + 833.2 MB written; compulsory: 268 MB
# weights + 52 MB x read, 839 MB hidden states written).
TRAFFIC_BYTES_PER_LAUNCH = 1550.9e6


def workload_config(world):
    """The same dictionary for both arms, so that their lines describe one configuration."""
    return {"workload": "stacked LSTM D16 H1024 I1024 N256 L100, bf16 weights/activations, fp32 cell state "
                        "(benchmark config 4)",
            "global_batch": CFG["N"], "seq_len": CFG["L"],
            "parallelism": "batch of 256 split into %d contiguous shard(s), weights replicated, one all-gather of "
                           "the top layer's output per step" % world,
            "cache": "per-step inputs exceed L2 (268 MB weights + hidden states vs 126 MB L2); no flush needed"}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(burst=d["bf16_tflops"], sustained=d["bf16_tflops_sustained"], hbm=d["hbm_gbs"], src="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, src="fallback")


# ------------------------------------------------------------------ seeded synthetic inputs
def lstm_inputs(D, L, N, I, H, seed, w_bound, dtype):
    """x ~ N(0,1) [L,N,I]; W [D,4,I,H], U [D,4,H,H] ~ U(-w_bound, w_bound)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(L, N, I, generator=g)
    W = (torch.rand(D, 4, I, H, generator=g) * 2 - 1) * w_bound
    U = (torch.rand(D, 4, H, H, generator=g) * 2 - 1) * w_bound
    return x.to(dtype), W.to(dtype), U.to(dtype)


class ClockSampler(object):
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index, period_ms=20):
        self.index = index
        self.period_ms = period_ms
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def window(self, t_begin, t_end):
        """Summary of the samples taken inside [t_begin, t_end] (host clock), all samples if that
        window caught none."""
        rows = [r for ts, r in self.rows if t_begin <= ts <= t_end + 0.05]
        if not rows:
            rows = [r for _, r in self.rows]
        num = lambda s: s.replace(".", "").isdigit()
        sm = sorted(float(r[0]) for r in rows if len(r) >= 7 and num(r[0]))
        mx = [float(r[1]) for r in rows if len(r) >= 7 and num(r[1])]
        pw = [float(r[2]) for r in rows if len(r) >= 7 and num(r[2])]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 7 and r[3 + i] == "Active" for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "power_w_max": max(pw) if pw else None, "reasons": reasons,
                "samples": len(sm)}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            self.t.join(timeout=2)


# ----------------------------------------------------------------------- CPU legs (oracle port)
def cpu_lstm_rate(sample_steps, threads, passes=1):
    """Oracle port (dense fp32 restatement of the reference program) on the host cores: full depth
    and batch of config 4, `sample_steps` timesteps, `passes` times.  Returns samples*steps/s and the
    seconds of one pass."""
    from oracle import dense
    torch.set_num_threads(threads)
    x, W, U = lstm_inputs(CFG["D"], sample_steps, CFG["N"], CFG["I"], CFG["H"], CFG["seed"], CFG["w_bound"],
                          torch.bfloat16)
    x, W, U = x.float(), W.float(), U.float()
    t0 = time.perf_counter()
    for _ in range(passes):
        dense.stacked_lstm_dense(x, W, U)
    dt = (time.perf_counter() - t0) / passes
    return CFG["N"] * sample_steps / dt, dt


def cpu_other_configs(threads):
    """The oracle port timed on bounded samples of the other benchmark configurations, in the unit
    the GPU entry of the same configuration is quoted in."""
    from oracle import dense
    torch.set_num_threads(threads)
    out = {}
    g = torch.Generator().manual_seed(7)
    # config 1 at full size
    x, W, U = lstm_inputs(4, 64, 32, 256, 256, 0, 1.0 / 16, torch.float32)
    dense.stacked_lstm_dense(x[:4], W, U)
    t0 = time.perf_counter()
    for _ in range(5):
        dense.stacked_lstm_dense(x, W, U)
    dt = (time.perf_counter() - t0) / 5
    out["1"] = {"value": 32 * 64 / dt, "unit": UNIT, "cores": threads, "kind": "port",
                "sample": "the whole configuration, mean of 5 passes (%.2f s each)" % dt}
    # config 2: the whole configuration, three times (after one untimed pass)
    s = 1 / math.sqrt(128)
    A = (torch.randn(16, 16384, 128, generator=g) * s).half()
    B = (torch.randn(16, 128, 128, generator=g) * s).half()
    C = (torch.randn(16, 128, 128, generator=g) * s).half()
    dense.b2b_gemm_dense(A[:2], B[:2], C[:2])
    t0 = time.perf_counter()
    for _ in range(3):
        dense.b2b_gemm_dense(A, B, C)
    dt = (time.perf_counter() - t0) / 3
    out["2"] = {"value": 16 * 4 * 16384 * 128 * 128 / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                "sample": "all 16 batch entries, fp32 arithmetic on fp16 data, mean of 3 passes (%.2f s each)" % dt}
    # config 3: 32 of the 256 (batch, head) pairs
    q, k, v = (torch.randn(2, 16, 2048, 128, generator=g) for _ in range(3))
    dense.flash_attention_dense(q[:1, :2], k[:1, :2], v[:1, :2], scale=1 / math.sqrt(128), block=128)
    t0 = time.perf_counter()
    dense.flash_attention_dense(q, k, v, scale=1 / math.sqrt(128), block=128)
    dt = time.perf_counter() - t0
    out["3"] = {"value": 32 * 4 * 2048 * 2048 * 128 / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                "sample": "32 of 256 (batch, head) pairs, fp32 (%.2f s)" % dt}
    # config 5a: all 256 samples, all 6 layers, 256 of 512 steps
    x, W, U = lstm_inputs(6, 256, 256, 256, 256, 4, 1.0 / 16, torch.float32)
    t0 = time.perf_counter()
    dense.dilated_lstm_dense(x, W, U, [1, 2, 4, 8, 16, 32])
    dt = time.perf_counter() - t0
    out["5a"] = {"value": 256 * 256 / dt, "unit": UNIT, "cores": threads, "kind": "port",
                 "sample": "full batch and depth, 256 of 512 steps, fp32 (%.2f s)" % dt}
    # config 5b: the whole configuration
    X, Y, p = dense.make_grid_inputs(1, 32, 32, 64, 256, 4, 1.0 / 16)
    t0 = time.perf_counter()
    dense.grid_rnn_dense(X, Y, p["i2h_x"], p["h2h_x"], None, p["i2h_y"], p["h2h_y"], None)
    dt = time.perf_counter() - t0
    out["5b"] = {"value": 32 * 32 * 64 / dt, "unit": "cells*samples/s", "cores": threads, "kind": "port",
                 "sample": "the whole configuration, fp32 (%.2f s)" % dt}
    # sparse attention: 2 of the 32 (batch, head) pairs at sequence 4096
    q, k, v = (torch.rand(1, 2, 4096, 64, generator=g) for _ in range(3))
    pos = torch.randint(0, 4096, (1, 2, 4090, 3), generator=g, dtype=torch.int32)
    t0 = time.perf_counter()
    dense.sparse_attention_dense(q * 0.125, k, v, pos, 5, 2, 3)
    dt = time.perf_counter() - t0
    out["sparse"] = {"value": 2 * 4096 / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
                     "sample": "2 of 32 (batch, head) pairs, fp32 (%.2f s)" % dt}
    # attention RNN: 8 of the 64 sequences
    Hr = 512
    wr = [(torch.rand(Hr, Hr, generator=g) * 2 - 1) / math.sqrt(Hr) for _ in range(4)]
    zb = torch.zeros(1, Hr)
    t0 = time.perf_counter()
    dense.rnn_attention_dense(torch.randn(8 * 50, Hr, generator=g), torch.randn(8 * 50, Hr, generator=g), [50] * 8,
                              [50] * 8, wr[0], wr[1], zb, wr[2], wr[3], zb, torch.rand(Hr, 1, generator=g),
                              torch.rand(Hr, 1, generator=g))
    dt = time.perf_counter() - t0
    out["rnn_attention"] = {"value": 8 * 100 / dt, "unit": UNIT, "cores": threads, "kind": "port",
                            "sample": "8 of 64 sequences, 50 + 50 steps, fp32 (%.2f s)" % dt}
    return out


def run_reference(args, rank, world):
    """CPU arm: the reference has no GPU implementation that runs here, and its eager Python
    frontend does not travel; its semantics are timed through the oracle port."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample = 10
    rates = []
    for i in range(args.warmup + args.steps):
        r, dt = cpu_lstm_rate(sample, threads)
        if i >= args.warmup:
            rates.append((r, dt))
    value = sum(r for r, _ in rates) / len(rates)
    ms = 1e3 * sum(dt for _, dt in rates) / len(rates)
    sample_desc = ("full depth 16 and batch 256 of config 4, %d of 100 timesteps per step, fp32 on bf16-rounded "
                   "inputs" % sample)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": workload_config(world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample_desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------ the other configurations
def other_configs(ops, dev, pk, cpu):
    """The path's other benchmark configurations, each timed alone on resident data with CUDA events
    after 3 warm-up calls (rank 0, single-GPU runs only), each against the roofline that bounds it:
    algorithmic bytes over the measured copy bandwidth, or algorithmic FLOPs over the measured bf16
    GEMM peak (the latency-bound wavefronts too: their fraction says how far from the tensor
    roofline the dependent chain leaves them)."""

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ops.check_status()
        return e0.elapsed_time(e1) / iters

    def tensor_entry(name, ms, flops, **extra):
        ach = flops / (ms * 1e-3) / 1e12
        e = {"config": name, "ms": ms, "bound": "tensor", "achieved": ach, "peak": pk["burst"], "unit": "TFLOP/s",
             "frac": ach / pk["burst"], "frac_sustained": ach / pk["sustained"]}
        e.update(extra)
        return e

    def hbm_entry(name, ms, nbytes, **extra):
        ach = nbytes / (ms * 1e-3) / 1e9
        e = {"config": name, "ms": ms, "bound": "hbm", "achieved": ach, "peak": pk["hbm"], "unit": "GB/s",
             "frac": ach / pk["hbm"]}
        e.update(extra)
        return e

    out = []
    g = torch.Generator(device=dev).manual_seed(1)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    uni = lambda b, *s: (torch.rand(*s, device=dev, generator=g) * 2 - 1) * b
    turn = [0]

    # config 2: 16 x [16384,128].[128,128].[128,128], fp16; three buffer sets in turn (each > L2)
    s = 1 / math.sqrt(128)
    sets = [((rnd(16, 16384, 128) * s).half(), (rnd(16, 128, 128) * s).half(), (rnd(16, 128, 128) * s).half(),
             torch.empty(16, 16384, 128, device=dev, dtype=torch.half)) for _ in range(3)]

    def b2b():
        turn[0] = (turn[0] + 1) % 3
        ops.b2b_gemm(*sets[turn[0]])

    ms = timed(b2b, 60)
    nbytes = 16 * (2 * 16384 * 128 + 2 * 128 * 128) * 2
    out.append(hbm_entry("2: fused two GEMMs 16x(16384x128x128x128) fp16", ms, nbytes,
                         tflops=16 * 4 * 16384 * 128 * 128 / (ms * 1e-3) / 1e12,
                         cache="three rotating buffer sets of 135 MB", cpu_baseline=cpu.get("2")))
    del sets

    # config 3: attention B16 h16 S2048 d128 fp16 (q, k, v, o: 537 MB > L2)
    q, k, v = (rnd(16, 16, 2048, 128).half() for _ in range(3))
    o = torch.empty_like(q)
    ms = timed(lambda: ops.flash_attention(q, k, v, scale=1 / math.sqrt(128), out=o), 20)
    out.append(tensor_entry("3: flash attention B16 h16 S2048 d128 fp16", ms, 4 * 16 * 16 * 2048 * 2048 * 128,
                            cpu_baseline=cpu.get("3")))
    ms = timed(lambda: ops.flash_attention(q, k, v, scale=1 / math.sqrt(128), out=o, causal=True), 20)
    out.append(tensor_entry("3 with a causal mask (not a reference configuration; visible pairs only)", ms,
                            2 * 16 * 16 * 2048 * 2049 * 128))
    del q, k, v, o

    # config 5a: dilated LSTM, 6 layers, dilation 2^l, H256 N256 L512 fp16
    x = rnd(512, 256, 256).half()
    Wp, _ = ops.lstm_pack_weights(uni(1 / 16, 6, 4, 256, 256).half(), uni(1 / 16, 6, 4, 256, 256).half())
    dil = [2 ** l for l in range(6)]
    ms = timed(lambda: ops.lstm_dilated(x, Wp, dil), 5)
    out.append(tensor_entry("5a: dilated LSTM 6 layers H256 N256 L512 fp16", ms, 6 * 512 * 256 * 2 * 1024 * 512,
                            samples_steps_per_s=256 * 512 / (ms * 1e-3),
                            note="latency-bound: about 520 dependent levels", cpu_baseline=cpu.get("5a")))

    # config 5b: grid RNN 32x32, H256, N64, fp16
    X, Y = rnd(32, 32, 64, 256).half(), rnd(32, 32, 64, 256).half()
    Wpx = ops.grid_pack_weights(uni(1 / 16, 1, 512, 256).half(), uni(1 / 16, 1, 256, 256).half())
    Wpy = ops.grid_pack_weights(uni(1 / 16, 1, 512, 256).half(), uni(1 / 16, 1, 256, 256).half())
    ms = timed(lambda: ops.grid_rnn(X, Y, Wpx, Wpy), 10)
    out.append(tensor_entry("5b: grid RNN 32x32 H256 N64 fp16", ms, 32 * 32 * 2 * 64 * 2 * 768 * 256,
                            cells_samples_per_s=32 * 32 * 64 / (ms * 1e-3),
                            note="latency-bound: 63 dependent anti-diagonals", cpu_baseline=cpu.get("5b")))

    # stand-alone online softmax, fp32 16384 x 4096 (three input/output pairs in turn, 1.6 GB > L2)
    xs = [rnd(16384, 4096) for _ in range(3)]
    ys = [torch.empty_like(xs[0]) for _ in range(3)]

    def softmax():
        turn[0] = (turn[0] + 1) % 3
        ops.online_softmax(xs[turn[0]], ys[turn[0]])

    ms = timed(softmax, 30)
    out.append(hbm_entry("online softmax fp32 16384x4096", ms, 2 * 16384 * 4096 * 4,
                         cache="three rotating buffer pairs of 537 MB"))
    del xs, ys

    # embedding lookup in front of config 4: 25 600 words, table 50 000 x 1024 bf16
    table = rnd(50000, 1024).bfloat16()
    ids = torch.randint(0, 50000, (25600,), device=dev, generator=g)
    rows_out = torch.empty(25600, 1024, device=dev, dtype=torch.bfloat16)
    ms = timed(lambda: ops.embedding_gather(table, ids, rows_out), 30)
    out.append(hbm_entry("embedding lookup 25600 words, table 50000x1024 bf16", ms, 25600 * (2 * 1024 * 2 + 8),
                         cache="105 MB per call: fits L2, so this is a launch- and latency-bound size"))
    del table, ids, rows_out

    # token-level sparse attention at the size the example names for real use: batch 2, 16 heads of 64,
    # sequence 4096, window 5 dilation 2, 3 random keys, 3 + 3 global tokens, fp32 (three rotating sets)
    sa = [[rnd(2, 16, 4096, 64) for _ in range(3)] + [torch.empty(2, 16, 4096, 64, device=dev)] for _ in range(3)]
    pos = torch.randint(0, 4096, (2, 16, 4090, 3), device=dev, generator=g, dtype=torch.int32)

    def sparse():
        turn[0] = (turn[0] + 1) % 3
        q_, k_, v_, o_ = sa[turn[0]]
        ops.sparse_attention(q_, k_, v_, pos, 5, 2, 3, scale=0.125, out=o_)

    ms = timed(sparse, 30)
    out.append(hbm_entry("sparse attention fp32 B2 h16 S4096 d64, window 5 dilation 2, 3 random, 6 global", ms,
                         4 * 2 * 16 * 4096 * 64 * 4 + 2 * 16 * 4090 * 3 * 4,
                         cache="three rotating q/k/v/o sets of 134 MB", tokens_per_s=2 * 16 * 4096 / (ms * 1e-3),
                         cpu_baseline=cpu.get("sparse")))
    del sa, pos

    # attention RNN at the example's hidden size (512), batch 64, 50 source and 50 target positions, bf16
    Hr, Nr, Lr = 512, 64, 50
    rp = [uni(1 / math.sqrt(Hr), Hr, Hr).bfloat16() for _ in range(4)]
    Wps, Wpt = ops.rnn_pack_weights(rp[0], rp[1]), ops.rnn_pack_weights(rp[2], rp[3])
    xs_, ys_ = rnd(Lr, Nr, Hr).bfloat16(), rnd(Lr, Nr, Hr).bfloat16()
    ep, dp = torch.rand(Hr, device=dev, generator=g).bfloat16(), torch.rand(Hr, device=dev, generator=g).bfloat16()
    ms = timed(lambda: ops.rnn_attention(xs_, ys_, Wps, Wpt, None, None, ep, dp), 10)
    out.append(tensor_entry("attention RNN bf16 H512 N64, 50 source + 50 target steps", ms,
                            2 * Lr * Nr * 2 * (2 * Hr) * Hr, samples_steps_per_s=Nr * 2 * Lr / (ms * 1e-3),
                            note="one launch per source step, two per target step: 151 dependent launches; "
                                 "latency-bound, the tensor roofline is quoted for context",
                            cpu_baseline=cpu.get("rnn_attention")))
    del rp, Wps, Wpt, xs_, ys_

    # config 1: stacked LSTM fp32 D4 H256 N32 L64 (CUDA cores; the reference's own CPU-runnable case)
    x1, W1, U1 = lstm_inputs(4, 64, 32, 256, 256, 0, 1.0 / 16, torch.float32)
    Wp1, _ = ops.lstm_pack_weights(W1.to(dev), U1.to(dev))
    x1 = x1.to(dev)
    ms = timed(lambda: ops.lstm_stacked(x1, Wp1), 10)
    out.append(tensor_entry("1: stacked LSTM fp32 D4 H256 N32 L64", ms, 4 * 64 * 32 * 2 * 1024 * 512,
                            samples_steps_per_s=32 * 64 / (ms * 1e-3),
                            note="fp32 on CUDA cores (the 1e-5 bound rules out tf32 tensor cores); one persistent launch, "
                                 "weights resident in shared memory; 67 dependent levels; "
                                 "the tensor roofline is quoted for context",
                            cpu_baseline=cpu.get("1")))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ftb200", choices=["ftb200", "reference"])
    ap.add_argument("--layers-per-group", type=int, default=0)
    ap.add_argument("--schedule", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true")
    ap.add_argument("--no-weak", action="store_true")
    ap.add_argument("--sustain-seconds", type=float, default=1.5)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ftb200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    from fractaltensor_b200 import ops, sharding
    from fractaltensor_b200._lib import lib

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    D, L, N, I, H = CFG["D"], CFG["L"], CFG["N"], CFG["I"], CFG["H"]
    x_full, W, U = lstm_inputs(D, L, N, I, H, CFG["seed"], CFG["w_bound"], torch.bfloat16)
    Wp, _ = ops.lstm_pack_weights(W.to(dev), U.to(dev))
    del W, U
    lo, hi = sharding.shard_range(N, rank, world)
    if (hi - lo) * world != N:
        raise SystemExit("bench.py: the batch of %d does not split evenly over %d GPUs" % (N, world))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    class Leg(object):
        """One measurement set-up: `n_local` sequences on this GPU (a shard of the batch, or a full
        batch of its own for the weak-scaling line)."""

        def __init__(self, x_local):
            self.n = x_local.shape[1]
            self.x_pinned = x_local.contiguous().pin_memory()
            self.x_dev = self.x_pinned.to(dev)
            n_buf = 2
            self.hs = [torch.empty(D, L, self.n, H, dtype=torch.bfloat16, device=dev) for _ in range(n_buf)]
            self.c = torch.empty(D, self.n, H, dtype=torch.float32, device=dev)
            self.gathered = [torch.empty(world, L, self.n, H, dtype=torch.bfloat16, device=dev) for _ in range(2)] \
                if world > 1 else None
            self.s_comm = torch.cuda.Stream(device=dev) if world > 1 else None
            self.ev_done = [torch.cuda.Event() for _ in range(2)]
            self.ev_gathered = [torch.cuda.Event() for _ in range(2)]
            self.i = 0
            # end to end: three streams and two buffer sets
            self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
            self.x_buf = [torch.empty_like(self.x_dev) for _ in range(2)]
            self.out_buf = [torch.empty(L, self.n, H, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
            self.ev_in = [torch.cuda.Event() for _ in range(2)]
            self.ev_run = [torch.cuda.Event() for _ in range(2)]
            self.ev_out = [torch.cuda.Event() for _ in range(2)]
            self.j = 0

        def forward(self, x, hs):
            ops.lstm_stacked(x, Wp, None, hs, self.c, layers_per_group=args.layers_per_group, schedule=args.schedule)

        def gather(self, b, after):
            """All-gather of the top layer's shard of buffer set b on the communication stream."""
            with torch.cuda.stream(self.s_comm):
                self.s_comm.wait_event(after)
                dist.all_gather_into_tensor(self.gathered[b], self.hs[b][D - 1])
                self.ev_gathered[b].record(self.s_comm)

        # Resident steps.  Multi-GPU: the all-gather of step i runs on its own stream while step i+1
        # computes into the other hidden-state buffer; a step is complete when its gather is.
        def step_resident(self):
            if world == 1:
                self.forward(self.x_dev, self.hs[0])
                return
            b = self.i & 1
            cur = torch.cuda.current_stream()
            if self.i >= 2:
                cur.wait_event(self.ev_gathered[b])  # hs[b] was read by the gather of step i-2
            self.forward(self.x_dev, self.hs[b])
            self.ev_done[b].record(cur)
            self.gather(b, self.ev_done[b])
            self.i += 1

        def drain_resident(self):
            if world > 1:
                cur = torch.cuda.current_stream()
                for ev in self.ev_gathered:
                    cur.wait_event(ev)

        def timed_resident(self, steps):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                self.step_resident()
            self.drain_resident()
            e1.record()
            barrier()
            ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return ms.item()

        # End to end: every step copies its input shard from pinned host memory, runs the forward
        # through the public operator, all-gathers the top layer (multi-GPU) and copies the top
        # layer's shard back to pinned host memory; step i's copies overlap step i+-1's compute.
        def step_e2e(self):
            b = self.j & 1
            with torch.cuda.stream(self.s_in):
                if self.j >= 2:
                    self.s_in.wait_event(self.ev_run[b])   # x_buf[b] was read by step j-2
                self.x_buf[b].copy_(self.x_pinned, non_blocking=True)
                self.ev_in[b].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[b])
                if self.j >= 2:
                    self.s_run.wait_event(self.ev_out[b])  # hs[b] was copied out by step j-2
                    if world > 1:
                        self.s_run.wait_event(self.ev_gathered[b])
                self.forward(self.x_buf[b], self.hs[b])
                self.ev_run[b].record(self.s_run)
            if world > 1:
                self.gather(b, self.ev_run[b])
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[b])
                self.out_buf[b].copy_(self.hs[b][D - 1], non_blocking=True)
                self.ev_out[b].record(self.s_out)
            self.j += 1

        def timed_e2e(self, steps):
            barrier()
            self.j = 0
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            cur = torch.cuda.current_stream()
            e0.record(cur)
            for st in (self.s_in, self.s_run, self.s_out) + ((self.s_comm,) if world > 1 else ()):
                st.wait_event(e0)
            for _ in range(steps):
                self.step_e2e()
            for ev in self.ev_out + (self.ev_gathered if world > 1 else []):
                cur.wait_event(ev)
            e1.record(cur)
            barrier()
            ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return ms.item()

    leg = Leg(x_full[:, lo:hi])

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to start: launch it before the warm-up
    for _ in range(args.warmup):
        leg.step_resident()
    leg.drain_resident()
    ops.check_status()

    n0 = lib.ftb_launch_count()
    t_begin = time.perf_counter()
    total_ms = leg.timed_resident(args.steps)
    t_end = time.perf_counter()
    launches = lib.ftb_launch_count() - n0
    ops.check_status()

    leg.timed_e2e(2)
    e2e_ms = leg.timed_e2e(args.steps)
    ops.check_status()

    # A longer repeat of the same resident step: enough clock samples to see where the SM clock
    # settles under the power cap, and the step time that goes with it.
    sustain = None
    if args.sustain_seconds > 0:
        est = max(total_ms / args.steps, 1e-3)
        n_sus = max(args.steps, int(args.sustain_seconds * 1e3 / est))
        ts0 = time.perf_counter()
        sus_ms = leg.timed_resident(n_sus)
        ts1 = time.perf_counter()
        sustain = (n_sus, sus_ms, ts0, ts1)
    ops.check_status()

    # Weak scaling as a second line: every GPU runs a full batch of 256 of its own.
    weak = None
    if world > 1 and not args.no_weak:
        del leg.hs, leg.gathered
        torch.cuda.empty_cache()
        xw, _, _ = lstm_inputs(1, L, N, I, 1, CFG["seed"] + 1000 * rank, CFG["w_bound"], torch.bfloat16)
        wleg = Leg(xw)
        for _ in range(3):
            wleg.step_resident()
        wleg.drain_resident()
        w_ms = wleg.timed_resident(args.steps)
        ops.check_status()
        weak = {"scaling": "weak", "value": world * N * L / (w_ms / args.steps * 1e-3), "unit": UNIT,
                "ms_per_step": w_ms / args.steps, "global_batch": world * N,
                "note": "256 sequences on every GPU, all-gather of %d x 52 MB into every GPU per step" % world}
    torch.cuda.synchronize()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    sampler.stop()
    clocks = sampler.window(t_begin, t_end)
    ms_per_step = total_ms / args.steps
    value = N * L / (ms_per_step * 1e-3)
    e2e_value = N * L / (e2e_ms / args.steps * 1e-3)
    pk = peaks()
    n_local = hi - lo
    # Dominant kernel: one cooperative launch per step does the whole wavefront of this GPU's shard;
    # nothing else of ours launches in a step, so the launch's duration is the step's (at N > 1 the
    # all-gather overlaps the next step's launch).
    kernel = ("lstm_static_kernel<bf16> (persistent, CTA pairs, static tile ownership)" if n_local > 128 else
              "lstm_wmajor_kernel<bf16, %d> (persistent, weights on the M side, static tile ownership)"
              % (32 if n_local <= 32 else 64 if n_local <= 64 else 128))
    flops_per_launch = FLOPS_PER_SAMPLE_STEP * n_local * L
    achieved = flops_per_launch / (ms_per_step * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": achieved, "peak": pk["burst"], "unit": "TFLOP/s",
                "frac": achieved / pk["burst"], "frac_burst": achieved / pk["burst"],
                "traffic": TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None,
                "peak_source": "%s burst bf16 GEMM (the timed region lasts %.2f s)" % (pk["src"], total_ms * 1e-3),
                "kernel": kernel, "launches_per_step": launches / args.steps, "dominant_launches_per_step": 1,
                "avg_launch_us": 1e3 * ms_per_step, "flops_per_launch": flops_per_launch}
    if sustain is not None:
        n_sus, sus_ms, ts0, ts1 = sustain
        sus_step = sus_ms / n_sus
        sus_clk = sampler.window(ts0, ts1)
        sus_ach = flops_per_launch / (sus_step * 1e-3) / 1e12
        roofline.update({
            "frac_sustained": sus_ach / pk["sustained"], "sustained_achieved": sus_ach,
            "sustained_peak": pk["sustained"], "sustained_ms_per_step": sus_step, "sustained_steps": n_sus,
            "sustained_clocks": sus_clk,
            "ms_times_sm_mhz": {"timed": ms_per_step * clocks["sm_mhz"] if clocks["sm_mhz"] else None,
                                "sustained": sus_step * sus_clk["sm_mhz"] if sus_clk["sm_mhz"] else None}})
    cpu = None
    cpu_others = {}
    if world == 1 and not args.no_cpu_baseline:  # timed on rank 0 of single-GPU runs only
        threads = os.cpu_count() or 1
        sample, passes = 100, 3
        cpu_lstm_rate(10, threads)  # thread pool and allocator warm
        rate, dt = cpu_lstm_rate(sample, threads, passes)
        cpu = {"value": rate, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": "the whole of config 4 (depth 16, batch 256, %d timesteps), fp32 on bf16-rounded inputs, "
                         "mean of %d passes (%.1f s each)" % (sample, passes, dt)}
        if not args.no_other_configs:
            cpu_others = cpu_other_configs(threads)
    others = None
    if world == 1 and not args.no_other_configs:
        others = other_configs(ops, dev, pk, cpu_others)
    shard_bytes = leg.x_pinned.numel() * 2
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(world), "per_gpu_batch": n_local,
        "roofline": roofline, "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": shard_bytes, "d2h_bytes_per_step": shard_bytes,
                "note": "bytes per GPU; the all-gather of the top layer is inside the timed region" if world > 1 else
                        "input copied from and top layer copied back to pinned host memory every step"},
        "gpu_launches": int(launches), "clocks": clocks, "weak_scaling": weak, "other_configs": others,
    }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
