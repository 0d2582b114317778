"""Headline benchmark: stacked LSTM forward, benchmark config 4 (depth 16, hidden 1024,
batch 256 per GPU, 100 steps, bf16 with fp32 cell state), metric samples*steps/s.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # CPU arm: the oracle port on host cores

One "step" is one full forward pass of the wavefront over one batch of synthetic
input.  Batch sharding across GPUs is weak scaling (256 samples per GPU, weights
replicated, one all-gather of the top-layer output shards per step).  Prints one
JSON line on rank 0.
"""
import argparse
import json
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
# DRAM bytes (read + write) of one launch of the dominant kernel at this exact workload, from the
# one-pass ncu capture summarised in profiles/lstm_static_config4.md (775.7 MB read + 832.0 MB
# written; compulsory: 268 MB weights + 52 MB x read, 839 MB hidden states written).
TRAFFIC_BYTES_PER_LAUNCH = 1607.7e6


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(burst=d["bf16_tflops"], sustained=d["bf16_tflops_sustained"], hbm=d["hbm_gbs"], src="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, src="fallback")


class ClockSampler(object):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples taken inside [t_begin, t_end] (host clock), all samples if that
        window caught none."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.t.join(timeout=2)
        rows = [r for ts, r in self.rows if t_begin is None or t_begin <= ts <= t_end + 0.15]
        if not rows:
            rows = [r for _, r in self.rows]
        sm = sorted(float(r[0]) for r in rows if len(r) >= 7 and r[0].replace(".", "").isdigit())
        mx = [float(r[1]) for r in rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        pw = [float(r[2]) for r in rows if len(r) >= 7 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 7 and r[3 + i] == "Active" for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": reasons, "samples": len(sm)}


def cpu_port_rate(sample_steps, threads):
    """Oracle port (dense fp32 restatement of the reference program) on the host cores:
    full depth and batch of config 4, `sample_steps` timesteps.  Returns samples*steps/s."""
    from oracle import dense
    torch.set_num_threads(threads)
    x, W, U, _ = dense.make_lstm_inputs(CFG["D"], sample_steps, CFG["N"], CFG["I"], CFG["H"], CFG["seed"],
                                        CFG["w_bound"], dtype=torch.bfloat16)
    x, W, U = x.float(), W.float(), U.float()
    t0 = time.perf_counter()
    dense.stacked_lstm_dense(x, W, U)
    dt = time.perf_counter() - t0
    return CFG["N"] * sample_steps / dt, dt


def run_reference(args, rank):
    """CPU arm: the reference has no GPU implementation that runs here, and its eager Python
    frontend does not travel; its semantics are timed through the oracle port."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample = 10
    rates = []
    for i in range(args.warmup + args.steps):
        r, dt = cpu_port_rate(sample, threads)
        if i >= args.warmup:
            rates.append((r, dt))
    value = sum(r for r, _ in rates) / len(rates)
    ms = 1e3 * sum(dt for _, dt in rates) / len(rates)
    sample_desc = "full depth 16 and batch 256 of config 4, %d of 100 timesteps per step, fp32 on bf16-rounded inputs" % sample
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "stacked LSTM D16 H1024 I1024 N256 L100 (benchmark config 4)", "sample": sample_desc},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample_desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def other_configs(ops, dense, dev, pk):
    """The path's other benchmark configurations, each timed alone on the resident data with CUDA
    events after 3 warm-up calls (rank 0, single-GPU runs only): the B2B GEMM against the HBM
    roofline, attention against the tensor roofline, and the latency-bound wavefronts as times."""
    import math

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

    out = []
    g = torch.Generator(device=dev).manual_seed(1)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    uni = lambda b, *s: (torch.rand(*s, device=dev, generator=g) * 2 - 1) * b

    # config 2: 16 x [16384,128].[128,128].[128,128], fp16; three buffer sets in turn (each > L2)
    s = 1 / math.sqrt(128)
    sets = [((rnd(16, 16384, 128) * s).half(), (rnd(16, 128, 128) * s).half(), (rnd(16, 128, 128) * s).half(),
             torch.empty(16, 16384, 128, device=dev, dtype=torch.half)) for _ in range(3)]
    turn = [0]

    def b2b():
        turn[0] = (turn[0] + 1) % 3
        ops.b2b_gemm(*sets[turn[0]])

    ms = timed(b2b, 60)
    nbytes = 16 * (2 * 16384 * 128 + 2 * 128 * 128) * 2
    out.append({"config": "2: fused two GEMMs 16x(16384x128x128x128) fp16", "ms": ms, "bound": "hbm",
                "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": pk["hbm"], "unit": "GB/s",
                "frac": nbytes / (ms * 1e-3) / 1e9 / pk["hbm"], "tflops": 16 * 4 * 16384 * 128 * 128 / (ms * 1e-3) / 1e12,
                "cache": "three rotating buffer sets of 135 MB"})
    del sets

    # config 3: attention B16 h16 S2048 d128 fp16 (q, k, v, o: 537 MB > L2)
    q, k, v = (rnd(16, 16, 2048, 128).half() for _ in range(3))
    o = torch.empty_like(q)
    ms = timed(lambda: ops.flash_attention(q, k, v, scale=1 / math.sqrt(128), out=o), 20)
    fl = 4 * 16 * 16 * 2048 * 2048 * 128
    out.append({"config": "3: flash attention B16 h16 S2048 d128 fp16", "ms": ms, "bound": "tensor",
                "achieved": fl / (ms * 1e-3) / 1e12, "peak": pk["burst"], "unit": "TFLOP/s",
                "frac": fl / (ms * 1e-3) / 1e12 / pk["burst"]})
    ms = timed(lambda: ops.flash_attention(q, k, v, scale=1 / math.sqrt(128), out=o, causal=True), 20)
    fl = 2 * 16 * 16 * 2048 * 2049 * 128  # visible (query, key) pairs only
    out.append({"config": "3 with a causal mask (not a reference configuration)", "ms": ms, "bound": "tensor",
                "achieved": fl / (ms * 1e-3) / 1e12, "peak": pk["burst"], "unit": "TFLOP/s",
                "frac": fl / (ms * 1e-3) / 1e12 / pk["burst"]})
    del q, k, v, o

    # config 5a: dilated LSTM, 6 layers, dilation 2^l, H256 N256 L512 fp16
    x = rnd(512, 256, 256).half()
    Wp, _ = ops.lstm_pack_weights(uni(1 / 16, 6, 4, 256, 256).half(), uni(1 / 16, 6, 4, 256, 256).half())
    dil = [2 ** l for l in range(6)]
    ms = timed(lambda: ops.lstm_dilated(x, Wp, dil), 5)
    out.append({"config": "5a: dilated LSTM 6 layers H256 N256 L512 fp16", "ms": ms,
                "samples_steps_per_s": 256 * 512 / (ms * 1e-3), "bound": "latency (about 520 dependent levels)"})

    # config 5b: grid RNN 32x32, H256, N64, fp16
    X, Y = rnd(32, 32, 64, 256).half(), rnd(32, 32, 64, 256).half()
    Wpx = ops.grid_pack_weights(uni(1 / 16, 1, 512, 256).half(), uni(1 / 16, 1, 256, 256).half())
    Wpy = ops.grid_pack_weights(uni(1 / 16, 1, 512, 256).half(), uni(1 / 16, 1, 256, 256).half())
    ms = timed(lambda: ops.grid_rnn(X, Y, Wpx, Wpy), 10)
    out.append({"config": "5b: grid RNN 32x32 H256 N64 fp16", "ms": ms,
                "cells_per_s": 32 * 32 * 64 / (ms * 1e-3), "bound": "latency (63 anti-diagonals)"})

    # stand-alone online softmax, fp32 16384 x 4096 (three input/output pairs in turn, 1.6 GB > L2)
    xs = [rnd(16384, 4096) for _ in range(3)]
    ys = [torch.empty_like(xs[0]) for _ in range(3)]

    def softmax():
        turn[0] = (turn[0] + 1) % 3
        ops.online_softmax(xs[turn[0]], ys[turn[0]])

    ms = timed(softmax, 30)
    nbytes = 2 * 16384 * 4096 * 4
    out.append({"config": "online softmax fp32 16384x4096", "ms": ms, "bound": "hbm",
                "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": pk["hbm"], "unit": "GB/s",
                "frac": nbytes / (ms * 1e-3) / 1e9 / pk["hbm"], "cache": "three rotating buffer pairs of 537 MB"})
    del xs, ys

    # embedding lookup in front of config 4: 25 600 words, table 50 000 x 1024 bf16
    table = rnd(50000, 1024).bfloat16()
    ids = torch.randint(0, 50000, (25600,), device=dev, generator=g)
    rows_out = torch.empty(25600, 1024, device=dev, dtype=torch.bfloat16)
    ms = timed(lambda: ops.embedding_gather(table, ids, rows_out), 30)
    nbytes = 25600 * (2 * 1024 * 2 + 8)
    out.append({"config": "embedding lookup 25600 words, table 50000x1024 bf16", "ms": ms, "bound": "hbm",
                "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": pk["hbm"], "unit": "GB/s",
                "frac": nbytes / (ms * 1e-3) / 1e9 / pk["hbm"],
                "cache": "105 MB per call: fits L2, so this is a launch- and latency-bound size"})
    del table, ids, rows_out

    # config 1: stacked LSTM fp32 D4 H256 N32 L64 (CUDA cores; the reference's own CPU-runnable case)
    x1, W1, U1, _ = dense.make_lstm_inputs(4, 64, 32, 256, 256, 0, 1.0 / 16)
    Wp1, _ = ops.lstm_pack_weights(W1.to(dev), U1.to(dev))
    x1 = x1.to(dev)
    ms = timed(lambda: ops.lstm_stacked(x1, Wp1), 10)
    out.append({"config": "1: stacked LSTM fp32 D4 H256 N32 L64", "ms": ms,
                "samples_steps_per_s": 32 * 64 / (ms * 1e-3), "bound": "latency (67 levels), fp32 on CUDA cores"})
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ftb200", choices=["ftb200", "reference"])
    ap.add_argument("--layers-per-group", type=int, default=0)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ftb200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    from fractaltensor_b200 import ops, sharding
    from fractaltensor_b200._lib import lib
    from oracle import dense  # seeded synthetic inputs + the cpu_baseline leg only

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    D, L, N, I, H = CFG["D"], CFG["L"], CFG["N"], CFG["I"], CFG["H"]
    # Every rank draws its own 256-sample shard of the global batch (seed offset by rank).
    x_host, W, U, _ = dense.make_lstm_inputs(D, L, N, I, H, CFG["seed"] + 1000 * rank, CFG["w_bound"],
                                             dtype=torch.bfloat16)
    _, W, U, _ = dense.make_lstm_inputs(D, 1, 1, I, H, CFG["seed"], CFG["w_bound"], dtype=torch.bfloat16)
    Wp, _ = ops.lstm_pack_weights(W.to(dev), U.to(dev))
    del W, U
    x_pinned = x_host.pin_memory()
    x_dev = x_pinned.to(dev)
    hs = torch.empty(D, L, N, H, dtype=torch.bfloat16, device=dev)
    c = torch.empty(D, N, H, dtype=torch.float32, device=dev)
    out_pinned = torch.empty(L, N, H, dtype=torch.bfloat16).pin_memory()
    gathered = torch.empty(world * L, N, H, dtype=torch.bfloat16, device=dev) if world > 1 else None

    # Multi-GPU steps: the all-gather of step i's output runs on its own stream while step i+1's
    # wavefront computes into the other hidden-state buffer; a step is complete when its gather is.
    s_comm = torch.cuda.Stream(device=dev) if world > 1 else None
    hs_pair = [hs, torch.empty_like(hs)] if world > 1 else [hs]
    gathered_pair = [gathered, torch.empty_like(gathered)] if world > 1 else None
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_gathered = [torch.cuda.Event() for _ in range(2)]
    res_state = {"i": 0}

    def step_resident():
        if world == 1:
            ops.lstm_stacked(x_dev, Wp, None, hs, c, layers_per_group=args.layers_per_group, bn=args.bn)
            return
        i = res_state["i"]
        b = i & 1
        cur = torch.cuda.current_stream()
        if i >= 2:
            cur.wait_event(ev_gathered[b])  # hs_pair[b] was read by the gather of step i-2
        ops.lstm_stacked(x_dev, Wp, None, hs_pair[b], c, layers_per_group=args.layers_per_group, bn=args.bn)
        ev_done[b].record(cur)
        with torch.cuda.stream(s_comm):
            s_comm.wait_event(ev_done[b])
            dist.all_gather_into_tensor(gathered_pair[b], hs_pair[b][D - 1].reshape(L, N, H))
            ev_gathered[b].record(s_comm)
        res_state["i"] = i + 1

    def drain_resident():
        if world > 1:
            cur = torch.cuda.current_stream()
            for ev in ev_gathered:
                cur.wait_event(ev)

    # End-to-end pipeline: every step copies its input from pinned host memory, runs the forward
    # through the public operator and copies the top layer's hidden states back to pinned host
    # memory; three streams and two buffer sets let step i's copies overlap step i+-1's compute.
    s_in, s_run, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
    x_buf = [torch.empty_like(x_dev) for _ in range(2)]
    hs_buf = hs_pair if world > 1 else [hs, torch.empty_like(hs)]
    out_buf = [out_pinned, torch.empty_like(out_pinned).pin_memory()]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_run = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    e2e_state = {"i": 0}

    def step_e2e():
        i = e2e_state["i"]
        b = i & 1
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_run[b])   # x_buf[b] was read by step i-2
            x_buf[b].copy_(x_pinned, non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_in[b])
            if i >= 2:
                s_run.wait_event(ev_out[b])  # hs_buf[b] was copied out by step i-2
            ops.lstm_stacked(x_buf[b], Wp, None, hs_buf[b], c, layers_per_group=args.layers_per_group, bn=args.bn)
            ev_run[b].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_run[b])
            out_buf[b].copy_(hs_buf[b][D - 1], non_blocking=True)
            ev_out[b].record(s_out)
        e2e_state["i"] = i + 1

    def timed_e2e(steps):
        barrier()
        e2e_state["i"] = 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cur = torch.cuda.current_stream()
        e0.record(cur)
        for st in (s_in, s_run, s_out):
            st.wait_event(e0)
        for _ in range(steps):
            step_e2e()
        for ev in ev_out:
            cur.wait_event(ev)
        e1.record(cur)
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        drain_resident()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to start: launch it before the warm-up
    for _ in range(args.warmup):
        step_resident()
    drain_resident()
    ops.check_status()

    n0 = lib.ftb_launch_count()
    t_begin = time.perf_counter()
    total_ms = timed(step_resident, args.steps)
    t_end = time.perf_counter()
    launches = lib.ftb_launch_count() - n0
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    ops.check_status()

    timed_e2e(2)
    e2e_ms = timed_e2e(args.steps)
    ops.check_status()
    torch.cuda.synchronize()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_per_step = total_ms / args.steps
    value = world * N * L / (ms_per_step * 1e-3)
    e2e_value = world * N * L / (e2e_ms / args.steps * 1e-3)
    pk = peaks()
    peak_kind = "sustained" if total_ms >= 1000.0 else "burst"
    # Dominant kernel: lstm_static_kernel, one cooperative launch per step that does the whole
    # wavefront (6.872 TFLOP); nothing else of ours launches in a step, so the launch's duration
    # is the step's.
    flops_per_step = FLOPS_PER_SAMPLE_STEP * N * L
    achieved = flops_per_step / (ms_per_step * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": achieved, "peak": pk[peak_kind], "unit": "TFLOP/s",
                "frac": achieved / pk[peak_kind], "traffic": TRAFFIC_BYTES_PER_LAUNCH,
                "peak_source": "%s %s bf16 GEMM" % (pk["src"], peak_kind),
                "kernel": "lstm_static_kernel<bf16> (persistent, CTA pairs, static tile ownership)",
                "launches_per_step": launches / args.steps, "dominant_launches_per_step": 1,
                "avg_launch_us": 1e3 * ms_per_step, "flops_per_launch": flops_per_step}
    others = None
    if world == 1 and not args.no_other_configs:
        others = other_configs(ops, dense, dev, pk)
    cpu = None
    if world == 1 and not args.no_cpu_baseline:  # timed on rank 0 of single-GPU runs only
        threads = os.cpu_count() or 1
        sample = 50
        rate, dt = cpu_port_rate(sample, threads)
        cpu = {"value": rate, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": "full depth 16 and batch 256, %d of 100 timesteps, fp32 on bf16-rounded inputs (%.1f s)" % (sample, dt)}
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "stacked LSTM D16 H1024 I1024 N256/GPU L100, bf16 weights/activations, fp32 cell state "
                               "(benchmark config 4)", "global_batch": world * N, "seq_len": L,
                   "parallelism": "batch-sharded x%d, weights replicated, all-gather of top-layer output (on its own stream, overlapping the next step)" % world,
                   "cache": "per-step inputs exceed L2 (268 MB weights + 839 MB states vs 126 MB L2); no flush needed",
                   "layers_per_group": args.layers_per_group, "bn": args.bn},
        "roofline": roofline, "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": x_pinned.numel() * 2,
                "d2h_bytes_per_step": out_pinned.numel() * 2},
        "gpu_launches": int(launches), "clocks": clocks, "other_configs": others,
    }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
