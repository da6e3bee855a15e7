#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --benchmark --benchmark_input_seq_length 511 --benchmark_output_seq_length 256

Headline workload ("cfg4"): one decode step of a Qwen2.5-14B-shaped model's
attention -- 48 layers, batch 64, 40 query heads on 8 KV heads, head_dim 128,
bf16, per-sequence cache lengths uniform in [1024, 4096] from a seed, RoPE theta
1e6 -- with the KV heads sharded over the N GPUs (no collective on the data
path).  One step = the step's work partition uploaded once, then for every layer
one fused launch group: rotate the new token's Q/K, append K/V to the cache,
grouped-query attention over the cache, merge of the cut caches.  The metric is
algorithmic HBM GB/s (every K/V byte once + q/k/v in + o out), the sum over all
ranks divided by the slowest rank's device time.  K steps are timed as one
interval, five times over; the median interval gives the value.

Also in the same JSON line: `parity` (the step's output against the CPU checker,
every rank), the prefill leg ("cfg3": Llama-2-13B-shaped causal prefill, batch
8 x 2048 tokens, 40 heads, fp16; algorithmic TFLOP/s; "cfg5": 32768 tokens in
chunks), the end-to-end figure with host buffers through the host layer's C ABI,
the roofline of the dominant kernel, the reference's own measuring mode over the
attention layers (`benchmark_mode`) and the CPU restatement of the reference's
layer timed on the host cores (one thread, as the reference builds, and all cores).

Synthetic seeded N(0,1) tensors stand in for real activations (no checkpoints
here).  `--impl reference` times only the CPU restatement of the reference path
(the reference's own CPU layer needs Eigen/boost/spdlog, which are not
installed, so it cannot be built).
"""
import argparse
import concurrent.futures
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

D = 128
DT_FP16, DT_BF16 = 4, 5
MAX_ABS, MEAN_ABS = 1e-2, 1e-3   # the parity bound for fp16 / bf16 attention with fp32 accumulation

CFG4 = dict(name="cfg4 Qwen2.5-14B-shaped batched GQA decode", layers=48, batch=64, n_heads=40, n_kv_heads=8,
            len_lo=1024, len_hi=4096, theta=1e6, neox=True, seed=20254)
# DRAM bytes (read + write) per algorithmic byte of the decode kernel, from one profiler capture of
# this workload's one-layer launch on one GPU; a shard of the launch is scaled by its bytes
DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.010
CFG2 = dict(name="cfg2 Qwen2.5-1.5B-shaped GQA decode", layers=28, n_heads=12, n_kv_heads=2, theta=1e6, neox=True)
CFG3 = dict(name="cfg3 Llama-2-13B-shaped causal prefill", layers=40, batch=8, seq=2048, n_heads=40, theta=1e4,
            neox=False)
CFG5 = dict(name="cfg5 Qwen2.5-32B-shaped chunked causal prefill", batch=1, seq=32768, chunk=4096, n_heads=40,
            n_kv_heads=8, theta=1e6, neox=True)
REPEATS = 5


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], tensor=p["bf16_tflops"], tensor_sustained=p.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm=6650.0, tensor=1590.0, tensor_sustained=1400.0, source="fallback")


def decode_bytes(lens_with_new, n_heads, n_kv_heads):
    """Algorithmic bytes of one layer's decode step: K and V once, q in, o out,
    raw k/v in, rotated k and v appended."""
    eb = 2
    per_seq = [2 * n_kv_heads * L * D * eb + 2 * n_heads * D * eb + 4 * n_kv_heads * D * eb for L in lens_with_new]
    return float(sum(per_seq))


def prefill_flops(batch, heads, m, offset):
    """4*D per unmasked (row, col) pair."""
    pairs = m * offset + m * (m + 1) // 2
    return 4.0 * D * heads * batch * pairs


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None
        self.t_begin = self.t_end = None

    def start(self):
        """Starts sampling (20 ms period), before the warm-up: the first sample arrives about 0.1 s
        after the sampler starts."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __enter__(self):
        if self.proc is None:
            self.start()
        self.t_begin = time.monotonic()
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [x.strip() for x in line.split(",")]))

    def __exit__(self, *a):
        self.t_end = time.monotonic()
        if self.proc:
            time.sleep(0.03)          # let a sample taken inside the region arrive
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        sm, mx, reasons = [], [], set()
        for t, r in self.rows:
            if t < (self.t_begin or 0.0) or t > (self.t_end or 1e30) + 0.03:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for i, n in enumerate(names):
                if len(r) > 3 + i and r[3 + i].lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "window": "timed region (all repeats)",
                "seconds": round((self.t_end or 0) - (self.t_begin or 0), 3)}


# ----------------------------------------------------------------------------
# parity (the CPU checker: test infrastructure, never on the measured path)
# ----------------------------------------------------------------------------
def parity_stats(orc, out_bits, golden_f32, dt):
    """A 16-bit result against the checker's fp32 golden: max / mean absolute error against the
    fp32 values and against the golden rounded to the dtype (how the reference's tests compare,
    tests/rope_single_layer_test.cpp:97); whether every element is within max(1e-2, one ulp of the
    dtype) and the mean within 1e-3; and the reference's own all_close(1e-3, 1e-3) verdict."""
    out = orc.to_f32(out_bits, dt).ravel().astype(np.float64)
    g32 = np.asarray(golden_f32, dtype=np.float32).ravel()
    g16 = orc.to_f32(orc.to_bits(g32, dt), dt).astype(np.float64)
    d32, d16 = np.abs(out - g32), np.abs(out - g16)
    mant = 10 if dt == DT_FP16 else 7
    ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(g16), 2.0 ** -14))) - mant)
    over = d16 > MAX_ABS
    ok = bool(np.all(np.isfinite(out)) and d16.mean() <= MEAN_ABS and np.all(d16 <= np.maximum(MAX_ABS, ulp)))
    return {"max_abs": float(d16.max()), "mean_abs": float(d16.mean()), "max_abs_vs_fp32": float(d32.max()),
            "mean_abs_vs_fp32": float(d32.mean()), "elements": int(out.size),
            "elements_above_1e-2_within_one_ulp": int(over.sum()), "within_bound": ok,
            "reference_all_close_1e-3": orc.all_close(out.astype(np.float32), g16.astype(np.float32)),
            "mode": "fp32 golden of the CPU checker, rounded to the dtype"}


def merge_parity(items):
    """Worst case over several parity records."""
    items = [p for p in items if p]
    if not items:
        return None
    n = sum(p["elements"] for p in items)
    return {"max_abs": max(p["max_abs"] for p in items),
            "mean_abs": sum(p["mean_abs"] * p["elements"] for p in items) / n,
            "max_abs_vs_fp32": max(p["max_abs_vs_fp32"] for p in items),
            "mean_abs_vs_fp32": sum(p["mean_abs_vs_fp32"] * p["elements"] for p in items) / n,
            "elements": n,
            "elements_above_1e-2_within_one_ulp": sum(p["elements_above_1e-2_within_one_ulp"] for p in items),
            "within_bound": all(p["within_bound"] for p in items),
            "reference_all_close_1e-3": all(p["reference_all_close_1e-3"] for p in items),
            "mode": items[0]["mode"]}


def oracle_decode_rows(orc, q, k_new, v_new, kc_head, vc_head, L, table, H, kvh, neox, dt):
    """One sequence's decode step on the CPU: rope -> append -> attention, fp32 golden.
    q [H*D], k_new / v_new [kvh*D] bits; kc_head / vc_head [kvh][>=L][D] bits (head-major)."""
    kc = np.ascontiguousarray(kc_head[:, :L + 1].transpose(1, 0, 2)).reshape(L + 1, kvh * D)
    vc = np.ascontiguousarray(vc_head[:, :L + 1].transpose(1, 0, 2)).reshape(L + 1, kvh * D)
    q_r = orc.rope_single_layer(q.reshape(1, -1), table, L, H, neox, dt)
    k_r = orc.rope_single_layer(k_new.reshape(1, -1), table, L, kvh, neox, dt)
    orc.kv_append(kc, vc, k_r, v_new.reshape(1, -1), L, kvh, D)
    return orc.attn(q_r, kc, vc, 1, L + 1, L, H // kvh, kvh, D, dt, orc.MODE_GOLDEN, threads=min(8, host_cores()))[0]


def bits(t):
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


# ----------------------------------------------------------------------------
# CPU restatement of the reference layer, timed (cpu_baseline / --impl reference)
# ----------------------------------------------------------------------------
def cpu_decode_layer(orc, cfg, lens, threads, rng):
    """One layer of the decode step on the host, the way the reference's layer runs it: rope(q),
    rope(k) -> append -> attention with the layer's rounding points, sequence by sequence; with
    more than one thread the sequences are spread over a pool (the reference itself is built
    without threading, src/CMakeLists.txt).  Returns seconds."""
    H, kvh = cfg["n_heads"], cfg["n_kv_heads"]
    dt = orc.DT_BFLOAT16
    table = orc.init_freq_cis(D, max(lens) + 1, cfg["theta"], dt)
    caches = [(orc.to_bits(rng.standard_normal((L + 1, kvh * D), dtype=np.float32), dt),
               orc.to_bits(rng.standard_normal((L + 1, kvh * D), dtype=np.float32), dt)) for L in lens]
    q = orc.to_bits(rng.standard_normal((len(lens), H * D), dtype=np.float32), dt)
    k = orc.to_bits(rng.standard_normal((len(lens), kvh * D), dtype=np.float32), dt)
    v = orc.to_bits(rng.standard_normal((len(lens), kvh * D), dtype=np.float32), dt)

    def one(b):
        L = lens[b]
        kc, vc = caches[b]
        q_r = orc.rope_single_layer(q[b:b + 1], table, L, H, cfg["neox"], dt)
        k_r = orc.rope_single_layer(k[b:b + 1], table, L, kvh, cfg["neox"], dt)
        orc.kv_append(kc, vc, k_r, v[b:b + 1], L, kvh, D)
        orc.attn(q_r, kc, vc, 1, L + 1, L, H // kvh, kvh, D, dt, orc.MODE_STRICT, threads=1)

    t0 = time.perf_counter()
    if threads <= 1:
        for b in range(len(lens)):
            one(b)
    else:
        with concurrent.futures.ThreadPoolExecutor(max_workers=threads) as pool:
            list(pool.map(one, range(len(lens))))
    return time.perf_counter() - t0


def cpu_figure(orc, cfg, lens, threads, budget_s, min_runs=1):
    rng = np.random.default_rng(7)
    nbytes = decode_bytes([L + 1 for L in lens], cfg["n_heads"], cfg["n_kv_heads"])
    times, t_start = [], time.perf_counter()
    while len(times) < min_runs or (time.perf_counter() - t_start < budget_s and len(times) < 5):
        times.append(cpu_decode_layer(orc, cfg, lens, threads, rng))
    return nbytes / min(times) / 1e9, min(times), len(times)


def cpu_baseline(cfg, lens):
    """The checker's restatement of the reference layer on the host cores: one thread (how the
    reference is built) on a quarter of the batch, and every core on the whole batch."""
    from oracle import oracle as orc
    cores = host_cores()
    all_gbs, all_s, all_n = cpu_figure(orc, cfg, lens, cores, 8.0)
    sub = lens[:max(1, len(lens) // 4)]
    one_gbs, one_s, one_n = cpu_figure(orc, cfg, sub, 1, 6.0)
    return {"value": all_gbs, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": "1 layer x all %d sequences, %d repeats, best; the reference layer's rounding points; "
                      "sequences spread over %d threads" % (len(lens), all_n, cores),
            "seconds": all_s,
            "single_thread": {"value": one_gbs, "unit": "GB/s", "cores": 1, "seconds": one_s,
                              "sample": "1 layer x %d of %d sequences, %d repeats, best (the reference builds "
                                        "without threading)" % (len(sub), len(lens), one_n)}}


def config_of(cfg, layers, batch, world, shard_of, launch, early, bytes_layer_rank):
    return {"workload": cfg["name"], "layers": layers, "batch": batch, "n_heads": cfg["n_heads"],
            "n_kv_heads": cfg["n_kv_heads"], "head_dim": D,
            "kv_len": "uniform[%d,%d] seed %d" % (cfg["len_lo"], cfg["len_hi"], cfg["seed"]),
            "sharding": "kv-head x%d" % world if shard_of <= 1 else
                        "rank 0's shard of a kv-head x%d split, alone on one GPU" % (world * shard_of),
            "launch": launch, "early_kv_prefetch": early, "cache_layout": "head-major",
            "l2": "inputs larger than L2 (%.0f MB per layer, %.1f GB per step per rank)"
                  % (bytes_layer_rank / 1e6, bytes_layer_rank * layers / 1e9)}


def run_reference_arm(args, cfg, lens):
    """The reference's CPU implementation of the path (its restatement: the reference itself cannot
    be built here) on the host cores; each step = one of the layers, the whole batch."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc
    cores = host_cores()     # the launcher's OMP_NUM_THREADS does not matter: the thread count is passed
    rng = np.random.default_rng(7)
    nbytes = decode_bytes([L + 1 for L in lens], cfg["n_heads"], cfg["n_kv_heads"])
    for _ in range(args.warmup):
        cpu_decode_layer(orc, cfg, lens, cores, rng)
    t = 0.0
    for _ in range(args.steps):
        t += cpu_decode_layer(orc, cfg, lens, cores, rng)
    value = nbytes * args.steps / t / 1e9
    sub = lens[:max(1, len(lens) // 4)]
    one_gbs, one_s, one_n = cpu_figure(orc, cfg, sub, 1, 6.0)
    conf = config_of(cfg, cfg["layers"], cfg["batch"], max(args.gpus, 1), 1, "host threads", False,
                     nbytes / max(args.gpus, 1))
    conf["note"] = "CPU restatement of the reference layer on the host cores; each step = 1 of the layers"
    line = {
        "impl": "reference", "metric": "attn decode HBM GB/s per layer", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": conf,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "each step = 1 of %d layers, all %d sequences, spread over %d threads"
                                   % (cfg["layers"], len(lens), cores),
                         "single_thread": {"value": one_gbs, "unit": "GB/s", "cores": 1, "seconds": one_s,
                                           "sample": "1 layer x %d of %d sequences, %d repeats, best"
                                                     % (len(sub), len(lens), one_n)}},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------
class Env:
    """What every leg needs."""
    pass


def timed_repeats(env, step, steps, repeats=REPEATS, min_total_s=0.0, queue_behind_ms=0.0):
    """Times `steps` calls of step() as one CUDA-event interval on env.stream, `repeats` times (more
    until min_total_s of device time has been covered); a barrier and a synchronize on both sides of
    every interval; the maximum over the ranks per interval.  Returns the list of ms per interval.
    queue_behind_ms > 0: the interval starts behind a sleep kernel of that length, so that the host has
    queued the launches by the time the device gets to them and the interval holds device time, not the
    rate at which this script can issue launches."""
    torch, dist = env.torch, env.dist
    out, total = [], 0.0
    while len(out) < repeats or total < min_total_s * 1e3:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        env.barrier()
        if queue_behind_ms > 0:
            with torch.cuda.stream(env.stream):
                torch.cuda._sleep(int(queue_behind_ms * 1e-3 * 1.9e9))
        e0.record(env.stream)
        for _ in range(steps):
            step()
        e1.record(env.stream)
        env.barrier()
        ms = e0.elapsed_time(e1)
        if env.world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=env.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        out.append(ms)
        total += ms
        if len(out) >= 200:
            break
    return out


def spread(ms_list, per=1.0):
    return {"median": statistics.median(ms_list) / per, "min": min(ms_list) / per, "max": max(ms_list) / per,
            "repeats": len(ms_list)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (profiling on a small case)")
    ap.add_argument("--batch", type=int, default=None, help="override the batch (profiling on a small case)")
    ap.add_argument("--no-extras", action="store_true", help="headline leg only: no parity, prefill, e2e, CPU legs")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="on ONE GPU, run rank 0's shard of an N-way KV-head split (sizing a multi-GPU shard)")
    ap.add_argument("--early-prefetch", type=int, default=1,
                    help="1: the decode kernel requests its first K/V tiles before the preceding kernels of the "
                         "stream have finished (legal here: consecutive launches read different layers' caches)")
    ap.add_argument("--graph", type=int, default=1,
                    help="1: replay the step's launches from a CUDA graph (default), 0: launch them one by one")
    ap.add_argument("--planned", type=int, default=1,
                    help="1: gpu_attn_decode_planned_layer on a per-step work partition (default); 0: "
                         "gpu_attn_decode_layer, which cuts every cache into equal splits on the device")
    ap.add_argument("--leg", default="all", choices=["all", "prefill"],
                    help="prefill: run only the prefill leg (small, for profiling) and print its object")
    ap.add_argument("--benchmark", action="store_true",
                    help="only the reference's measuring mode (Qwen2Model::Benchmark, src/qwen2_model.cpp:225-255) "
                         "over the attention layers: a prompt of --benchmark_input_seq_length tokens, then decode "
                         "steps until input + output tokens; time to first token and ms per step")
    ap.add_argument("--benchmark_input_seq_length", type=int, default=511)
    ap.add_argument("--benchmark_output_seq_length", type=int, default=256)
    ap.add_argument("--benchmark_config", default="cfg2", choices=["cfg2", "cfg3"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    cfg = dict(CFG4)
    if args.layers:
        cfg["layers"] = args.layers
    if args.batch:
        cfg["batch"] = args.batch
    rng = np.random.default_rng(cfg["seed"])
    lens = [int(x) for x in rng.integers(cfg["len_lo"], cfg["len_hi"] + 1, size=cfg["batch"])]

    if args.impl == "reference":
        run_reference_arm(args, cfg, lens)
        return

    import torch
    import torch.distributed as dist
    from llm_simple_b200 import layer as lay
    from llm_simple_b200 import ops

    env = Env()
    env.torch, env.dist, env.ops, env.lay = torch, dist, ops, lay
    env.world = int(os.environ.get("WORLD_SIZE", "1"))
    env.rank = int(os.environ.get("RANK", "0"))
    env.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(env.local_rank)
    env.dev = torch.device("cuda", env.local_rank)
    if env.world > 1:
        # keep stdout for the one JSON line: NCCL prints its version banner there at VERSION level
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=env.dev)
    ops.lib()
    env.pk = peaks()
    env.stream = torch.cuda.current_stream()
    env.args = args

    def barrier():
        if env.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    env.barrier = barrier

    def table(max_pos, theta, dt):
        """The RoPE table as the product's host layer builds it (gpu_init_freq_cis)."""
        return torch.from_numpy(lay.init_freq_cis(D, max_pos, theta, dt)).to(env.dev)
    env.table = table

    if args.benchmark:
        res = benchmark_mode_leg(env, args.benchmark_config, args.benchmark_input_seq_length,
                                 args.benchmark_output_seq_length, check=True)
        if env.rank == 0:
            print(json.dumps({"benchmark_mode": res}))
        if env.world > 1:
            dist.destroy_process_group()
        return
    if args.leg == "prefill":
        res = prefill_leg(env, check=False)
        if env.rank == 0:
            print(json.dumps({"prefill": res}))
        if env.world > 1:
            dist.destroy_process_group()
        return

    world, rank, dev = env.world, env.rank, env.dev
    H, kvh = cfg["n_heads"], cfg["n_kv_heads"]
    if kvh % world:
        raise SystemExit("KV heads (%d) do not divide over %d ranks" % (kvh, world))
    split = world * max(args.shard_of, 1)
    if kvh % split:
        raise SystemExit("KV heads (%d) do not divide into %d shards" % (kvh, split))
    kvh_l, H_l = kvh // split, H // split
    head0 = rank * kvh_l if args.shard_of <= 1 else 0     # first KV head of this rank's shard
    layers, batch = cfg["layers"], cfg["batch"]
    max_pos = cfg["len_hi"] + 8
    max_kv = max(lens) + 1

    # ---- device state: per-layer head-major caches [batch][kvh_l][max_pos][D], seeded N(0,1)
    gen = torch.Generator(device=dev)
    gen.manual_seed(cfg["seed"] + rank)
    k_cache = [torch.empty((batch, kvh_l, max_pos, D), dtype=torch.bfloat16, device=dev).normal_(generator=gen)
               for _ in range(layers)]
    v_cache = [torch.empty((batch, kvh_l, max_pos, D), dtype=torch.bfloat16, device=dev).normal_(generator=gen)
               for _ in range(layers)]
    q_in = torch.empty((layers, batch, H_l * D), dtype=torch.bfloat16, device=dev).normal_(generator=gen)
    k_in = torch.empty((layers, batch, kvh_l * D), dtype=torch.bfloat16, device=dev).normal_(generator=gen)
    v_in = torch.empty((layers, batch, kvh_l * D), dtype=torch.bfloat16, device=dev).normal_(generator=gen)
    out = torch.empty((layers, batch, H_l * D), dtype=torch.bfloat16, device=dev)
    tab = table(max_pos, cfg["theta"], DT_BF16)
    lens_d = torch.tensor(lens, dtype=torch.int32, device=dev)
    desc = ops.make_desc(DT_BF16, batch, H_l, kvh_l, 1, max_pos, layout="head", is_neox=cfg["neox"])
    desc.total_kv_len = sum(L + 1 for L in lens)   # scheduling hint of the unplanned entry point
    # consecutive launches work on different layers' caches and the lengths are fixed for the step
    ops.gpu_attn_set_decode_early_prefetch(args.early_prefetch)
    if args.planned:
        # the host knows the lengths (as the reference's generation loop knows cur_pos): one work
        # partition per step, uploaded once, shared by the step's layers
        plan = ops.DecodePlan(desc, lens, True)
        plan.upload(dev)
        ws_bytes = plan.workspace_bytes
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)

        def step(st=None):
            st = st or env.stream
            for l in range(layers):
                ops.gpu_attn_decode_planned_layer(desc, None, plan, out[l], None, None, q_in[l], k_in[l], v_in[l],
                                                  k_cache[l], v_cache[l], tab, None, ws, ws_bytes, stream=st)
        kernel_name = "attn_decode_tma_kernel (+ attn_plan_merge_kernel, one launch pair per layer)"
    else:
        ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, max_kv)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)

        def step(st=None):
            st = st or env.stream
            for l in range(layers):
                ops.gpu_attn_decode_layer(desc, out[l], None, None, q_in[l], k_in[l], v_in[l], k_cache[l], v_cache[l],
                                          tab, lens_d, None, True, max_kv, ws, ws_bytes, stream=st)
        kernel_name = "attn_decode_kernel (+ attn_merge_kernel, one launch pair per layer)"

    run_step, graph, launches_per_step = step, None, None
    step()
    barrier()
    ops.gpu_ops_launch_count(True)
    if args.graph:
        # A decode step is a fixed sequence of launches: capture it once and replay it, as a
        # serving loop would; this removes the per-call host cost (a few per cent of the step).
        try:
            cap = torch.cuda.Stream(device=dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(cap):
                graph.capture_begin()
                step(cap)
                graph.capture_end()
            run_step = graph.replay
        except Exception as e:  # capture unavailable: launch call by call
            sys.stderr.write("cuda graph capture failed (%s); launching call by call\n" % e)
            graph = None
    else:
        step()
    launches_per_step = ops.gpu_ops_launch_count(True)

    sampler = ClockSampler(env.local_rank).start()
    for _ in range(max(args.warmup, 3)):
        run_step()
    # keep the load up until the sampler has delivered its first row (nvidia-smi takes up to a few seconds to
    # start on a box with many GPUs), so that the timed region below is always covered by samples
    t_wait = time.monotonic()
    while not sampler.rows and sampler.proc is not None and time.monotonic() - t_wait < 5.0:
        run_step()
        torch.cuda.synchronize()
    barrier()
    with sampler as clk:
        # at least five intervals of K steps, and more until 0.3 s are covered, so that the clock
        # sampler always sees the timed load
        ms_list = timed_repeats(env, run_step, args.steps, REPEATS, min_total_s=0.3)
    launches = launches_per_step * args.steps
    if world > 1:
        lt = torch.tensor([launches], dtype=torch.int64, device=dev)
        dist.all_reduce(lt)
        launches = int(lt.item())
    ms_per_step = statistics.median(ms_list) / args.steps
    so = max(args.shard_of, 1)
    bytes_layer_all = decode_bytes([L + 1 for L in lens], H // so, kvh // so)  # all ranks, one layer
    bytes_layer_rank = decode_bytes([L + 1 for L in lens], H_l, kvh_l)    # this rank, one layer
    value = bytes_layer_all * layers / (ms_per_step * 1e-3) / 1e9
    layer_ms = ms_per_step / layers
    achieved = bytes_layer_rank / (layer_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": env.pk["hbm"], "unit": "GB/s",
                "frac": achieved / env.pk["hbm"], "traffic": DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE * bytes_layer_rank,
                "traffic_source": "profiler capture of the one-layer launch (dram bytes read + written = 1.010 x "
                                  "algorithmic), scaled by the algorithmic bytes of this launch; not measured in this run",
                "peak_source": env.pk["source"], "kernel": kernel_name, "launch_ms": layer_ms,
                "algorithmic_bytes_per_launch": bytes_layer_rank, "frac_of_nominal_8TBs": achieved / 8000.0}
    launch = ("cuda graph of the step's %d launches" % launches_per_step) if graph is not None else "one call per layer"
    conf = config_of(cfg, layers, batch, world, args.shard_of, launch, bool(args.early_prefetch), bytes_layer_rank)
    conf["entry_point"] = "gpu_attn_decode_planned_layer" if args.planned else "gpu_attn_decode_layer"
    if args.planned:
        conf["plan"] = {"ctas": plan.header["n_ctas"], "pieces": plan.header["n_items"],
                        "cut_caches": plan.header["n_groups"]}
    line = {
        "metric": "attn decode HBM GB/s per layer", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": conf,
        "ms_per_step_spread": spread(ms_list, args.steps), "roofline": roofline, "clocks": clk.summary(),
        "gpu_launches": launches, "kernel_status": ops.gpu_ops_kernel_status(),
    }

    if not args.no_extras:
        def leg(name, fn, *a, **kw):
            # an extra leg that fails must not cost the headline line; every rank takes the same path,
            # because a failure inside a collective leg raises on all of them
            try:
                line[name] = fn(*a, **kw)
            except Exception as e:  # noqa: BLE001
                line[name] = {"error": "%s: %s" % (type(e).__name__, e)}
                sys.stderr.write("leg %s failed: %s\n" % (name, e))
        leg("parity", decode_parity_leg, env, cfg, lens, out, q_in, k_in, v_in, k_cache, v_cache, H_l, kvh_l, head0)
        leg("e2e", e2e_leg, env, cfg, lens, k_cache, v_cache, tab, H_l, kvh_l, bytes_layer_all)
        leg("prefill", prefill_leg, env)
        leg("cfg5_split_kv_decode", split_kv_leg, env)
        if world == 1:
            leg("other_configs", other_configs_leg, env)
            leg("paged_decode", paged_leg, env, cfg, lens, tab, H_l, kvh_l)
            leg("benchmark_mode", lambda: {c: benchmark_mode_leg(env, c, None, None, check=True)
                                           for c in ("cfg2", "cfg3")})
        if rank == 0 and world == 1:
            leg("cpu_baseline", cpu_baseline, cfg, lens)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def decode_parity_leg(env, cfg, lens, out, q_in, k_in, v_in, k_cache, v_cache, H_l, kvh_l, head0):
    """Untimed: this rank's output of the step (layer 0 and the last layer; the shortest, the longest
    and two more sequences) against the CPU checker run the way the reference's layer does it (rope ->
    append -> attention); every rank checks its own KV-head shard, rank 0 reports the worst case."""
    from oracle import oracle as orc
    torch, dist = env.torch, env.dist
    order = np.argsort(lens)
    seqs = sorted({int(order[0]), int(order[-1]), int(order[len(order) // 3]), int(order[2 * len(order) // 3])})
    tab = orc.init_freq_cis(D, max(lens) + 2, cfg["theta"], orc.DT_BFLOAT16)
    assert np.array_equal(tab.view(np.uint32),
                          env.lay.init_freq_cis(D, max(lens) + 2, cfg["theta"], DT_BF16).view(np.uint32))
    recs, rows_equal = [], True
    for l in sorted({0, len(out) - 1}):
        for b in seqs:
            L = lens[b]
            kc, vc = bits(k_cache[l][b, :, :L + 1]), bits(v_cache[l][b, :, :L + 1])
            gold = oracle_decode_rows(orc, bits(q_in[l][b]), bits(k_in[l][b]), bits(v_in[l][b]), kc, vc, L, tab, H_l,
                                      kvh_l, cfg["neox"], orc.DT_BFLOAT16)
            recs.append(parity_stats(orc, bits(out[l][b]), gold, orc.DT_BFLOAT16))
            # the appended row holds the checker's rotated K and the raw V, bit for bit
            k_r = orc.rope_single_layer(bits(k_in[l][b]).reshape(1, -1), tab, L, kvh_l, cfg["neox"], orc.DT_BFLOAT16)
            rows_equal &= bool(np.array_equal(kc[:, L].reshape(-1), k_r.reshape(-1)) and
                               np.array_equal(vc[:, L].reshape(-1), bits(v_in[l][b]).reshape(-1)))
    mine = merge_parity(recs)
    mine["appended_rows_bit_identical"] = rows_equal
    mine["checked"] = "layers 0 and %d, sequences %s of every rank's KV-head shard (first KV head %d here)" % (
        len(out) - 1, seqs, head0)
    if env.world > 1:
        gathered = [None] * env.world
        dist.all_gather_object(gathered, mine)
        worst = merge_parity(gathered)
        worst["appended_rows_bit_identical"] = all(g["appended_rows_bit_identical"] for g in gathered)
        worst["checked"] = mine["checked"]
        worst["ranks"] = env.world
        return worst
    return mine


def e2e_leg(env, cfg, lens, k_cache, v_cache, tab, H_l, kvh_l, bytes_layer_all):
    """The same step through the host layer with HOST buffers: one attention-layer object per layer
    (llm_simple_b200.layer.AttentionLayer, the mirror of the reference's Qwen2 layer class) adopts
    that layer's KV cache; the model-level step state (lengths -> work partition) is prepared once
    per step; every layer call takes the new token's packed q/k/v row from pinned host memory and
    returns the attention output to pinned host memory, the copies enqueued around the kernels inside
    the timed region.  Headline: everything on ONE stream, as a stack whose layers depend on each
    other must run.  Beside it: the layers alternating between two streams, which this benchmark's
    independent layers allow and a real stack's do not."""
    torch, ops, lay, args = env.torch, env.ops, env.lay, env.args
    layers, batch = cfg["layers"], cfg["batch"]
    dev = env.dev
    qkv_w = (H_l + 2 * kvh_l) * D
    h_in = torch.empty((layers, batch, qkv_w), dtype=torch.bfloat16).normal_().pin_memory()
    h_out = torch.empty((layers, batch, H_l * D), dtype=torch.bfloat16).pin_memory()
    max_pos = cfg["len_hi"] + 8
    step_state = lay.DecodeStep(batch, H_l, kvh_l, DT_BF16)
    objs = []
    for l in range(layers):
        o = lay.AttentionLayer(lay.QWEN2, H_l, kvh_l, max_pos, batch, DT_BF16, cfg["theta"], cfg["neox"],
                               lay.HEAD_MAJOR, shared_freq_cis=tab, k_cache=k_cache[l], v_cache=v_cache[l])
        o.set_shared_step(step_state)
        objs.append(o)
    cur = env.stream
    side = [torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)]
    steps = max(3, args.steps // 2)
    res = {}
    for name, streams in (("one_stream", [cur]), ("two_streams", side)):
        def step():
            step_state.prepare(lens, True, stream=cur)      # once per step by the model, not per layer
            if len(streams) > 1:
                ev = torch.cuda.Event()
                ev.record(cur)
                for st in streams:
                    st.wait_event(ev)
            for l in range(layers):
                objs[l].forward_host(h_out[l], h_in[l], batch, 1, 0, stream=streams[l % len(streams)])
            if len(streams) > 1:
                for st in streams:
                    e = torch.cuda.Event()
                    e.record(st)
                    cur.wait_event(e)
        for _ in range(3):
            step()
        ops.gpu_ops_launch_count(True)
        ms_list = timed_repeats(env, step, steps, 3)
        per_step = statistics.median(ms_list) / steps
        res[name] = {"value": bytes_layer_all * layers / (per_step * 1e-3) / 1e9, "ms_per_step": per_step,
                     "ms_per_step_spread": spread(ms_list, steps)}
    head = res["one_stream"]
    out = {"value": head["value"], "unit": "GB/s",
           "h2d_bytes_per_step": int(layers * batch * qkv_w * 2 * env.world),
           "d2h_bytes_per_step": int(layers * batch * H_l * D * 2 * env.world), "ms_per_step": head["ms_per_step"],
           "ms_per_step_spread": head["ms_per_step_spread"], "steps": steps,
           "api": "gpu_decode_step_prepare once per step + gpu_attention_layer_forward_host per layer (C ABI of the "
                  "host layer): pinned host q/k/v row in, attention output back to pinned host memory, one caller "
                  "stream (the layer's default: its input copy runs on a stream of its own, so it overlaps the "
                  "previous layer's kernels; output copy and kernels on the caller's stream)",
           "two_streams": dict(res["two_streams"], note="layers alternate between two streams: possible only because "
                               "this benchmark's layers are independent; not the headline")}
    for o in objs:
        o.close()
    step_state.close()
    return out


def paged_leg(env, cfg, lens, tab, H_l, kvh_l, layers=4, page_size=256):
    """The decode step over a PAGED cache (pages of 256 positions handed out in random order), on
    `layers` layers with pools of their own: the same kernels, the page table looked up once per tile
    of 64 positions."""
    torch, ops, dev = env.torch, env.ops, env.dev
    batch = cfg["batch"]
    per_seq = (cfg["len_hi"] + 8 + page_size - 1) // page_size
    n_pages = batch * per_seq
    gen = torch.Generator(device=dev)
    gen.manual_seed(cfg["seed"] + 77)
    tbl = torch.randperm(n_pages, generator=gen, device=dev).to(torch.int32).reshape(batch, per_seq)
    pools = [(torch.empty((n_pages, kvh_l, page_size, D), dtype=torch.bfloat16, device=dev).normal_(generator=gen),
              torch.empty((n_pages, kvh_l, page_size, D), dtype=torch.bfloat16, device=dev).normal_(generator=gen))
             for _ in range(layers)]
    q = torch.empty((layers, batch, H_l * D), dtype=torch.bfloat16, device=dev).normal_(generator=gen)
    k = torch.empty((layers, batch, kvh_l * D), dtype=torch.bfloat16, device=dev).normal_(generator=gen)
    v = torch.empty((layers, batch, kvh_l * D), dtype=torch.bfloat16, device=dev).normal_(generator=gen)
    out = torch.empty((layers, batch, H_l * D), dtype=torch.bfloat16, device=dev)
    desc = ops.make_desc(DT_BF16, batch, H_l, kvh_l, 1, page_size, layout="head", is_neox=cfg["neox"])
    pages = ops.make_pages(tbl, page_size, kvh_l * page_size * D, n_pages)
    plan = ops.DecodePlan(desc, lens, True)
    plan.upload(dev)
    ws = torch.empty(max(plan.workspace_bytes, 16), dtype=torch.uint8, device=dev)

    def step():
        for l in range(layers):
            ops.gpu_attn_decode_planned_layer(desc, pages, plan, out[l], None, None, q[l], k[l], v[l], pools[l][0],
                                              pools[l][1], tab, None, ws, plan.workspace_bytes, stream=env.stream)
    for _ in range(3):
        step()
    ms_list = timed_repeats(env, step, 20, 3)
    ms_layer = statistics.median(ms_list) / (20 * layers)
    gbs = decode_bytes([L + 1 for L in lens], H_l, kvh_l) / (ms_layer * 1e-3) / 1e9
    return {"value": gbs, "unit": "GB/s", "ms_per_layer": ms_layer, "page_size": page_size, "layers": layers,
            "frac_of_hbm_peak": gbs / env.pk["hbm"], "entry_point": "gpu_attn_decode_planned_layer with a page table",
            "l2": "four layers' pools, 2.8 GB, cycled: inputs larger than L2"}


def other_configs_leg(env):
    """The remaining configurations on one GPU, one figure each: cfg1 (Llama-2-7B-shaped prefill,
    m = n = 256: launch-bound), cfg2 (Qwen2.5-1.5B-shaped one-sequence decode step: latency-bound,
    28 layers replayed from a graph), cfg3's decode phase (batch 8, MHA 40 heads, about 2176 cached
    positions: HBM-bound with one query row per KV head)."""
    torch, ops, dev, pk = env.torch, env.ops, env.dev, env.pk
    stream = env.stream
    res = {}

    def time_us(fn, reps, inner=1):
        for _ in range(3):
            fn()
        ms_list = timed_repeats(env, fn, reps, 3)
        return statistics.median(ms_list) * 1e3 / (reps * inner)

    # ---- cfg1
    m, H = 256, 32
    q = torch.randn((m, H * D), dtype=torch.float16, device=dev)
    k, v, o = torch.randn_like(q), torch.randn_like(q), torch.empty_like(q)
    us = time_us(lambda: ops.gpu_flash_attn_layer(o, q, k, v, m, m, 0, H, D, DT_FP16, stream=stream), 200)
    fl = prefill_flops(1, H, m, 0)
    res["cfg1_prefill"] = {"us": us, "tflops": fl / (us * 1e-6) / 1e12, "kernel": ops.gpu_attn_last_prefill_kernel(),
                           "note": "m = n = 256, 32 heads, fp16; launch-bound (0.54 GFLOP), inputs stay in L2"}
    # ---- cfg2
    c2 = CFG2
    layers, Hq, kvh, L, max_pos = c2["layers"], c2["n_heads"], c2["n_kv_heads"], 640, 776
    kc = [torch.randn((1, kvh, max_pos, D), dtype=torch.bfloat16, device=dev) for _ in range(layers)]
    vc = [torch.randn((1, kvh, max_pos, D), dtype=torch.bfloat16, device=dev) for _ in range(layers)]
    q2 = torch.randn((layers, 1, Hq * D), dtype=torch.bfloat16, device=dev)
    k2 = torch.randn((layers, 1, kvh * D), dtype=torch.bfloat16, device=dev)
    v2 = torch.randn_like(k2)
    o2 = torch.empty_like(q2)
    tab = env.table(max_pos, 1e6, DT_BF16)
    desc = ops.make_desc(DT_BF16, 1, Hq, kvh, 1, max_pos, layout="head", is_neox=True)
    plan = ops.DecodePlan(desc, [L], True)
    plan.upload(dev)
    ws = torch.empty(max(plan.workspace_bytes, 16), dtype=torch.uint8, device=dev)

    def step2(st):
        for l in range(layers):
            ops.gpu_attn_decode_planned_layer(desc, None, plan, o2[l], None, None, q2[l], k2[l], v2[l], kc[l], vc[l], tab,
                                              None, ws, plan.workspace_bytes, stream=st)
    step2(stream)
    torch.cuda.synchronize()
    cap = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(cap):
        graph.capture_begin()
        step2(cap)
        graph.capture_end()
    us_call = time_us(lambda: step2(stream), 20, layers)
    us_graph = time_us(graph.replay, 50, layers)
    res["cfg2_decode"] = {"us_per_layer_graph": us_graph, "us_per_layer_calls": us_call,
                          "bytes_per_layer": decode_bytes([L + 1], Hq, kvh),
                          "note": "batch 1, 12/2 heads, 640 cached positions (0.66 MB per layer): latency-bound; the "
                                  "28 layers' caches (18 MB) stay in L2"}
    # ---- cfg3 decode phase
    B, H3, L3, max3 = 8, 40, 2176, 2304
    nl = 4
    kc3 = [torch.randn((B, H3, max3, D), dtype=torch.float16, device=dev) for _ in range(nl)]
    vc3 = [torch.randn((B, H3, max3, D), dtype=torch.float16, device=dev) for _ in range(nl)]
    q3 = torch.randn((nl, B, H3 * D), dtype=torch.float16, device=dev)
    k3, v3, o3 = torch.randn_like(q3), torch.randn_like(q3), torch.empty_like(q3)
    t3 = env.table(max3, 1e4, DT_FP16)
    d3 = ops.make_desc(DT_FP16, B, H3, H3, 1, max3, layout="head", is_neox=False)
    plan3 = ops.DecodePlan(d3, [L3] * B, True)
    plan3.upload(dev)
    ws3 = torch.empty(max(plan3.workspace_bytes, 16), dtype=torch.uint8, device=dev)

    def step3():
        for l in range(nl):
            ops.gpu_attn_decode_planned_layer(d3, None, plan3, o3[l], None, None, q3[l], k3[l], v3[l], kc3[l], vc3[l], t3,
                                              None, ws3, plan3.workspace_bytes, stream=stream)
    us3 = time_us(step3, 20, nl)
    nb3 = decode_bytes([L3 + 1] * B, H3, H3)
    gbs3 = nb3 / (us3 * 1e-6) / 1e9
    res["cfg3_decode"] = {"us_per_layer": us3, "gbs": gbs3, "frac_of_hbm_peak": gbs3 / pk["hbm"], "bytes_per_layer": nb3,
                          "note": "batch 8, 40 heads MHA, 2176 cached positions, fp16; four layers' caches (2.9 GB) cycled"}
    return res


def split_kv_leg(env, layers=16, reps=20):
    """cfg5 decode: one sequence of 32768 cached positions, bf16 GQA 40/8, the cache sharded by
    POSITION over the ranks; every rank attends over its slice, the (O, LSE) partials are exchanged
    and merged (all ranks get the output).  Timed per layer for both exchanges: NCCL all-gather +
    merge kernel, and the one-kernel exchange over peer memory; both checked against the CPU checker
    on one layer and against each other bit for bit.  `layers` layers with caches of their own are
    cycled so that a rank's working set exceeds L2 at 8 GPUs (16 x 16.8 MB)."""
    from oracle import oracle as orc
    torch, dist, ops, dev, world, rank = env.torch, env.dist, env.ops, env.dev, env.world, env.rank
    from llm_simple_b200 import sharding
    c = CFG5
    H, kvh, L = c["n_heads"], c["n_kv_heads"], c["seq"]
    lo, hi = sharding.position_slices(L, world)[rank]
    n_loc = hi - lo
    cap = n_loc + 136
    gen = torch.Generator(device=dev)
    gen.manual_seed(20255 + rank)
    kc = [torch.empty((1, kvh, cap, D), dtype=torch.bfloat16, device=dev).normal_(generator=gen) for _ in range(layers)]
    vc = [torch.empty((1, kvh, cap, D), dtype=torch.bfloat16, device=dev).normal_(generator=gen) for _ in range(layers)]
    # q and the new token are the same on every rank (they come from the replicated projections)
    genq = torch.Generator(device=dev)
    genq.manual_seed(20255)
    q = torch.empty((layers, 1, H * D), dtype=torch.bfloat16, device=dev).normal_(generator=genq)
    k = torch.empty((layers, 1, kvh * D), dtype=torch.bfloat16, device=dev).normal_(generator=genq)
    v = torch.empty((layers, 1, kvh * D), dtype=torch.bfloat16, device=dev).normal_(generator=genq)
    out = torch.empty((layers, 1, H * D), dtype=torch.bfloat16, device=dev)
    tab = env.table(L + 8, c["theta"], DT_BF16)
    desc = ops.make_desc(DT_BF16, 1, H, kvh, 1, cap, layout="head", is_neox=c["neox"])
    desc.total_kv_len = n_loc + 1
    len_d = torch.tensor([n_loc], dtype=torch.int32, device=dev)
    pos_d = torch.tensor([L], dtype=torch.int32, device=dev)
    nbytes = decode_bytes([L + 1], H, kvh)
    res = {"workload": "cfg5 decode step, 32768 cached positions, position-sharded x%d" % world,
           "bytes_per_layer": nbytes, "layers_cycled": layers}

    def timed(step):
        for _ in range(3):
            step()
        ms_list = timed_repeats(env, step, reps, 3)
        us_calls = statistics.median(ms_list) * 1e3 / (reps * layers)
        # The steps are issued layer by layer from this script, several launches each: at these sizes the
        # interval above holds the script's launch rate.  Again with the launches queued behind a sleep
        # kernel (fewer steps, so that they fit the launch queue): the device time of the same work.
        short = max(2, reps // 4)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(short):
            step()
        host_ms = (time.perf_counter() - t0) * 1e3
        torch.cuda.synchronize()
        host = torch.tensor([host_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(host, op=dist.ReduceOp.MAX)
        ms_list = timed_repeats(env, step, short, 3, queue_behind_ms=1.5 * float(host.item()) + 1.0)
        us = statistics.median(ms_list) * 1e3 / (short * layers)
        return {"us_per_layer": us, "gbs": nbytes / (us * 1e-6) / 1e9, "frac_of_hbm_peak_all_ranks":
                nbytes / (us * 1e-6) / 1e9 / (env.pk["hbm"] * world), "us_per_layer_issued_call_by_call": us_calls,
                "timing": "launches queued behind a sleep kernel: device time; the call-by-call figure holds the "
                          "launch rate of this script"}

    def golden_layer0():
        """Rank 0: the whole cache of layer 0 from the ranks' slices, then the checker."""
        parts_k = [torch.empty((kvh, s[1] - s[0], D), dtype=torch.bfloat16, device=dev)
                   for s in sharding.position_slices(L, world)]
        parts_v = [torch.empty_like(p) for p in parts_k]
        if world > 1:
            # slices differ in length by at most one position: gather padded copies
            width = max(p.shape[1] for p in parts_k)
            pad_k = torch.zeros((kvh, width, D), dtype=torch.bfloat16, device=dev)
            pad_v = torch.zeros_like(pad_k)
            pad_k[:, :n_loc], pad_v[:, :n_loc] = kc[0][0, :, :n_loc], vc[0][0, :, :n_loc]
            gk = [torch.empty_like(pad_k) for _ in range(world)]
            gv = [torch.empty_like(pad_v) for _ in range(world)]
            dist.all_gather(gk, pad_k)
            dist.all_gather(gv, pad_v)
            parts_k = [gk[r][:, :parts_k[r].shape[1]] for r in range(world)]
            parts_v = [gv[r][:, :parts_v[r].shape[1]] for r in range(world)]
        else:
            parts_k, parts_v = [kc[0][0, :, :n_loc]], [vc[0][0, :, :n_loc]]
        if rank != 0:
            return None
        full_k = np.concatenate([bits(p) for p in parts_k], axis=1)
        full_v = np.concatenate([bits(p) for p in parts_v], axis=1)
        pad = np.zeros((kvh, 1, D), np.uint16)
        t = orc.init_freq_cis(D, L + 2, c["theta"], orc.DT_BFLOAT16)
        return oracle_decode_rows(orc, bits(q[0][0]), bits(k[0][0]), bits(v[0][0]), np.concatenate([full_k, pad], 1),
                                  np.concatenate([full_v, pad], 1), L, t, H, kvh, c["neox"], orc.DT_BFLOAT16)

    gold = golden_layer0()    # before any step: the steps append to the last rank's slice
    if world == 1:
        plan = ops.DecodePlan(desc, [n_loc], True)
        plan.upload(dev)
        ws = torch.empty(max(plan.workspace_bytes, 16), dtype=torch.uint8, device=dev)

        def step():
            for l in range(layers):
                ops.gpu_attn_decode_planned_layer(desc, None, plan, out[l], None, None, q[l], k[l], v[l], kc[l], vc[l],
                                                  tab, pos_d, ws, plan.workspace_bytes, stream=env.stream)
        res["single_gpu"] = timed(step)
        res["parity"] = parity_stats(orc, bits(out[0][0]), gold, orc.DT_BFLOAT16)
        return res
    ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, cap)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    outs = {}
    for mode in ("nccl", "peer"):
        dec = sharding.SplitKVDecoder(desc, DT_BF16, exchange=mode)

        def step():
            for l in range(layers):
                dec.step(out[l], q[l], k[l], v[l], kc[l], vc[l], tab, len_d, pos_d, n_loc, ws, ws_bytes)
        res[mode] = timed(step)
        outs[mode] = bits(out[0][0]).copy()
        dec.close()
    # the all-gather exchange behind the planned decode kernel (the slice length is known on the host)
    dec = sharding.SplitKVDecoder(desc, DT_BF16, exchange="nccl")
    state = {"plan": None, "ws": None}

    def step_planned():
        for l in range(layers):
            state["plan"], state["ws"] = dec.step_planned(out[l], q[l], k[l], v[l], kc[l], vc[l], tab, n_loc, pos_d,
                                                          state["plan"], state["ws"])
    res["nccl_planned_kernel"] = timed(step_planned)
    outs["nccl_planned_kernel"] = bits(out[0][0]).copy()
    dec.close()
    # and the peer-memory exchange behind the planned decode kernel
    dec = sharding.SplitKVDecoder(desc, DT_BF16, exchange="peer")
    state = {"plan": None, "ws": None}
    res["peer_planned_kernel"] = timed(step_planned)
    outs["peer_planned_kernel"] = bits(out[0][0]).copy()
    dec.close()
    res["kernel_status"] = ops.gpu_ops_kernel_status()
    same = bool(np.array_equal(outs["nccl"], outs["peer"]))
    flags = [None] * world
    dist.all_gather_object(flags, same)
    if rank == 0:
        res["parity"] = dict(parity_stats(orc, outs["nccl"], gold, orc.DT_BFLOAT16),
                             bit_identical_nccl_vs_peer=all(flags),
                             checked="layer 0: merged output of all ranks' position slices against the checker over "
                                     "the whole 32769-position cache; both exchanges")
        res["parity_planned_kernel"] = dict(parity_stats(orc, outs["nccl_planned_kernel"], gold, orc.DT_BFLOAT16),
                                            bit_identical_nccl_vs_peer=bool(np.array_equal(
                                                outs["nccl_planned_kernel"], outs["peer_planned_kernel"])))
    return res


def sampled_prefill_parity(env, orc, out, q_raw, k_raw, v_raw, table_np, H, kvh, neox, dt, samples):
    """Sampled (sequence, KV head, row block)s of a prefill output against the checker.
    out / q_raw [batch][S][H*D], k_raw / v_raw [batch][S][kvh*D] device tensors (raw, unrotated)."""
    recs = []
    g = H // kvh
    for b, kh, (lo, hi) in samples:
        q_r = orc.rope_single_layer(bits(q_raw[b, lo:hi]), table_np, lo, H, neox, dt)
        k_r = orc.rope_single_layer(bits(k_raw[b, :hi]), table_np, 0, kvh, neox, dt)
        qs = np.ascontiguousarray(q_r.reshape(hi - lo, H, D)[:, kh * g:(kh + 1) * g].reshape(hi - lo, -1))
        ks = np.ascontiguousarray(k_r.reshape(-1, kvh, D)[:, kh])
        vs = np.ascontiguousarray(bits(v_raw[b, :hi]).reshape(-1, kvh, D)[:, kh])
        gold = orc.attn(qs, ks, vs, hi - lo, hi, lo, g, 1, D, dt, orc.MODE_GOLDEN, threads=min(8, host_cores()))
        got = bits(out[b, lo:hi]).reshape(hi - lo, H, D)[:, kh * g:(kh + 1) * g].reshape(hi - lo, -1)
        recs.append(parity_stats(orc, got, gold, dt))
    return merge_parity(recs)


def long_prefill_leg(env, flush, check):
    """cfg5, one layer: a 32768-token prompt prefilled in chunks of 4096 (RoPE + append of the
    chunk, then causal attention of the chunk over everything cached so far), bf16, GQA 40/8,
    KV heads sharded over the ranks.  10.995 TFLOP per layer over all ranks."""
    torch, ops, dev, world = env.torch, env.ops, env.dev, env.world
    c = CFG5
    if c["n_kv_heads"] % world:
        return {"skipped": "KV heads do not divide"}
    kvh_l = c["n_kv_heads"] // world
    H_l = c["n_heads"] // world
    S, m = c["seq"], c["chunk"]
    max_pos = S + 128
    desc = ops.make_desc(DT_BF16, 1, H_l, kvh_l, m, max_pos, layout="head", is_neox=c["neox"])
    q = torch.randn((S // m, m, H_l * D), dtype=torch.bfloat16, device=dev)
    k = torch.randn((S // m, m, kvh_l * D), dtype=torch.bfloat16, device=dev)
    v = torch.randn_like(k)
    qe = torch.empty((m, H_l * D), dtype=torch.bfloat16, device=dev)
    o = torch.empty((S // m, m, H_l * D), dtype=torch.bfloat16, device=dev)
    kc = torch.zeros((1, kvh_l, max_pos, D), dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    tab = env.table(max_pos, c["theta"], DT_BF16)
    stream = env.stream
    kernels = set()

    def layer_pass():
        for ci in range(S // m):
            ops.gpu_rope_kv_append_layer(desc, qe, kc, vc, q[ci], k[ci], v[ci], tab, None, ci * m, m, stream=stream)
            ops.gpu_attn_prefill_layer(desc, o[ci], qe, kc, vc, m, ci * m, stream=stream)
            kernels.add(ops.gpu_attn_last_prefill_kernel())

    for _ in range(2):
        layer_pass()

    ms_list = timed_one_by_one(env, layer_pass, flush, 5)
    ms = statistics.median(ms_list)
    fl = sum(prefill_flops(1, c["n_heads"], m, ci * m) for ci in range(S // m))
    tf = fl / (ms * 1e-3) / 1e12
    res = {"workload": c["name"], "dtype": "bf16", "ms_per_layer": ms, "ms_spread": spread(ms_list), "tflops": tf,
           "flops_per_layer": fl, "per_rank_frac_of_tensor_peak": tf / world / env.pk["tensor"], "chunks": S // m,
           "tcgen05_kernel_served_every_call": kernels <= {2, 3}, "prefill_kernels": sorted(kernels),
           "note": "layer pass: RoPE + append and attention of all 8 chunks; 256 MB L2 flush before each pass"}
    if kernels != {2}:
        raise RuntimeError("the prefill leg was served by kernel(s) %s, not by the tcgen05 kernel" % sorted(kernels))
    if check and env.rank == 0:
        from oracle import oracle as orc
        t = orc.init_freq_cis(D, max_pos, c["theta"], orc.DT_BFLOAT16)
        qf, kf, vf = q.reshape(1, S, -1), k.reshape(1, S, -1), v.reshape(1, S, -1)
        samples = [(0, 0, (0, 48)), (0, kvh_l - 1, (4090, 4110)), (0, 0, (S - 24, S))]
        res["parity"] = dict(sampled_prefill_parity(env, orc, o.reshape(1, S, -1), qf, kf, vf, t, H_l, kvh_l, c["neox"],
                                                    orc.DT_BFLOAT16, samples),
                             checked="sampled (KV head, row block)s incl. a chunk boundary and the last rows")
    return res


def timed_one_by_one(env, fn, flush, n):
    """n single calls of fn, each behind an L2 flush, timed with CUDA events; max over ranks."""
    torch, dist = env.torch, env.dist
    out = []
    for _ in range(n):
        flush.zero_()
        env.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(env.stream)
        fn()
        e1.record(env.stream)
        env.barrier()
        ms = e0.elapsed_time(e1)
        if env.world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=env.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        out.append(ms)
    return out


def prefill_leg(env, check=True):
    """cfg3 prefill, one layer pass: fused RoPE + KV append, then causal attention."""
    torch, ops, dev, world = env.torch, env.ops, env.dev, env.world
    c = CFG3
    if c["n_heads"] % world:
        return {"skipped": "heads do not divide"}
    H_l = c["n_heads"] // world
    batch, S = c["batch"], c["seq"]
    max_pos = S + 256
    desc = ops.make_desc(DT_FP16, batch, H_l, H_l, S, max_pos, layout="head", is_neox=c["neox"])
    q = torch.randn((batch, S, H_l * D), dtype=torch.float16, device=dev)
    k = torch.randn_like(q)
    v = torch.randn_like(q)
    qe = torch.empty_like(q)
    o = torch.empty_like(q)
    kc = torch.zeros((batch, H_l, max_pos, D), dtype=torch.float16, device=dev)
    vc = torch.zeros_like(kc)
    tab = env.table(max_pos, c["theta"], DT_FP16)
    stream = env.stream
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2
    kernels = set()

    def layer_pass(attn_only=False):
        if not attn_only:
            ops.gpu_rope_kv_append_layer(desc, qe, kc, vc, q, k, v, tab, None, 0, S, stream=stream)
        ops.gpu_attn_prefill_layer(desc, o, qe, kc, vc, S, 0, stream=stream)
        kernels.add(ops.gpu_attn_last_prefill_kernel())

    res = {}
    fl = prefill_flops(batch, c["n_heads"], S, 0)
    for name, attn_only in (("layer_pass", False), ("attention_only", True)):
        for _ in range(3):
            layer_pass(attn_only)
        ms_list = timed_one_by_one(env, lambda: layer_pass(attn_only), flush, 10)
        ms = statistics.median(ms_list)
        res[name] = {"ms": ms, "tflops": fl / (ms * 1e-3) / 1e12, "ms_min": min(ms_list), "ms_max": max(ms_list)}
    if not kernels <= {2, 3}:
        raise RuntimeError("the prefill leg was served by kernel(s) %s, not by the tcgen05 kernels" % sorted(kernels))
    res["tcgen05_kernel_served_every_call"] = True
    res["prefill_kernels"] = sorted(kernels)       # 2: one CTA per 256 rows, 3: persistent
    if check and env.rank == 0:
        from oracle import oracle as orc
        t = orc.init_freq_cis(D, max_pos, c["theta"], orc.DT_FLOAT16)
        samples = [(0, 0, (0, 64)), (batch // 2, H_l // 2, (960, 1088)), (batch - 1, H_l - 1, (S - 64, S))]
        res["parity"] = dict(sampled_prefill_parity(env, orc, o, q, k, v, t, H_l, H_l, c["neox"], orc.DT_FLOAT16, samples),
                             checked="sampled (sequence, head, row block)s incl. the first and the last rows")
    # The RoPE + append pass on its own, fed from three tensors and from one fused q|k|v
    # projection row with a bias row (HBM-bound: every element read once, written once).
    row = 3 * H_l * D
    qkv = torch.randn((batch, S, row), dtype=torch.float16, device=dev)
    bias = torch.randn((row,), dtype=torch.float16, device=dev)
    pass_bytes = 2 * batch * S * row * 2
    for name in ("rope_append_pass", "qkv_fused_rope_append_pass"):
        def run():
            if name == "rope_append_pass":
                ops.gpu_rope_kv_append_layer(desc, qe, kc, vc, q, k, v, tab, None, 0, S, stream=stream)
            else:
                ops.gpu_qkv_rope_kv_append_layer(desc, qe, kc, vc, qkv, S * row, row, bias, tab, None, 0, S,
                                                 stream=stream)
        for _ in range(3):
            run()
        ms_list = timed_one_by_one(env, run, flush, 10)
        ms = statistics.median(ms_list)
        gbs = pass_bytes / (ms * 1e-3) / 1e9
        res[name] = {"ms": ms, "gbs": gbs, "bytes": pass_bytes, "frac_of_hbm_peak": gbs / env.pk["hbm"]}
    del qkv, bias
    res["cfg5_chunked_prefill"] = long_prefill_leg(env, flush, check)
    per_rank = res["attention_only"]["tflops"] / world
    res.update({"workload": c["name"], "dtype": "fp16", "flops_per_layer": fl, "l2": "256 MB flush between iterations",
                "roofline": {"bound": "tensor", "achieved": per_rank, "peak": env.pk["tensor"], "unit": "TFLOP/s",
                             "frac": per_rank / env.pk["tensor"], "peak_source": env.pk["source"],
                             "frac_of_nominal_2250": per_rank / 2250.0, "kernel": "attn_prefill_tc5_kernel"}})
    return res


def benchmark_mode_leg(env, which, n_in, n_out, check=True):
    """The reference's own measuring mode over the attention layers (Qwen2Model::Benchmark,
    src/qwen2_model.cpp:225-255, driven by scripts/benchmark_qwen2.5.sh): a prompt of n_in tokens is
    prefilled through every layer object, then one token per step is generated until n_in + n_out
    tokens, the cache growing every step; time to first token and ms per step are reported.  What the
    layers are fed stands in for the projections' outputs: seeded N(0,1) rows, a fresh one per step.
    cfg2: 28 layers, batch 1, 12/2 heads, bf16 (prompt 511, 256 steps); cfg3: 40 layers, batch 8,
    40 heads MHA, fp16 (prompt 2048, 256 steps).  The last step's output of the last layer is checked
    against the CPU checker fed with the same token rows."""
    torch, ops, lay, dev = env.torch, env.ops, env.lay, env.dev
    if which == "cfg2":
        c, kind, dt, tdt, batch = CFG2, lay.QWEN2, DT_BF16, torch.bfloat16, 1
        H, kvh, n_in, n_out = c["n_heads"], c["n_kv_heads"], n_in or 511, n_out or 256
    else:
        c, kind, dt, tdt, batch = CFG3, lay.LLAMA2, DT_FP16, torch.float16, CFG3["batch"]
        H, kvh, n_in, n_out = c["n_heads"], c["n_heads"], n_in or 2048, n_out or 256
    layers = c["layers"]
    max_seq = n_in + n_out + 8
    tab = env.table(max_seq, c["theta"], dt)
    objs = [lay.AttentionLayer(kind, H, kvh, max_seq, batch, dt, c["theta"], c["neox"], lay.HEAD_MAJOR,
                               shared_freq_cis=tab) for _ in range(layers)]
    step_state = lay.DecodeStep(batch, H, kvh, dt)
    for o in objs:
        o.set_shared_step(step_state)
    row = (H + 2 * kvh) * D
    gen = torch.Generator(device=dev)
    gen.manual_seed(20250 + (2 if which == "cfg2" else 3))
    # layer 0's rows are kept for the check; the other layers reuse one buffer per phase
    prompt = torch.empty((batch, n_in, row), dtype=tdt, device=dev).normal_(generator=gen)
    toks = torch.empty((n_out, batch, row), dtype=tdt, device=dev).normal_(generator=gen)
    out_p = torch.empty((batch, n_in, H * D), dtype=tdt, device=dev)
    out_d = torch.empty((layers, batch, H * D), dtype=tdt, device=dev)
    stream = env.stream
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    torch.cuda.synchronize()
    ops.gpu_ops_launch_count(True)
    t0 = time.perf_counter()
    e[0].record(stream)
    for o in objs:       # prefill: every layer consumes the same synthetic projection rows
        o.forward_fused(out_p, prompt, None, batch, n_in, 0, stream=stream)
    e[1].record(stream)
    for s in range(n_out):
        pos = n_in + s
        step_state.prepare([pos] * batch, True, stream=stream)
        for l, o in enumerate(objs):
            o.forward_fused(out_d[l], toks[s], None, batch, pos + 1, pos, stream=stream)
    e[2].record(stream)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ttft, dec = e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2])
    res = {"workload": "%s: %d layers, batch %d, %d/%d heads, prompt %d, %d generated tokens" %
                       (c["name"], layers, batch, H, kvh, n_in, n_out),
           "ttft_ms": ttft, "ms_per_step": dec / n_out, "us_per_layer_step": dec * 1e3 / (n_out * layers),
           "wall_ms_total": wall * 1e3, "gpu_launches": ops.gpu_ops_launch_count(True),
           "api": "gpu_attention_layer_forward_fused per layer (prefill, then one call per generated token); "
                  "gpu_decode_step_prepare once per step; launched call by call, no graph",
           "kernel_status": ops.gpu_ops_kernel_status()}
    if check:
        from oracle import oracle as orc
        t = orc.init_freq_cis(D, max_seq, c["theta"], dt)
        n = n_in + n_out
        b = batch - 1
        rows = np.concatenate([bits(prompt[b]), bits(toks[:, b])], axis=0)          # [n][row]
        q_raw, k_raw, v_raw = rows[:, :H * D], rows[:, H * D:(H + kvh) * D], rows[:, (H + kvh) * D:]
        k_r = orc.rope_single_layer(np.ascontiguousarray(k_raw), t, 0, kvh, c["neox"], dt)
        q_last = orc.rope_single_layer(np.ascontiguousarray(q_raw[n - 1:n]), t, n - 1, H, c["neox"], dt)
        gold = orc.attn(q_last, k_r, np.ascontiguousarray(v_raw), 1, n, n - 1, H // kvh, kvh, D, dt, orc.MODE_GOLDEN,
                        threads=min(8, host_cores()))[0]
        res["parity"] = dict(parity_stats(orc, bits(out_d[layers - 1][b]), gold, dt),
                             checked="last generated token, last layer, last sequence: attention over all %d cached "
                                     "positions against the checker fed with the same rows" % n)
    for o in objs:
        o.close()
    step_state.close()
    return res


if __name__ == "__main__":
    main()
