#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Headline workload ("cfg4"): one decode step of a Qwen2.5-14B-shaped model's
attention -- 48 layers, batch 64, 40 query heads on 8 KV heads, head_dim 128,
bf16, per-sequence cache lengths uniform in [1024, 4096] from a seed, RoPE theta
1e6 -- with the KV heads sharded over the N GPUs (no collective on the data
path).  One step = for every layer one fused launch group: rotate the new
token's Q/K, append K/V to the cache, split-KV grouped-query attention, merge.
The metric is algorithmic HBM GB/s (every K/V byte once + q/k/v in + o out), the
sum over all ranks divided by the slowest rank's device time.

Also reported in the same JSON line: the prefill leg ("cfg3": Llama-2-13B-shaped
causal prefill, batch 8 x 2048 tokens, 40 heads, fp16; algorithmic TFLOP/s), the
end-to-end figure with host buffers, the roofline of the dominant kernel, and the
CPU restatement of the reference's layer timed on the host cores.

Synthetic seeded N(0,1) tensors stand in for real activations (no checkpoints
here).  `--impl reference` times only the CPU restatement of the reference path
(the reference's own CPU layer needs Eigen/boost/spdlog, which are not
installed, so it cannot be built).
"""
import argparse
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

CFG4 = dict(name="cfg4 Qwen2.5-14B-shaped batched GQA decode", layers=48, batch=64, n_heads=40, n_kv_heads=8,
            len_lo=1024, len_hi=4096, theta=1e6, neox=True, seed=20254)
# dram__bytes_read.sum + dram__bytes_write.sum of attn_decode_kernel over its algorithmic bytes,
# from the ncu capture summarised in profiles/attn_decode_kernel_cfg4_1layer.md (700.9 / 693.68 MB)
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 700.9 / 693.68
CFG3 = dict(name="cfg3 Llama-2-13B-shaped causal prefill", batch=8, seq=2048, n_heads=40, theta=1e4, neox=False)
CFG5 = dict(name="cfg5 Qwen2.5-32B-shaped chunked causal prefill", batch=1, seq=32768, chunk=4096, n_heads=40,
            n_kv_heads=8, theta=1e6, neox=True)


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


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None
        self.t_begin = self.t_end = None

    def start(self):
        """Starts sampling (20 ms period).  Called before the warm-up, because the first sample
        arrives about 0.1 s after the sampler starts and a timed region can be shorter than that."""
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

        def collect(lo, hi):
            sm, mx, reasons = [], [], set()
            for t, r in self.rows:
                if t < lo or t > hi:
                    continue
                try:
                    sm.append(float(r[0]))
                    mx.append(float(r[1]))
                except (ValueError, IndexError):
                    continue
                for i, n in enumerate(names):
                    if len(r) > 3 + i and r[3 + i].lower().startswith("active"):
                        reasons.add(n)
            return sm, mx, reasons
        window = "timed region"
        sm, mx, reasons = collect(self.t_begin or 0.0, (self.t_end or 1e30) + 0.03)
        if not sm:
            # the region was shorter than the sampling period: the warm-up steps just before it ran
            # the same launches back to back, so their samples show the same load
            window = "warm-up and timed region (timed region shorter than the sampling period)"
            sm, mx, reasons = collect(0.0, (self.t_end or 1e30) + 0.03)
            sm, mx = sm[-5:], mx[-5:]
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "window": window}


# ----------------------------------------------------------------------------
# CPU restatement of the reference layer, timed (cpu_baseline / --impl reference)
# ----------------------------------------------------------------------------
def cpu_decode_layer(orc, cfg, lens, threads, rng):
    """One layer of the decode step on the host, the way the reference's layer
    runs it: rope(q), rope(k) -> append -> attention, strict rounding points,
    sequence by sequence.  Returns seconds."""
    H, kvh = cfg["n_heads"], cfg["n_kv_heads"]
    dt = orc.DT_BFLOAT16
    max_pos = max(lens) + 1
    table = orc.init_freq_cis(D, max_pos, cfg["theta"], dt)
    caches = []
    for L in lens:
        caches.append((orc.to_bits(rng.standard_normal((L + 1, kvh * D), dtype=np.float32), dt),
                       orc.to_bits(rng.standard_normal((L + 1, kvh * D), dtype=np.float32), dt)))
    q = orc.to_bits(rng.standard_normal((len(lens), H * D), dtype=np.float32), dt)
    k = orc.to_bits(rng.standard_normal((len(lens), kvh * D), dtype=np.float32), dt)
    v = orc.to_bits(rng.standard_normal((len(lens), kvh * D), dtype=np.float32), dt)
    t0 = time.perf_counter()
    for b, L in enumerate(lens):
        kc, vc = caches[b]
        q_r = orc.rope_single_layer(q[b:b + 1], table, L, H, cfg["neox"], dt)
        k_r = orc.rope_single_layer(k[b:b + 1], table, L, kvh, cfg["neox"], dt)
        orc.kv_append(kc, vc, k_r, v[b:b + 1], L, kvh, D)
        orc.attn(q_r, kc, vc, 1, L + 1, L, H // kvh, kvh, D, dt, orc.MODE_STRICT, threads=threads)
    return time.perf_counter() - t0


def cpu_baseline(cfg, lens, budget_s=12.0, seqs=None):
    from oracle import oracle as orc
    threads = orc.max_threads()
    rng = np.random.default_rng(7)
    sample = list(lens if seqs is None else lens[:seqs])
    nbytes = decode_bytes([L + 1 for L in sample], cfg["n_heads"], cfg["n_kv_heads"])
    times = []
    t_start = time.perf_counter()
    while not times or (time.perf_counter() - t_start < budget_s and len(times) < 5):
        times.append(cpu_decode_layer(orc, cfg, sample, threads, rng))
    best = min(times)
    return {"value": nbytes / best / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": "1 layer x %d of %d sequences, %d repeats, best; strict rounding points, OpenMP over KV heads"
                      % (len(sample), len(lens), len(times)),
            "seconds": best}


def run_reference_arm(args, cfg, lens):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc
    threads = orc.max_threads()
    rng = np.random.default_rng(7)
    seqs = len(lens)  # bounded sample: one of the layers, the whole batch
    sample = lens[:seqs]
    nbytes = decode_bytes([L + 1 for L in sample], cfg["n_heads"], cfg["n_kv_heads"])
    for _ in range(args.warmup):
        cpu_decode_layer(orc, cfg, sample, threads, rng)
    t = 0.0
    for _ in range(args.steps):
        t += cpu_decode_layer(orc, cfg, sample, threads, rng)
    value = nbytes * args.steps / t / 1e9
    line = {
        "impl": "reference", "metric": "attn decode HBM GB/s per layer", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg["name"], "note": "CPU restatement of the reference layer on the host cores"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": "each step = 1 of %d layers, all %d sequences" % (cfg["layers"], seqs)},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (profiling on a small case)")
    ap.add_argument("--batch", type=int, default=None, help="override the batch (profiling on a small case)")
    ap.add_argument("--no-extras", action="store_true", help="skip prefill leg, e2e and CPU baseline")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="on ONE GPU, run rank 0's shard of an N-way KV-head split (sizing a multi-GPU shard)")
    ap.add_argument("--early-prefetch", type=int, default=1,
                    help="1: the decode kernel requests its first K/V tiles before the preceding kernels of the "
                         "stream have finished (legal here: consecutive launches read different layers' caches)")
    ap.add_argument("--graph", type=int, default=1,
                    help="1: replay the step's launches from a CUDA graph (default), 0: launch them one by one")
    ap.add_argument("--leg", default="all", choices=["all", "prefill"],
                    help="prefill: run only the prefill leg (small, for profiling) and print its object")
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
    from llm_simple_b200 import ops
    from oracle import oracle as orc  # table builder + cpu_baseline leg only

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        # keep stdout for the one JSON line: NCCL prints its version banner there at VERSION level
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ops.lib()
    pk = peaks()

    def barrier0():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.leg == "prefill":
        res = prefill_leg(torch, ops, orc, world, torch.device("cuda", local_rank), barrier0, pk)
        if rank == 0:
            print(json.dumps({"prefill": res}))
        if world > 1:
            dist.destroy_process_group()
        return

    H, kvh = cfg["n_heads"], cfg["n_kv_heads"]
    if kvh % world:
        raise SystemExit("KV heads (%d) do not divide over %d ranks" % (kvh, world))
    split = world * max(args.shard_of, 1)
    if kvh % split:
        raise SystemExit("KV heads (%d) do not divide into %d shards" % (kvh, split))
    kvh_l, H_l = kvh // split, H // split
    layers, batch = cfg["layers"], cfg["batch"]
    max_pos = cfg["len_hi"] + 8
    max_kv = max(lens) + 1
    dev = torch.device("cuda", local_rank)

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
    table = torch.from_numpy(orc.init_freq_cis(D, max_pos, cfg["theta"], orc.DT_BFLOAT16)).to(dev)
    lens_d = torch.tensor(lens, dtype=torch.int32, device=dev)
    desc = ops.make_desc(DT_BF16, batch, H_l, kvh_l, 1, max_pos, layout="head", is_neox=cfg["neox"])
    desc.total_kv_len = sum(L + 1 for L in lens)   # scheduling hint: the host knows the lengths
    ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, max_kv)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream()

    # consecutive launches work on different layers' caches and the lengths are fixed for the step
    ops.gpu_attn_set_decode_early_prefetch(args.early_prefetch)

    def step():
        for l in range(layers):
            ops.gpu_attn_decode_layer(desc, out[l], None, None, q_in[l], k_in[l], v_in[l], k_cache[l], v_cache[l],
                                      table, lens_d, None, True, max_kv, ws, ws_bytes, stream=stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    launch_step = step
    graph = None
    if args.graph:
        # A decode step is a fixed sequence of launches: capture it once and replay it, as a
        # serving loop would; this removes the per-call host cost (a few per cent of the step).
        step()
        barrier()
        ops.gpu_ops_launch_count(True)
        try:
            cap = torch.cuda.Stream(device=dev)
            graph = torch.cuda.CUDAGraph()
            stream = cap
            with torch.cuda.stream(cap):
                graph.capture_begin()
                launch_step()
                graph.capture_end()
        except Exception as e:  # capture unavailable: launch call by call
            sys.stderr.write("cuda graph capture failed (%s); launching call by call\n" % e)
            graph = None
        launches_per_step = ops.gpu_ops_launch_count(True)
        stream = torch.cuda.current_stream()
        if graph is not None:
            def step():
                graph.replay()

    sampler = ClockSampler(local_rank).start()
    t_warm = time.monotonic()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    # extra untimed steps until the clock sampler has seen this load for a quarter of a second
    # (the same count on every rank: the decision is rank 0's)
    while True:
        more = torch.tensor([1 if time.monotonic() - t_warm < 0.25 else 0], device=dev)
        if world > 1:
            dist.broadcast(more, 0)
        if not int(more.item()):
            break
        step()
        barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ops.gpu_ops_launch_count(True)
    with sampler as clk:
        barrier()
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        barrier()
    launches = ops.gpu_ops_launch_count(True)
    if graph is not None:
        launches = launches_per_step * args.steps   # kernels replayed from the graph
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        lt = torch.tensor([launches], dtype=torch.int64, device=dev)
        dist.all_reduce(lt)
        launches = int(lt.item())
    ms_per_step = ms / args.steps
    so = max(args.shard_of, 1)
    bytes_layer_all = decode_bytes([L + 1 for L in lens], H // so, kvh // so)  # all ranks, one layer
    bytes_layer_rank = decode_bytes([L + 1 for L in lens], H_l, kvh_l)    # this rank, one layer
    value = bytes_layer_all * layers / (ms_per_step * 1e-3) / 1e9
    layer_ms = ms_per_step / layers
    achieved = bytes_layer_rank / (layer_ms * 1e-3) / 1e9
    # DRAM bytes per launch: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this
    # workload's own one-layer launch at N = 1 (700.9 MB against 693.68 MB algorithmic, profiles/);
    # a shard of the same launch is scaled by the bytes it processes (traffic is all K/V streaming).
    traffic = NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * bytes_layer_rank
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s",
                "frac": achieved / pk["hbm"], "traffic": traffic,
                "traffic_source": "ncu capture of the one-layer launch, scaled by algorithmic bytes",
                "peak_source": pk["source"],
                "kernel": "attn_decode_kernel (+ attn_merge_kernel, one launch pair per layer)",
                "launch_ms": layer_ms, "algorithmic_bytes_per_launch": bytes_layer_rank,
                "frac_of_nominal_8TBs": achieved / 8000.0}

    line = {
        "metric": "attn decode HBM GB/s per layer", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg["name"], "layers": layers, "batch": batch, "n_heads": H, "n_kv_heads": kvh,
                   "head_dim": D, "kv_len": "uniform[%d,%d] seed %d" % (cfg["len_lo"], cfg["len_hi"], cfg["seed"]),
                   "sharding": "kv-head x%d" % world if args.shard_of <= 1 else
                               "rank 0's shard of a kv-head x%d split, alone on one GPU" % split,
                   "launch": "cuda graph of the step's %d launches" % launches_per_step if graph is not None
                             else "one call per layer",
                   "early_kv_prefetch": bool(args.early_prefetch),
                   "cache_layout": "head-major",
                   "l2": "inputs larger than L2 (%.0f MB per layer, %.1f GB per step per rank)"
                         % (bytes_layer_rank / 1e6, bytes_layer_rank * layers / 1e9)},
        "roofline": roofline, "clocks": clk.summary(), "gpu_launches": launches,
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
        leg("e2e", e2e_leg, torch, ops, args, cfg, desc, lens, lens_d, k_cache, v_cache, table, ws, ws_bytes, max_kv, H_l,
            kvh_l, world, dev, barrier, bytes_layer_all)
        leg("prefill", prefill_leg, torch, ops, orc, world, dev, barrier, pk)
        leg("cfg5_split_kv_decode", split_kv_leg, torch, ops, orc, world, rank, dev, barrier, pk)
        if world == 1:
            leg("other_configs", other_configs_leg, torch, ops, orc, dev, pk)
            leg("paged_decode", paged_leg, torch, ops, cfg, lens, lens_d, table, ws, ws_bytes, max_kv, H_l, kvh_l, dev, pk)
        if rank == 0 and world == 1:
            leg("cpu_baseline", cpu_baseline, cfg, lens)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def e2e_leg(torch, ops, args, cfg, desc, lens, lens_d, k_cache, v_cache, table, ws, ws_bytes, max_kv, H_l, kvh_l,
            world, dev, barrier, bytes_layer_all):
    """The same step through the host layer with HOST buffers: one attention-layer
    object per layer (llm_simple_b200.layer.AttentionLayer, the mirror of the
    reference's Qwen2 layer class) adopts that layer's KV cache; every call takes
    the new token's packed q/k/v row from pinned host memory and returns the
    attention output to pinned host memory, the copies enqueued around the kernels
    inside the timed region.  Layers alternate between two streams so that one
    layer's copies overlap the other's kernel.  The KV cache is device state."""
    import torch.distributed as dist
    from llm_simple_b200 import layer as lay
    layers, batch = cfg["layers"], cfg["batch"]
    qkv_w = (H_l + 2 * kvh_l) * D
    h_in = torch.empty((layers, batch, qkv_w), dtype=torch.bfloat16).normal_().pin_memory()
    h_out = torch.empty((layers, batch, H_l * D), dtype=torch.bfloat16).pin_memory()
    max_pos = cfg["len_hi"] + 8
    objs = []
    for l in range(layers):
        o = lay.AttentionLayer(lay.QWEN2, H_l, kvh_l, max_pos, batch, DT_BF16, cfg["theta"], cfg["neox"],
                               lay.HEAD_MAJOR, shared_freq_cis=table, k_cache=k_cache[l], v_cache=v_cache[l])
        o.set_shared_lens(lens_d, max_kv, sum(L + 1 for L in lens))   # once per step by the model, not per layer
        objs.append(o)
    cur = torch.cuda.current_stream()
    side = [torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)]

    def step():
        for l in range(layers):
            objs[l].forward_host(h_out[l], h_in[l], batch, 1, 0, stream=side[l & 1])

    def fork(ev):
        ev.record(cur)
        for st in side:
            st.wait_event(ev)

    def join(ev):
        for st in side:
            e = torch.cuda.Event()
            e.record(st)
            cur.wait_event(e)
        ev.record(cur)

    steps = max(3, args.steps // 2)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fork(ev0)
    for _ in range(3):
        step()
    join(ev1)
    barrier()
    ops.gpu_ops_launch_count(True)
    t0 = time.perf_counter()
    fork(ev0)
    for _ in range(steps):
        step()
    join(ev1)
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    ms = max(ev0.elapsed_time(ev1), 0.0)
    if world > 1:
        t = torch.tensor([ms, wall_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, wall_ms = float(t[0].item()), float(t[1].item())
    per_step = ms / steps
    res = {"value": bytes_layer_all * layers / (per_step * 1e-3) / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": int(layers * batch * qkv_w * 2 * world),
           "d2h_bytes_per_step": int(layers * batch * H_l * D * 2 * world), "ms_per_step": per_step,
           "wall_ms_per_step": wall_ms / steps, "steps": steps,
           "api": "gpu_attention_layer_forward_host per layer (C ABI of the host layer): pinned host q/k/v row in, "
                  "attention output back to pinned host memory, two streams"}
    for o in objs:
        o.close()
    return res


def paged_leg(torch, ops, cfg, lens, lens_d, table, ws, ws_bytes, max_kv, H_l, kvh_l, dev, pk, layers=4, page_size=256):
    """The decode step over a PAGED cache (pages of 256 positions handed out in random
    order), on `layers` layers with caches of their own: the same kernel, the page table
    looked up once per tile of 64 positions."""
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
    desc.total_kv_len = sum(L + 1 for L in lens)
    pages = ops.make_pages(tbl, page_size, kvh_l * page_size * D, n_pages)
    stream = torch.cuda.current_stream()

    def step():
        for l in range(layers):
            ops.gpu_attn_decode_paged_layer(desc, pages, out[l], q[l], k[l], v[l], pools[l][0], pools[l][1], table,
                                            lens_d, True, max_kv, ws, ws_bytes, stream=stream)
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 20
    e0.record(stream)
    for _ in range(reps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    ms_layer = e0.elapsed_time(e1) / (reps * layers)
    gbs = decode_bytes([L + 1 for L in lens], H_l, kvh_l) / (ms_layer * 1e-3) / 1e9
    return {"value": gbs, "unit": "GB/s", "ms_per_layer": ms_layer, "page_size": page_size, "layers": layers,
            "frac_of_hbm_peak": gbs / pk["hbm"],
            "l2": "four layers' pools, 2.8 GB, cycled: inputs larger than L2"}


def other_configs_leg(torch, ops, orc, dev, pk):
    """The remaining configurations on one GPU, one figure each: cfg1 (Llama-2-7B-shaped prefill,
    m = n = 256: launch-bound), cfg2 (Qwen2.5-1.5B-shaped one-sequence decode step: latency-bound,
    28 layers replayed from a graph), cfg3's decode phase (batch 8, MHA 40 heads, about 2176 cached
    positions: HBM-bound with one query row per KV head)."""
    stream = torch.cuda.current_stream()
    res = {}

    def time_us(fn, reps, inner=1):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (reps * inner)

    # ---- cfg1
    m, H = 256, 32
    q = torch.randn((m, H * D), dtype=torch.float16, device=dev)
    k, v, o = torch.randn_like(q), torch.randn_like(q), torch.empty_like(q)
    us = time_us(lambda: ops.gpu_flash_attn_layer(o, q, k, v, m, m, 0, H, D, DT_FP16, stream=stream), 200)
    fl = prefill_flops(1, H, m, 0)
    res["cfg1_prefill"] = {"us": us, "tflops": fl / (us * 1e-6) / 1e12, "note": "m = n = 256, 32 heads, fp16; launch-bound "
                           "(0.54 GFLOP), inputs stay in L2"}
    # ---- cfg2
    layers, Hq, kvh, L, max_pos = 28, 12, 2, 640, 776
    kc = [torch.randn((1, kvh, max_pos, D), dtype=torch.bfloat16, device=dev) for _ in range(layers)]
    vc = [torch.randn((1, kvh, max_pos, D), dtype=torch.bfloat16, device=dev) for _ in range(layers)]
    q2 = torch.randn((layers, 1, Hq * D), dtype=torch.bfloat16, device=dev)
    k2 = torch.randn((layers, 1, kvh * D), dtype=torch.bfloat16, device=dev)
    v2 = torch.randn_like(k2)
    o2 = torch.empty_like(q2)
    table = torch.from_numpy(orc.init_freq_cis(D, max_pos, 1e6, orc.DT_BFLOAT16)).to(dev)
    desc = ops.make_desc(DT_BF16, 1, Hq, kvh, 1, max_pos, layout="head", is_neox=True)
    desc.total_kv_len = L + 1
    wsb = ops.gpu_attn_decode_workspace_bytes(desc, L + 1)
    ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)
    len_d = torch.tensor([L], dtype=torch.int32, device=dev)

    def step2(st):
        for l in range(layers):
            ops.gpu_attn_decode_layer(desc, o2[l], None, None, q2[l], k2[l], v2[l], kc[l], vc[l], table, len_d, None, True,
                                      L + 1, ws, wsb, stream=st)
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
    t3 = torch.from_numpy(orc.init_freq_cis(D, max3, 1e4, orc.DT_FLOAT16)).to(dev)
    d3 = ops.make_desc(DT_FP16, B, H3, H3, 1, max3, layout="head", is_neox=False)
    d3.total_kv_len = B * (L3 + 1)
    wsb3 = ops.gpu_attn_decode_workspace_bytes(d3, L3 + 1)
    ws3 = torch.empty(max(wsb3, 16), dtype=torch.uint8, device=dev)
    len3 = torch.full((B,), L3, dtype=torch.int32, device=dev)

    def step3():
        for l in range(nl):
            ops.gpu_attn_decode_layer(d3, o3[l], None, None, q3[l], k3[l], v3[l], kc3[l], vc3[l], t3, len3, None, True,
                                      L3 + 1, ws3, wsb3, stream=stream)
    us3 = time_us(step3, 20, nl)
    nb3 = decode_bytes([L3 + 1] * B, H3, H3)
    gbs3 = nb3 / (us3 * 1e-6) / 1e9
    res["cfg3_decode"] = {"us_per_layer": us3, "gbs": gbs3, "frac_of_hbm_peak": gbs3 / pk["hbm"], "bytes_per_layer": nb3,
                          "note": "batch 8, 40 heads MHA, 2176 cached positions, fp16; four layers' caches (2.9 GB) cycled"}
    return res


def split_kv_leg(torch, ops, orc, world, rank, dev, barrier, pk, layers=16, reps=20):
    """cfg5 decode: one sequence of 32768 cached positions, bf16 GQA 40/8, the cache sharded by
    POSITION over the ranks; every rank attends over its slice, the (O, LSE) partials are exchanged
    and merged (all ranks get the output).  Timed per layer for both exchanges: NCCL all-gather +
    merge kernel, and the one-kernel exchange over peer memory.  `layers` layers with caches of
    their own are cycled so that a rank's working set exceeds L2 at 8 GPUs (16 x 16.8 MB)."""
    import torch.distributed as dist
    from llm_simple_b200 import sharding
    c = CFG5
    H, kvh, L = c["n_heads"], c["n_kv_heads"], c["seq"]
    lo, hi = sharding.position_slices(L, world)[rank]
    n_loc = hi - lo
    cap = n_loc + 136
    tail = rank == world - 1
    gen = torch.Generator(device=dev)
    gen.manual_seed(20255 + rank)
    kc = [torch.empty((1, kvh, cap, D), dtype=torch.bfloat16, device=dev).normal_(generator=gen) for _ in range(layers)]
    vc = [torch.empty((1, kvh, cap, D), dtype=torch.bfloat16, device=dev).normal_(generator=gen) for _ in range(layers)]
    q = torch.empty((layers, 1, H * D), dtype=torch.bfloat16, device=dev).normal_(generator=gen)
    k = torch.empty((layers, 1, kvh * D), dtype=torch.bfloat16, device=dev).normal_(generator=gen)
    v = torch.empty((layers, 1, kvh * D), dtype=torch.bfloat16, device=dev).normal_(generator=gen)
    out = torch.empty((layers, 1, H * D), dtype=torch.bfloat16, device=dev)
    table = torch.from_numpy(orc.init_freq_cis(D, L + 8, c["theta"], orc.DT_BFLOAT16)).to(dev)
    desc = ops.make_desc(DT_BF16, 1, H, kvh, 1, cap, layout="head", is_neox=c["neox"])
    desc.total_kv_len = n_loc + 1
    ws_bytes = ops.gpu_attn_decode_workspace_bytes(desc, cap)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    len_d = torch.tensor([n_loc], dtype=torch.int32, device=dev)
    pos_d = torch.tensor([L], dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream()
    nbytes = decode_bytes([L + 1], H, kvh)
    res = {"workload": "cfg5 decode step, 32768 cached positions, position-sharded x%d" % world,
           "bytes_per_layer": nbytes, "layers_cycled": layers}

    def timed(step):
        for _ in range(3):
            step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            step()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        us = ms * 1e3 / (reps * layers)
        return {"us_per_layer": us, "gbs": nbytes / (us * 1e-6) / 1e9}

    if world == 1:
        def step():
            for l in range(layers):
                ops.gpu_attn_decode_layer(desc, out[l], None, None, q[l], k[l], v[l], kc[l], vc[l], table, len_d, pos_d,
                                          True, n_loc + 1, ws, ws_bytes, stream=stream)
        res["single_gpu"] = timed(step)
        return res
    for mode in ("nccl", "peer"):
        dec = sharding.SplitKVDecoder(desc, DT_BF16, exchange=mode)

        def step():
            for l in range(layers):
                dec.step(out[l], q[l], k[l], v[l], kc[l], vc[l], table, len_d, pos_d, n_loc, ws, ws_bytes)
        res[mode] = timed(step)
        dec.close()
    res["kernel_status"] = ops.gpu_ops_kernel_status()
    return res


def long_prefill_leg(torch, ops, orc, world, dev, barrier, pk, flush):
    """cfg5, one layer: a 32768-token prompt prefilled in chunks of 4096 (RoPE + append of the
    chunk, then causal attention of the chunk over everything cached so far), bf16, GQA 40/8,
    KV heads sharded over the ranks.  10.995 TFLOP per layer over all ranks."""
    import torch.distributed as dist
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
    o = torch.empty_like(qe)
    kc = torch.zeros((1, kvh_l, max_pos, D), dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    table = torch.from_numpy(orc.init_freq_cis(D, max_pos, c["theta"], orc.DT_BFLOAT16)).to(dev)
    stream = torch.cuda.current_stream()

    def layer_pass():
        for ci in range(S // m):
            ops.gpu_rope_kv_append_layer(desc, qe, kc, vc, q[ci], k[ci], v[ci], table, None, ci * m, m, stream=stream)
            ops.gpu_attn_prefill_layer(desc, o, qe, kc, vc, m, ci * m, stream=stream)

    for _ in range(2):
        layer_pass()
    times = []
    for _ in range(5):
        flush.zero_()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        layer_pass()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        times.append(ms)
    ms = statistics.median(times)
    fl = sum(prefill_flops(1, c["n_heads"], m, ci * m) for ci in range(S // m))
    tf = fl / (ms * 1e-3) / 1e12
    return {"workload": c["name"], "dtype": "bf16", "ms_per_layer": ms, "tflops": tf, "flops_per_layer": fl,
            "per_rank_frac_of_tensor_peak": tf / world / pk["tensor"], "chunks": S // m,
            "note": "layer pass: RoPE + append and attention of all 8 chunks; 256 MB L2 flush before each pass"}


def prefill_leg(torch, ops, orc, world, dev, barrier, pk):
    """cfg3 prefill, one layer pass: fused RoPE + KV append, then causal attention."""
    import torch.distributed as dist
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
    table = torch.from_numpy(orc.init_freq_cis(D, max_pos, c["theta"], orc.DT_FLOAT16)).to(dev)
    stream = torch.cuda.current_stream()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2

    def layer_pass(attn_only=False):
        if not attn_only:
            ops.gpu_rope_kv_append_layer(desc, qe, kc, vc, q, k, v, table, None, 0, S, stream=stream)
        ops.gpu_attn_prefill_layer(desc, o, qe, kc, vc, S, 0, stream=stream)

    res = {}
    for name, attn_only in (("layer_pass", False), ("attention_only", True)):
        for _ in range(3):
            layer_pass(attn_only)
        times = []
        for _ in range(10):
            flush.zero_()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            layer_pass(attn_only)
            e1.record(stream)
            barrier()
            ms = e0.elapsed_time(e1)
            if world > 1:
                t = torch.tensor([ms], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            times.append(ms)
        ms = statistics.median(times)
        fl = prefill_flops(batch, c["n_heads"], S, 0)
        res[name] = {"ms": ms, "tflops": fl / (ms * 1e-3) / 1e12, "ms_min": min(times)}
    # The RoPE + append pass on its own, fed from three tensors and from one fused q|k|v
    # projection row with a bias row (HBM-bound: every element read once, written once).
    row = 3 * H_l * D
    qkv = torch.randn((batch, S, row), dtype=torch.float16, device=dev)
    bias = torch.randn((row,), dtype=torch.float16, device=dev)
    pass_bytes = 2 * batch * S * row * 2
    for name in ("rope_append_pass", "qkv_fused_rope_append_pass"):
        def run():
            if name == "rope_append_pass":
                ops.gpu_rope_kv_append_layer(desc, qe, kc, vc, q, k, v, table, None, 0, S, stream=stream)
            else:
                ops.gpu_qkv_rope_kv_append_layer(desc, qe, kc, vc, qkv, S * row, row, bias, table, None, 0, S,
                                                 stream=stream)
        for _ in range(3):
            run()
        times = []
        for _ in range(10):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            run()
            e1.record(stream)
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        gbs = pass_bytes / (ms * 1e-3) / 1e9
        res[name] = {"ms": ms, "gbs": gbs, "bytes": pass_bytes, "frac_of_hbm_peak": gbs / pk["hbm"]}
    res["cfg5_chunked_prefill"] = long_prefill_leg(torch, ops, orc, world, dev, barrier, pk, flush)
    per_rank = res["attention_only"]["tflops"] / world
    res.update({"workload": c["name"], "dtype": "fp16", "flops_per_layer": prefill_flops(batch, c["n_heads"], S, 0),
                "l2": "256 MB flush between iterations",
                "roofline": {"bound": "tensor", "achieved": per_rank, "peak": pk["tensor"], "unit": "TFLOP/s",
                             "frac": per_rank / pk["tensor"], "peak_source": pk["source"],
                             "frac_of_nominal_2250": per_rank / 2250.0, "kernel": "prefill attention kernel"}})
    return res


if __name__ == "__main__":
    main()
