"""Benchmark of the quantized-KV decode attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1|c3|c4|c5] [--only]

One step = one decode-attention pass of one layer over a batch of synthetic sequences whose
compressed KV cache is resident in HBM (a ragged batch of 64 sequences with 512-8192 MXFP4 keys
by default: 32 query heads, 8 kv heads, head dim 128, bf16 queries). The metric is the achieved HBM
bandwidth on the algorithmic bytes of the step (packed code and scale bytes of every visible K and
V row, plus queries and outputs), with tokens/s beside it. With N > 1 every rank holds its own
batch (weak scaling, no data-path collective: nothing in a rank's step depends on another rank).
Where one problem is split over the ranks (c4, c5) the outputs of all ranks are assembled on every
rank inside the step, by the attention's own epilogue; a short line times the headline workload
with that exchange too.

The last line printed is the headline workload. Before it come short lines for the other
configurations of the benchmark (unless --only): single FP8 decode (c1), prefill with cache append
(c3, one GPU), TurboQuant decode sharded by kv head (c4) and the MXFP8 decode sharded by batch
(c5), the last two as strong scaling over the N ranks.

`--impl reference` times the reference's CPU path for the same step (dequantize the cached rows to
the cache dtype, then unfused softmax(Q K^T) V; candle-nn/src/turbo_quant.rs:947-991,
candle-nn/src/flash_attn.rs:930-1000) through the C restatement in oracle/, on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PAYLOAD = {0: 68, 2: 68, 3: 76, 4: 132, 5: 132}  # algorithmic bytes of one packed row at head dim 128 (codes + scales)
METRIC = "quantized_kv_decode_attention_hbm_bandwidth"

WORKLOADS = {
    # b, hq, hkv: the whole problem; `shard` says how N ranks split it (strong scaling), None = every rank its own copy
    "c2": dict(b=64, hq=32, hkv=8, d=128, fmt="mxfp4", mode=2, qdt="bf16", rot="none", lens="uniform512-8192", shard=None,
               desc="ragged MXFP4 decode, B=64, lengths uniform in [512, 8192]"),
    "c1": dict(b=1, hq=32, hkv=8, d=128, fmt="fp8", mode=5, qdt="f16", rot="none", lens=2048, shard=None,
               desc="single FP8 decode, 2048 keys"),
    "c4": dict(b=32, hq=64, hkv=8, d=128, fmt="turbo4", mode=0, qdt="bf16", rot="hadamard", lens=32768, shard="kv_head",
               desc="TurboQuant-4 decode, B=32 x 32768 keys, Hq=64, Hkv=8, kv heads split over the GPUs"),
    "c5": dict(b=128, hq=32, hkv=8, d=128, fmt="mxfp8", mode=4, qdt="f16", rot="none", lens=16384, shard="batch",
               desc="MXFP8 decode, B=128 x 16384 keys, one layer, batch split over the GPUs"),
}
# on one GPU c4 is timed on the share that one of eight GPUs holds (one kv head): the configuration is defined sharded
C4_SINGLE = dict(hq=8, hkv=1, desc="TurboQuant-4 decode, one kv head (of 8) of B=32 x 32768 keys: the share of one of 8 GPUs")

GOLDEN = 0x9E3779B97F4A7C15
MASK64 = (1 << 64) - 1


def splitmix64(seed, n):
    """The first n outputs of SplitMix64(seed), the generator the reference seeds its test data with
    (candle-core/src/accel/turbo.rs:148-160)."""
    out = np.empty(n, dtype=np.uint64)
    state = seed & MASK64
    for i in range(n):
        state = (state + GOLDEN) & MASK64
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        out[i] = z ^ (z >> 31)
    return out


def seq_lens(w, rank=0):
    if w["lens"] == "uniform512-8192":
        # every rank gets the same multiset of lengths (weak scaling: the work per GPU is fixed), in its own order
        lens = (512 + splitmix64(2002, w["b"]) % np.uint64(7681)).astype(np.int32)
        return np.roll(lens, 7 * rank)
    return np.full(w["b"], w["lens"], np.int32)


def algorithmic_bytes(w, lens):
    qo = w["b"] * w["hq"] * w["d"] * 2 * 2  # queries read + outputs written, 16-bit
    return int(lens.astype(np.int64).sum()) * w["hkv"] * 2 * PAYLOAD[w["mode"]] + qo


def shard_of(w, world):
    """The part of workload `w` that one of `world` ranks holds (all ranks alike), or None when it does not divide."""
    s = dict(w)
    if w["shard"] == "batch":
        if w["b"] % world:
            return None
        s["b"] = w["b"] // world
    elif w["shard"] == "kv_head":
        if w["hkv"] % world:
            return None
        s["hkv"] = w["hkv"] // world
        s["hq"] = w["hq"] // world
    return s


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        mhz = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


# ---------------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU path, timed on the host cores
# ---------------------------------------------------------------------------------------------------------------------

class CpuSample:
    """A bounded sample of a decode workload for the CPU arm: `nseq` sequences, inputs generated and quantized once
    (outside any timed region); a pass runs the reference's CPU path for each of them in C (dequantize the cached rows
    to the cache dtype, unfused attention of the query token)."""

    def __init__(self, w, lens, nseq):
        from oracle import oracle as O
        self.O = O
        if os.environ.get("OMP_NUM_THREADS") == "1" and "LOCAL_RANK" in os.environ:
            # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm runs on one rank and may use the host's cores
            O.set_num_threads(len(os.sched_getaffinity(0)))
        self.w, self.lens = w, lens[:nseq]
        d, hq, hkv, mode = w["d"], w["hq"], w["hkv"], w["mode"]
        self.tab = O.codebook(d, 4) if mode == 0 else np.zeros(32, np.float32)
        self.rows, self.qs = [], []
        for i, L in enumerate(self.lens):
            kx = O.normal(1002 + i, hkv * int(L) * d).reshape(-1, d)
            vx = O.normal(1003 + i, hkv * int(L) * d).reshape(-1, d)
            self.rows.append((O.quantize_rows(kx, mode, 4, self.tab).reshape(hkv, int(L), -1),
                              O.quantize_rows(vx, mode, 4, self.tab).reshape(hkv, int(L), -1)))
            self.qs.append(O.round_to(O.normal(1001 + i, hq * d).reshape(hq, d), w["qdt"]))
        sub = dict(w)
        sub["b"] = len(self.lens)
        self.bytes = algorithmic_bytes(sub, self.lens)

    def run(self):
        """One pass; returns seconds."""
        w = self.w
        t0 = time.perf_counter()
        for (kw, vw), q in zip(self.rows, self.qs):
            self.O.cpu_decode_step(kw, vw, q, w["mode"], 4, self.tab, self.tab, w["qdt"], w["d"] ** -0.5)
        return time.perf_counter() - t0

    def describe(self):
        return (f"{len(self.lens)} of {self.w['b']} sequences per step ({int(self.lens.sum())} keys x {self.w['hkv']} kv heads): "
                f"dequantize the cached rows to {self.w['qdt']} + unfused attention, C with OpenMP")


def cpu_sample_size(w, lens, budget_keys=1 << 18):
    """Sequences of the batch for one pass of the CPU arm: all of a ragged batch of a few hundred thousand keys, else as
    many as hold about that number of keys (a pass is a fraction of a second to a few seconds of the host's cores)."""
    if w["lens"] == "uniform512-8192":
        return w["b"]
    return min(w["b"], max(1, budget_keys // int(lens[0])))


def cpu_best_pass(sample, seconds=3.0, max_passes=20):
    """(best time of a pass, passes run): one untimed pass, then passes until `seconds` have gone by (at least two)."""
    sample.run()
    t0, best, n = time.perf_counter(), float("inf"), 0
    while n < 2 or (time.perf_counter() - t0 < seconds and n < max_passes):
        best = min(best, sample.run())
        n += 1
    return best, n


def cpu_prefill_sample():
    """The reference's CPU attention on a bounded sample of c3: the last 64 query tokens of one sequence, all heads,
    over the full 4096 keys (causal)."""
    from oracle import oracle as O
    if os.environ.get("OMP_NUM_THREADS") == "1" and "LOCAL_RANK" in os.environ:
        O.set_num_threads(len(os.sched_getaffinity(0)))
    s, hq, hkv, d, lq = 4096, 32, 8, 128, 64
    q = O.round_to(O.normal(1001, lq * hq * d).reshape(1, lq, hq, d), "bf16")
    k = O.round_to(O.normal(1002, s * hkv * d).reshape(1, s, hkv, d), "bf16")
    v = O.round_to(O.normal(1003, s * hkv * d).reshape(1, s, hkv, d), "bf16")
    O.reference_attention(q[:, :4], k, v, d ** -0.5, wr=0)
    t0 = time.perf_counter()
    O.reference_attention(q, k, v, d ** -0.5, wr=0)
    dt = time.perf_counter() - t0
    flops = 4.0 * hq * d * sum(s - lq + i + 1 for i in range(lq))
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"last {lq} query tokens of one sequence, all heads, {s} keys ({dt:.2f} s)"}, flops


def run_reference(args, w, rank, world):
    if rank != 0:
        return
    from oracle import oracle as O
    if args.workload == "c3":
        cpu, _ = cpu_prefill_sample()
        print(json.dumps({"impl": "reference", "metric": "prefill_attention_tflops", "value": cpu["value"], "unit": "TFLOP/s",
                          "n_gpus": args.gpus, "steps": 1, "warmup": 0, "higher_is_better": True, "config": {"workload": "c3 (sample)"},
                          "cpu_baseline": cpu, "e2e": {"value": cpu["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}),
              flush=True)
        return
    lens = seq_lens(w)
    nseq = cpu_sample_size(w, lens)
    # about a minute of CPU work for the whole run: fewer sequences per step when many steps are asked for
    nseq = max(1, min(nseq, int(60.0 / max(args.steps + args.warmup, 1) / 0.17)))
    sample = CpuSample(w, lens, nseq)
    for _ in range(args.warmup):
        sample.run()
    times = [sample.run() for _ in range(args.steps)]
    t = float(np.mean(times))
    gbs = sample.bytes / t / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": f"{args.workload}: {w['desc']}", "sample": sample.describe()},
            "tokens_per_s": nseq / t,
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": O.num_threads(), "kind": "port", "sample": sample.describe()},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------------------

def aggregate_over_ranks(times_ms, nbytes, world, dev):
    """(max over ranks of each time, sum over ranks of the bytes); every rank gets the same result."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(times_ms), device=dev, dtype=torch.float64)
    n = torch.tensor([float(nbytes)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(n, op=dist.ReduceOp.SUM)
    return [float(x) for x in t.cpu()], float(n.cpu()[0])


def clock_sample_steps(ms_per_step, seconds=0.6, cap=20000):
    """Untimed steps that keep the device under the measured load while nvidia-smi samples its clocks. Computed
    from the time already reduced over the ranks, so that all ranks run the same number of collectives."""
    return int(min(cap, max(50, seconds * 1e3 / max(ms_per_step, 1e-3))))


def peaks():
    try:
        return json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except OSError:
        return {}


class Env:
    """What all legs of one run share: the package, the device, the ranks."""

    def __init__(self, args, rank, world, local_rank):
        import torch
        import torch.distributed as dist

        import __graft_entry__ as G
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path (use --impl reference for the CPU arm)")
        torch.cuda.set_device(local_rank)
        self.torch, self.dist = torch, dist
        self.dev = torch.device("cuda", local_rank)
        self.rank, self.world, self.local_rank, self.args = rank, world, local_rank, args
        if world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        G.build()
        self.P = G.load_package()
        self.t0 = time.perf_counter()

    def stage(self, msg):
        if self.args.verbose:
            print(f"[bench rank {self.rank} +{time.perf_counter() - self.t0:6.1f}s] {msg}", file=sys.stderr, flush=True)

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()


def ref_gpu_decode(env, w, lens, caches, kq, vq, steps):
    """The reference's own GPU kernels (its kernel headers compiled for sm_100a, its launch plan replayed: baseline/ref_cuda.cu)
    on the same cached rows of the same device: attention and combine launches alone, f32 queries already rotated, no
    rotation, cast or allocation timed. A ragged batch is one call per sequence (the reference's cache has one length).
    Returns the "ref_gpu_kernels" object or None when the library was not built."""
    torch, dev = env.torch, env.dev
    from baseline import ref_cuda as R
    if not R.available():
        return None
    b, hq, hkv, d = w["b"], w["hq"], w["hkv"], w["d"]
    q32 = torch.randn((b, hq, 1, d), device=dev, dtype=torch.float32)
    tab = torch.cat([kq.tab, vq.tab])
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    refs = [R.TqAttention(torch, q32, kc, vc, lens, kq.layout, vq.layout, kq.format.mode, vq.format.mode, tab, d ** -0.5, sms)
            for kc, vc in caches]
    stream = torch.cuda.current_stream(dev)
    for r in refs:
        r.run(stream.cuda_stream)
    torch.cuda.synchronize()
    graphs = []
    for r in refs:
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            r.run(torch.cuda.current_stream(dev).cuda_stream)
        graphs.append(gr)
    n = max(2, min(steps, 20))
    for i in range(len(graphs)):
        graphs[i].replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(n):
        graphs[i % len(graphs)].replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    r0 = refs[0]
    return {"value": algorithmic_bytes(w, lens) / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "steps": n,
            "launches_per_step": r0.launches, "kernel": f"tq_attn{'g%d' % r0.group if r0.group > 1 else ''}{'_fp8' if w['mode'] == 5 else ''} + tq_combine",
            "what": (f"the reference's kernels compiled for sm_100a, its launch plan ({len(r0.calls)} call(s) per step, key splits "
                     f"{min(r0.splits)}-{max(r0.splits)}), CUDA graph replay; attention and combine launches only")}



def decode_leg(env, name, w_full, steps, warmup, with_e2e=True, with_cpu=True, layers=1, gather=None):
    """Times workload `w_full` (sharded over the ranks when it says so): exactly `steps` steps between two events.
    `gather`: assemble the outputs of all ranks on every rank inside the step. By default where one problem is split
    over the ranks (strong scaling: the layer's output has to be put together again); ranks that each hold a batch of
    their own (weak scaling) have nothing to exchange. Returns the result line (rank 0) or None."""
    torch, dist, P, dev, rank, world = env.torch, env.dist, env.P, env.dev, env.rank, env.world
    strong = w_full["shard"] is not None and world > 1
    use_gather = world > 1 and (strong if gather is None else bool(gather))
    w = shard_of(w_full, world) if strong else dict(w_full)
    if w is None:
        return None
    if name == "c4" and world == 1:
        w.update(C4_SINGLE)
    b, hq, hkv, d = w["b"], w["hq"], w["hkv"], w["d"]
    tdt = {"bf16": torch.bfloat16, "f16": torch.float16}[w["qdt"]]
    lens = seq_lens(w, rank)
    total_steps = steps + warmup + 8
    cap = int(lens.max()) + 2 * total_steps + 4
    kq = P.TurboQuantizer(P.QuantFormat.parse(w["fmt"]), d, w["rot"], 42, dev)
    vq = P.TurboQuantizer(P.QuantFormat.parse(w["fmt"]), d, w["rot"], 44, dev)
    rw = kq.row_words()
    # several distinct caches (the layers of a model), cycled, so that no step finds its rows in L2
    cache_bytes = b * hkv * cap * rw * 4 * 2
    nbuf = int(max(2, min(4, (3 * 126e6) // cache_bytes + 1)))
    from candle_rocm_vulkan_b200.turbo_quant import _kv_append
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    caches = []
    for _ in range(nbuf):
        kc = torch.zeros((b, hkv, cap, rw), dtype=torch.int32, device=dev)
        vc = torch.zeros((b, hkv, cap, rw), dtype=torch.int32, device=dev)
        # fill on the device in slabs: synthetic N(0, 1) keys / values with 1% outlier channels x8 (c2)
        slab = 1024
        chan = torch.ones((1, hkv, 1, d), device=dev, dtype=tdt)
        if name == "c2":
            idx = torch.randperm(hkv * d, generator=g, device=dev)[: (hkv * d + 99) // 100]
            chan.view(-1)[idx] = 8
        for p0 in range(0, int(lens.max()), slab):
            t = min(slab, int(lens.max()) - p0)
            k = torch.randn((b, hkv, t, d), generator=g, device=dev, dtype=tdt) * chan
            v = torch.randn((b, hkv, t, d), generator=g, device=dev, dtype=tdt) * chan
            _kv_append(k, v, kc, vc, kq, vq, p0)
        caches.append((kc, vc))
    env.stage(f"{name}: caches filled")
    kv_len = torch.from_numpy(lens).to(dev)
    # the step's inputs (queries and the new token's keys and values) are packed into one pinned host buffer, so that
    # the end-to-end step pays for one host-to-device copy
    nq, nkv = b * hq * d, b * hkv * d
    step_host = torch.randn(nq + 2 * nkv, dtype=tdt).pin_memory()
    step_dev = step_host.to(dev)
    out_host = torch.empty((b, hq, 1, d), dtype=tdt).pin_memory()
    q = step_dev[:nq].view(b, hq, 1, d)
    out = torch.empty((b, hq, 1, d), dtype=tdt, device=dev)
    gathered = torch.empty((world * b, hq, 1, d), dtype=tdt, device=dev) if use_gather else None
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    status = torch.zeros(1, dtype=torch.int32, device=dev)  # set by the kernels when a bounded device wait runs out

    # N > 1: the outputs of all ranks are assembled on every rank inside the step, by the attention's own epilogue
    # (peer stores over NVLink into symmetric memory, b200_tq_attention_gather); if symmetric memory cannot be had, by an
    # NCCL all-gather after the attention
    peer_gather = None
    if use_gather:
        try:
            peer_gather = P.OutputGather(b * hq, d, tdt, dev)
        except Exception as e:
            print(f"bench: symmetric memory for the fused gather is unavailable ({e}); using NCCL", file=sys.stderr)
        ok_all = torch.tensor([1 if peer_gather is not None else 0], device=dev)
        dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)
        if int(ok_all.item()) == 0:
            peer_gather = None
    # the timed steps stand for attention calls over caches that nobody writes meanwhile (lengths fixed before): each
    # attention takes its place on the GPU, and streams its first keys, while the previous one's kernel ends
    # (B200_TQ_AFTER_PREV | B200_TQ_INPUTS_FINAL). On one GPU the calls also come in runs with an output and a workspace
    # of their own each (B200_TQ_OUTPUTS_FREE), so that no store waits for the call before; a run is the steps of one graph
    # replay and starts with a plain launch, behind which nothing earlier is still running. With gathered outputs (several ranks) every call's stores
    # wait for the previous call, whose step word they follow.
    # one run = the steps of one graph replay (a replay starts when the one before has completed)
    group = steps if steps <= 128 else 32
    group = max(nbuf, group // nbuf * nbuf)  # whole rounds of the caches: a replay does not start on the cache that the one before ended on
    run_len = group if not use_gather else nbuf
    if not use_gather:
        outs = [out] + [torch.empty_like(out) for _ in range(run_len - 1)]
        calls = [P.PackedAttention(q, caches[j % nbuf][0], caches[j % nbuf][1], kv_len, kq, vq, cfg, out=outs[j], after_prev=j > 0,
                                   fresh_rows=0 if j > 0 else None, status=status, outputs_free=j > 0) for j in range(run_len)]
    else:
        calls = [P.PackedAttention(q, kc, vc, kv_len, kq, vq, cfg, out=out, gather=peer_gather, after_prev=True, fresh_rows=0, status=status)
                 for kc, vc in caches]

    def eager_step(i):
        calls[i % run_len].run()
        if use_gather and peer_gather is None:
            dist.all_gather_into_tensor(gathered, out)

    for i in range(nbuf):
        eager_step(i)
    torch.cuda.synchronize()
    # CUDA graphs: one per cache (a single step), and one of `group` consecutive steps (cache after cache), so that steps
    # of a few microseconds are not bound by the host's replay rate. Inside a graph every attention is the programmatic
    # dependent of the one before; between two replays there is no such edge, so the timed steps are one graph when
    # they are few (up to 128), groups of 32 otherwise.
    graphs, long_graph = [], None
    try:
        for i in range(nbuf):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                eager_step(i)
            graphs.append(gr)
        long_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(long_graph):
            for i in range(group):
                eager_step(i)
    except Exception as e:  # report and time the eager launches instead
        print(f"bench: CUDA graph capture failed ({e}); timing eager launches", file=sys.stderr)
        graphs, long_graph = [], None
        torch.cuda.synchronize()
    env.stage(f"{name}: graphs captured: {len(graphs)}")

    def run_steps(k):
        """Exactly k steps: whole groups through the long graph, the rest one by one."""
        i = 0
        while long_graph is not None and k - i >= group:
            long_graph.replay()
            i += group
        while i < k:
            if graphs:
                graphs[i % nbuf].replay()
            else:
                eager_step(i)
            i += 1

    run_steps(warmup)
    env.barrier()
    sampler = ClockSampler(env.local_rank)
    if rank == 0:
        sampler.start()
    # ---- device-resident timing: exactly K steps between two events on the launching stream
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    env.barrier()
    ev0.record()
    run_steps(steps)
    ev1.record()
    env.barrier()
    total_ms = ev0.elapsed_time(ev1)
    env.stage(f"{name}: timed region done")
    # beside it (not the value): the same K steps as calls that share one output and one workspace, so that the stores of
    # every call wait for the call before (B200_TQ_AFTER_PREV | B200_TQ_INPUTS_FINAL without B200_TQ_OUTPUTS_FREE)
    waiting_ms = None
    if not use_gather and with_cpu:
        wcalls = [P.PackedAttention(q, kc, vc, kv_len, kq, vq, cfg, out=out, after_prev=True, fresh_rows=0, status=status) for kc, vc in caches]
        for c in wcalls:
            c.run()
        torch.cuda.synchronize()
        try:
            wg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(wg):
                for i in range(group):
                    wcalls[i % nbuf].run()
            wg.replay()
            torch.cuda.synchronize()
            w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(1, steps // group)
            w0.record()
            for _ in range(reps):
                wg.replay()
            w1.record()
            torch.cuda.synchronize()
            waiting_ms = w0.elapsed_time(w1) / (reps * group)
            del wg
        except Exception as e:
            print(f"bench: the comparison leg could not be captured ({e})", file=sys.stderr)
            torch.cuda.synchronize()
        wcalls.clear()
    gather_note = "outputs all-gathered over NCCL"
    if peer_gather is not None and use_gather:
        # the gathered rows of the last step against an NCCL all-gather of the same outputs
        dist.all_gather_into_tensor(gathered, out)
        torch.cuda.synchronize()
        mine = peer_gather.gathered().reshape(gathered.shape)
        same = torch.tensor([1 if torch.equal(mine, gathered) else 0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        if int(same.item()) != 1:
            raise SystemExit(f"bench ({name}): the fused gather differs from the NCCL all-gather of the same outputs")
        gather_note = "outputs gathered on every rank by the attention epilogue (peer stores over NVLink; checked against NCCL)"
    e2e_ms = None
    if with_e2e:
        # ---- end to end through the public API with host buffers: H2D of the step's inputs, append of the new token,
        # attention, D2H of the outputs. A serving loop overlaps the copies of neighbouring steps with the kernels: inputs
        # are triple and outputs double buffered, the host-to-device copy of step i + 1 and the device-to-host copy of
        # step i - 1 run on their own streams beside the kernels of step i. Every step still copies its own inputs in and
        # its own result out.
        lens_dev = kv_len.clone()
        # Rings of input and output buffers, and the main stream's waits for the copy streams taken in batches of RUN
        # steps: an event wait in front of a kernel makes it wait for the whole of its predecessor, so a wait per step
        # would keep every attention from starting before the one before has ended. Inside a batch nothing stands between
        # the kernels: the append of step i + 1 is launched while the attention of step i drains (B200_KV_AFTER_PREV: it
        # writes a row that this attention does not read), and the attention of step i + 1 behind it streams its old
        # rows meanwhile (B200_TQ_AFTER_PREV | B200_TQ_INPUTS_FINAL, fresh_rows = 1) and, on one GPU, stores into an
        # output and a workspace of its own (B200_TQ_OUTPUTS_FREE; the batch's first append is a plain launch behind
        # the waits). Every step still copies its own inputs in and its own result out; the copies run RUN to 2 RUN
        # steps ahead of / behind the kernels on their own streams.
        RUN = 16
        depth = 3 * RUN
        in_dev = [step_dev] + [torch.empty_like(step_dev) for _ in range(depth - 1)]
        out_dev = [out] + [torch.empty_like(out) for _ in range(depth - 1)]
        out_hosts = [out_host] + [torch.empty_like(out_host).pin_memory() for _ in range(depth - 1)]
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

        def e2e_steps(first, count):
            """Steps first .. first + count - 1 as a pipeline over the current stream and two copy streams."""
            main = torch.cuda.current_stream(dev)
            fork = torch.cuda.Event()
            fork.record(main)
            s_in.wait_event(fork)
            s_out.wait_event(fork)
            ev_in, ev_done, ev_out = {}, {}, {}
            end = first + count
            keep = []  # the calls of this group stay alive to its end: each owns its workspace, which no later call of the group may get

            def h2d(i):
                if i >= end or i in ev_in:
                    return
                with torch.cuda.stream(s_in):
                    if i - depth in ev_done:
                        s_in.wait_event(ev_done[i - depth])   # the kernels of step i - depth have read this input buffer
                    in_dev[i % depth].copy_(step_host, non_blocking=True)
                    ev_in[i] = torch.cuda.Event()
                    ev_in[i].record(s_in)

            for i in range(first, first + count):
                j = i - first
                if j % RUN == 0:
                    # a batch begins: the copies of the batch after it are queued, this batch's inputs (queued a batch ago)
                    # and the output buffers it writes (copied out two batches ago) are waited for, all at once
                    for x in range(i, i + 2 * RUN):
                        h2d(x)
                    for x in range(i, min(i + RUN, end)):
                        main.wait_event(ev_in[x])
                        if x - depth in ev_out:
                            main.wait_event(ev_out[x - depth])
                ob, ib = i % depth, i % depth
                kc, vc = caches[i % nbuf]
                qv = in_dev[ib][:nq].view(b, hq, 1, d)
                kn = in_dev[ib][nq:nq + nkv].view(b, hkv, 1, d)
                vn = in_dev[ib][nq + nkv:].view(b, hkv, 1, d)
                # the device lengths are those at the start of this group of steps: step j appends at lens + j and attends
                # to lens + j + 1 keys (offsets in the call arguments), so no kernel sits between append and attention
                _kv_append(kn, vn, kc, vc, kq, vq, lens_dev, pos_add=j, status=status, after_prev=(j % RUN != 0))
                keep.append(P.PackedAttention(qv, kc, vc, lens_dev, kq, vq, cfg, out=out_dev[ob], gather=peer_gather, kv_len_add=j + 1,
                                              after_prev=True, fresh_rows=1, status=status, outputs_free=not use_gather))
                keep[-1].run()
                if use_gather and peer_gather is None:
                    dist.all_gather_into_tensor(gathered, out_dev[ob])
                ev_done[i] = torch.cuda.Event()
                ev_done[i].record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[i])
                    out_hosts[ob].copy_(out_dev[ob], non_blocking=True)
                    ev_out[i] = torch.cuda.Event()
                    ev_out[i].record(s_out)
            lens_dev.add_(count)                              # one length update per group of steps
            # the group ends when its copies have ended
            main.wait_event(ev_in[end - 1])
            for x in range(max(first, end - depth), end):
                main.wait_event(ev_out[x])

        e2e_steps(0, max(min(warmup, 3), nbuf))
        env.barrier()
        # the same calls captured once (copies and stream dependencies included): a serving loop replays its steps
        # instead of paying the host's call path every token
        # like the device-timed loop: the timed steps are one graph when they are few, groups of 32 otherwise (a multiple of
        # the caches cycled, so that every replay starts on the same one)
        e2e_group = steps if steps <= 128 else 32
        e2e_group = max(nbuf, e2e_group - e2e_group % nbuf)
        e2e_graph = None
        if graphs:
            try:
                e2e_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(e2e_graph):
                    e2e_steps(0, e2e_group)
            except Exception as e:
                print(f"bench: capture of the end-to-end steps failed ({e}); timing eager calls", file=sys.stderr)
                e2e_graph = None
                torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        env.barrier()
        e0.record()
        i = 0
        while i < steps:
            if e2e_graph is not None and steps - i >= e2e_group:
                e2e_graph.replay()
                i += e2e_group
            else:
                e2e_steps(i, 1)
                i += 1
        e1.record()
        env.barrier()
        e2e_ms = e0.elapsed_time(e1)
        e2e_graph = None
        env.stage(f"{name}: end-to-end region done")
    # max over ranks of the times, sum over ranks of the bytes
    (total_ms, e2e_ms_r), job_bytes = aggregate_over_ranks([total_ms, e2e_ms or 0.0], algorithmic_bytes(w, lens), world, dev)
    # the timed regions last milliseconds: keep the same step running (untimed) until the clock sampler has seen
    # about half a second of this load. Every rank runs the same number of steps (they hold a collective).
    extra = clock_sample_steps(total_ms / steps, seconds=0.6 if name == "c2" else 0.3)
    for i in range(0, extra, 256):
        run_steps(min(256, extra - i))
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    bad = torch.tensor([int(status.item())], device=dev)
    if world > 1:
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
    if int(bad.item()) != 0 or P._abi.lib().b200_device_wait_status() != 0:
        raise SystemExit(f"bench ({name}): a bounded device wait ran out or an append position was out of range (status {int(bad.item())}); the numbers are void")
    line = None
    if rank == 0:
        pk = peaks()
        peak, peak_kind = (pk["hbm_gbs"], "measured copy bandwidth (MEASURED_PEAKS.json)") if "hbm_gbs" in pk else (6650.0, "fallback")
        ms = total_ms / steps
        value = job_bytes / (ms * 1e-3) / 1e9
        achieved = algorithmic_bytes(w, lens) / (ms * 1e-3) / 1e9
        cpu = None
        if with_cpu:
            from oracle import oracle as O
            sample = CpuSample(w, lens, cpu_sample_size(w, lens))
            dt, passes = cpu_best_pass(sample)
            cpu = {"value": sample.bytes / dt / 1e9, "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
                   "sample": f"{sample.describe()}; best of {passes} passes ({dt:.2f} s each)"}
        # one decode grid per step when it merges its segments itself (few segments per column: c2, c5); else a combine
        # grid follows (with N > 1 its last block publishes the gathered step)
        ncols = b * hkv * max(1, (hq // hkv + 7) // 8)
        pair = w["mode"] == 0  # the codebook formats run on the kernel whose workers are pairs of warps
        # (up to 128 workers per column for the calls of a run, which are declared independent of the call before)
        nworkers = min(148 * (2 if pair else 3) * 4, int(((lens.astype(np.int64) + 31) // 32).sum()) * (ncols // b))  # at most one worker per tile
        in_kernel = ncols * (8 if use_gather else 128) > nworkers
        launches_per_step = 1 if in_kernel else 2
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "f16 mma / f32 softmax", "data": "synthetic",
            "config": {"workload": f"{name}: {w_full['desc'] if not (name == 'c4' and world == 1) else w['desc']}",
                       "batch_per_gpu": b, "hq": hq, "hkv": hkv, "head_dim": d,
                       "kv_format": w["fmt"], "rotation": w["rot"], "total_keys_per_gpu": int(lens.sum()),
                       "launch": (f"CUDA graph replay ({group} steps per graph)" if graphs else "eager C ABI calls") + "; every attention is launched as a programmatic dependent of the previous one with its inputs declared final (B200_TQ_AFTER_PREV | B200_TQ_INPUTS_FINAL): it streams its first keys while the previous kernel drains" + (f"; runs of {run_len} calls with an output and a workspace of their own each (B200_TQ_OUTPUTS_FREE: no store waits for the call before), every run begun by a plain launch" if not use_gather else ""),
                       "l2": f"{nbuf} caches of {cache_bytes / 1e6:.0f} MB cycled (each step reads other rows than the last; L2 is 126 MB)",
                       "parallelism": (f"{'kv heads' if w_full['shard'] == 'kv_head' else 'batch'} split x{world}, {gather_note}" if strong
                                       else (f"a batch of its own on each of {world} ranks, " + (gather_note if use_gather else "no exchange (nothing depends on another rank)")
                                             if world > 1 else "single GPU")),
                       "output_gather": use_gather},
            "tokens_per_s": (w_full["b"] if strong else world * b) / (ms * 1e-3),
            "pct_of_8000_gbs_nominal": 100.0 * value / (8000.0 * world),
            "gpu_launches": steps * launches_per_step * world,  # of all ranks, like `value`
            "stores_wait_for_previous_call": (None if waiting_ms is None else
                                              {"ms_per_step": waiting_ms, "value": algorithmic_bytes(w, lens) / (waiting_ms * 1e-3) / 1e9, "unit": "GB/s",
                                               "what": "the same steps as calls that share one output and one workspace (no B200_TQ_OUTPUTS_FREE): not the value, beside it"}),
            "roofline": {"bound": "hbm", "kernel": "tq_decode_pair_kernel" if pair else "tq_decode_kernel",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_kind, "traffic": None, "traffic_unit": "bytes per launch", "traffic_source": None},
            "cpu_baseline": cpu, "clocks": clocks,
        }
        if layers > 1:
            line["tokens_per_s_model_step"] = (w_full["b"] if strong else world * b) / (ms * 1e-3 * layers)
            line["config"]["layers"] = f"{layers}-layer decode step = {layers} x this step ({nbuf} distinct layer caches cycled)"
        if with_e2e:
            line["e2e"] = {"value": job_bytes / (e2e_ms_r / steps * 1e-3) / 1e9, "unit": "GB/s",
                           "h2d_bytes_per_step": int(nq + 2 * nkv) * 2, "d2h_bytes_per_step": int(nq) * 2,
                           "ms_per_step": e2e_ms_r / steps, "tokens_per_s": (w_full["b"] if strong else world * b) / (e2e_ms_r / steps * 1e-3)}
    if line is not None and world == 1 and with_cpu:
        ref_gpu = ref_gpu_decode(env, w, lens, caches, kq, vq, steps)
        if ref_gpu is not None:
            line["ref_gpu_kernels"] = ref_gpu
    # release what the leg holds before the next one allocates
    graphs.clear()
    long_graph = None
    calls.clear()
    caches.clear()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    del peer_gather
    torch.cuda.empty_cache()
    return line


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline kernel, from the ncu capture of the same
# workload (profiles/): filled in for the workloads that have a committed capture
TRAFFIC = {"c2": (366_696_192, "ncu capture of this workload, profiles/tq_decode_kernel_c2_mxfp4.md")}


def prefill_leg(env, steps, warmup):
    """Workload c3: causal prefill of B=4 x S=4096 (Hq 32, Hkv 8, D 128, bf16) with the new K / V written into an
    NVFP4 cache in the same call. Metric: attention TFLOP/s (4 B Hq S^2 D / 2 flop per step). Several ranks split the
    batch entries (2 or 4 ranks) or the kv heads with their query heads (8 ranks): strong scaling, no exchange (the
    outputs and the cache rows stay with the rank that owns the sequence or the head). Returns the line on rank 0."""
    torch, P, dev, world = env.torch, env.P, env.dev, env.world
    F = P.flash_attn
    b, s, hq, hkv, d = 4, 4096, 32, 8, 128
    b_all, hq_all = b, hq
    shard = "single GPU"
    if world > 1:
        if b % world == 0:
            b //= world
            shard = f"batch entries split over {world} ranks ({b} per rank), no exchange"
        elif hkv % world == 0:
            hq, hkv = hq // world, hkv // world
            shard = f"kv heads split over {world} ranks ({hkv} per rank with their {hq} query heads), no exchange"
        else:
            return None
    nv = P.QuantFormat.parse("nvfp4")
    kq, vq = P.TurboQuantizer(nv, d, "none", 42, dev), P.TurboQuantizer(nv, d, "none", 44, dev)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    # q / k / v sets cycled (335 MB each on one GPU, a share of it on several): at least 400 MB pass before a set comes
    # round again, so that no step finds its inputs in L2
    nbuf = max(3, -(-400 * world // 335))
    sets = []
    for i in range(nbuf):
        g = torch.Generator(device=dev).manual_seed(77 + i)
        sets.append((torch.randn((b, s, hq, d), generator=g, device=dev, dtype=torch.bfloat16),
                     torch.randn((b, s, hkv, d), generator=g, device=dev, dtype=torch.bfloat16),
                     torch.randn((b, s, hkv, d), generator=g, device=dev, dtype=torch.bfloat16)))
    kc = torch.zeros((b, hkv, s, kq.row_words()), dtype=torch.int32, device=dev)
    vc = torch.zeros_like(kc)

    def step(i):
        q, k, v = sets[i % nbuf]
        return F.prefill_append(q, k, v, cfg, kc, vc, kq, vq, 0)

    for i in range(warmup):
        step(i)
    env.barrier()
    sampler = ClockSampler(env.local_rank)
    if env.rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    env.barrier()
    ms = e0.elapsed_time(e1) / steps
    # attention alone (the dominant kernel), for the roofline
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for i in range(steps):
        q, k, v = sets[i % nbuf]
        F.flash_attn_with_config(q, k, v, cfg)
    a1.record()
    torch.cuda.synchronize()
    attn_ms = a0.elapsed_time(a1) / steps
    env.barrier()
    # end to end: host q / k / v in, host output back
    hq_, hk_, hv_ = [t.cpu().pin_memory() for t in sets[0]]
    out_host = torch.empty((b, s, hq, d), dtype=torch.bfloat16).pin_memory()
    dq, dk, dv = [torch.empty_like(t) for t in sets[0]]

    def e2e_step():
        dq.copy_(hq_, non_blocking=True)
        dk.copy_(hk_, non_blocking=True)
        dv.copy_(hv_, non_blocking=True)
        out_host.copy_(F.prefill_append(dq, dk, dv, cfg, kc, vc, kq, vq, 0), non_blocking=True)

    e2e_step()
    env.barrier()
    n_e2e = max(2, min(steps, 5))
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    env.barrier()
    e2e_ms = e0.elapsed_time(e1) / n_e2e
    # the slowest rank's times; every rank runs the same number of untimed steps for the clock sampler
    (ms, attn_ms, e2e_ms), _ = aggregate_over_ranks((ms, attn_ms, e2e_ms), 0, world, dev)
    for i in range(clock_sample_steps(ms, seconds=0.4, cap=400)):
        step(i)
    torch.cuda.synchronize()
    clocks = sampler.stop() if env.rank == 0 else None
    if P._abi.lib().b200_device_wait_status() != 0:
        raise SystemExit("bench: a bounded device wait ran out; the numbers are void")
    if env.rank != 0:
        sets.clear()
        torch.cuda.empty_cache()
        return None
    flops = 4.0 * b_all * hq_all * s * s * d / 2  # the whole job
    pk = peaks()
    peak, kind = (pk["bf16_tflops"], "measured cuBLAS bf16 burst (MEASURED_PEAKS.json)") if "bf16_tflops" in pk else (1590.0, "fallback")
    cpu = cpu_prefill_sample()[0] if world == 1 else None
    achieved = flops / (attn_ms * 1e-3) / 1e12
    peak *= world
    line = {"metric": "prefill_attention_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "bf16 mma / f32 softmax", "data": "synthetic",
            "config": {"workload": "c3: causal prefill B=4 S=4096 Hq=32 Hkv=8 D=128 bf16 + NVFP4 cache append",
                       "l2": f"{nbuf} input sets of {335 // world} MB cycled (L2 is 126 MB)", "parallelism": shard},
            "tokens_per_s": b_all * s / (ms * 1e-3),
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(sum(t.numel() for t in sets[0])) * 2 * world, "d2h_bytes_per_step": int(out_host.numel()) * 2 * world},
            "gpu_launches": steps * 2 * world,  # the attention kernel and the quantize-on-append kernel (K and V in one grid)
            "roofline": {"bound": "tensor", "kernel": "fa_prefill_sm100_kernel2 (attention alone)", "achieved": achieved,
                         "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": kind + (f" x {world} GPUs" if world > 1 else ""),
                         "frac_of_sustained": achieved / (pk["bf16_tflops_sustained"] * world) if "bf16_tflops_sustained" in pk else None,
                         # dram read + write of one launch at B = 1 (50.4 + 3.0 MB, part of q / k / v still in L2 from the
                         # call before), times the 4 batch entries of c3, whose blocks do not share data
                         "traffic": 4 * 53_400_000 if world == 1 else None, "traffic_unit": "bytes per launch",
                         "traffic_source": "ncu capture at B=1 scaled by 4, profiles/fa_prefill_sm100_kernel2_b1_s4096.md"},
            "cpu_baseline": cpu, "clocks": clocks}
    from baseline import ref_cuda as R
    if R.available() and world == 1:
        # the reference's tile kernel of the tier a B200 selects, on the same tensors (attention alone; its append is a
        # second call in the reference and is not timed here)
        q, k, v = sets[0]
        o = torch.empty_like(q)
        st = torch.cuda.current_stream(dev).cuda_stream
        rc = R.lib().refcu_fa_prefill_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), b, s, hq, hkv, d ** -0.5, st)
        torch.cuda.synchronize()
        if rc == 0:
            e0.record()
            for i in range(2):
                q, k, v = sets[(i + 1) % nbuf]
                R.lib().refcu_fa_prefill_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), b, s, hq, hkv, d ** -0.5, st)
            e1.record()
            torch.cuda.synchronize()
            rms = e0.elapsed_time(e1) / 2
            ours = F.flash_attn_with_config(sets[0][0], sets[0][1], sets[0][2], cfg)
            R.lib().refcu_fa_prefill_bf16(sets[0][0].data_ptr(), sets[0][1].data_ptr(), sets[0][2].data_ptr(), o.data_ptr(), b, s, hq,
                                          hkv, d ** -0.5, st)
            torch.cuda.synchronize()
            line["ref_gpu_kernels"] = {"value": flops / (rms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": rms, "steps": 2,
                                       "launches_per_step": 1, "kernel": "fa3_d128_bf16_bf16 (BR 32, BC 64, grid 128 x 32 x 4)",
                                       "max_abs_diff_to_ours": float((ours.float() - o.float()).abs().max()),
                                       "what": "the reference's tile kernel compiled for sm_100a with its launch plan; attention alone"}
    sets.clear()
    torch.cuda.empty_cache()
    return line


def compact(line):
    """A result line cut down to what fits 600 characters: the extra workloads printed before the headline."""
    if line is None:
        return None
    c = {"extra_workload": line["config"]["workload"].split(":")[0], "metric": line["metric"], "value": round(line["value"], 1), "unit": line["unit"],
         "n_gpus": line["n_gpus"], "steps": line["steps"], "ms_per_step": round(line["ms_per_step"], 5), "scaling": line["scaling"],
         "roofline_frac": round(line["roofline"]["frac"], 4), "roofline_peak": line["roofline"]["peak"],
         "tokens_per_s": round(line["tokens_per_s"], 1)}
    if line["roofline"].get("frac_of_sustained") is not None:
        c["frac_of_sustained_peak"] = round(line["roofline"]["frac_of_sustained"], 4)
    if "tokens_per_s_model_step" in line:
        c["tokens_per_s_32_layer_step"] = round(line["tokens_per_s_model_step"], 1)
    if "e2e" in line:
        c["e2e"] = {"value": round(line["e2e"]["value"], 1), "ms_per_step": round(line["e2e"]["ms_per_step"], 5)}
    if line.get("cpu_baseline"):
        c["cpu_baseline"] = {"value": round(line["cpu_baseline"]["value"], 3), "cores": line["cpu_baseline"]["cores"]}
    if line.get("ref_gpu_kernels"):
        c["ref_gpu_kernels"] = {"value": round(line["ref_gpu_kernels"]["value"], 2), "ms_per_step": round(line["ref_gpu_kernels"]["ms_per_step"], 4)}
    if line.get("clocks"):
        c["clocks"] = {"sm_mhz": line["clocks"]["sm_mhz"], "reasons": line["clocks"]["reasons"]}
    c["batch_per_gpu"] = line["config"].get("batch_per_gpu")
    c["output_gather"] = line["config"].get("output_gather")
    c["hkv_per_gpu"] = line["config"].get("hkv")
    return c


def run_ours(args, rank, world, local_rank):
    env = Env(args, rank, world, local_rank)
    torch, dist = env.torch, env.dist
    head = args.workload
    lines = []
    if head == "c3":
        headline = prefill_leg(env, args.steps, args.warmup)
    else:
        wl = dict(WORKLOADS[head])
        if args.batch > 0:
            wl["b"] = args.batch
            wl["desc"] += f" [batch reduced to {args.batch}]"
        headline = decode_leg(env, head, wl, args.steps, args.warmup, layers=32 if head == "c5" else 1)
        if headline is not None and head in TRAFFIC and world == 1:
            headline["roofline"]["traffic"], headline["roofline"]["traffic_source"] = TRAFFIC[head]
    if not args.only:
        # the other configurations, shorter: c5, c4 and c3 as strong scaling over the ranks, c1 on one GPU
        short = max(8, min(args.steps, 48))
        for name in ("c5", "c4", "c1"):
            if name == head or (name == "c1" and world > 1):
                continue
            lines.append(compact(decode_leg(env, name, dict(WORKLOADS[name]), short, max(3, min(args.warmup, 6)), with_e2e=(name != "c5"),
                                            with_cpu=(world == 1), layers=32 if name == "c5" else 1)))
        if head != "c3":
            lines.append(compact(prefill_leg(env, max(3, min(args.steps, 10)), 3)))
        if head != "c3" and world > 1 and WORKLOADS[head]["shard"] is None:
            # the headline workload once more with the exchange that its own steps do not need: every rank's outputs
            # assembled on every rank by the attention's epilogue
            lines.append(compact(decode_leg(env, head, dict(WORKLOADS[head]), short, max(3, min(args.warmup, 6)), with_e2e=False,
                                            with_cpu=False, gather=True)))
    if rank == 0:
        for l in lines:
            if l is not None:
                print(json.dumps(l), flush=True)
        if headline is not None:
            print(json.dumps(headline), flush=True)
    if world > 1:
        # Release the device, meet the other ranks before the communicator goes. The teardown itself runs beside a
        # deadline, so that a rank whose peers are already gone still exits.
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        env.stage("tearing down the process group")
        th = threading.Thread(target=dist.destroy_process_group, daemon=True)
        th.start()
        th.join(timeout=20.0)
        sys.stdout.flush()
        sys.stderr.flush()
        # leave without the interpreter's own teardown of CUDA and NCCL objects, which can wait on a peer that is gone
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c3"], help="the headline workload (last line printed)")
    ap.add_argument("--only", action="store_true", help="time the headline workload alone")
    ap.add_argument("--batch", type=int, default=0, help="sequences of the headline workload (default: the configuration's); a "
                    "smaller batch keeps a profiler capture of the large configurations within a few GB")
    ap.add_argument("--verbose", action="store_true", help="print stage markers to stderr")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        w = dict(WORKLOADS[args.workload]) if args.workload != "c3" else None
        run_reference(args, w, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
