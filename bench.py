"""Benchmark of the quantized-KV decode attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1|c3|c4|c5]

One step = one decode-attention pass of one layer over a batch of synthetic sequences whose
compressed KV cache is resident in HBM (a ragged batch of 64 sequences with 512-8192 MXFP4 keys
by default: 32 query heads, 8 kv heads, head dim 128, bf16 queries). The metric is the achieved HBM
bandwidth on the algorithmic bytes of the step (packed code and scale bytes of every visible K and
V row, plus queries and outputs), with tokens/s beside it. With N > 1 every rank holds its own
batch (weak scaling, no data-path collective until the outputs are all-gathered over NCCL).

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
    # name: (batch, hq, hkv, d, format, q dtype, rotation, length rule, layers)
    "c2": dict(b=64, hq=32, hkv=8, d=128, fmt="mxfp4", mode=2, qdt="bf16", rot="none", lens="uniform512-8192", desc="ragged MXFP4 decode, B=64, lengths uniform in [512, 8192]"),
    "c1": dict(b=1, hq=32, hkv=8, d=128, fmt="fp8", mode=5, qdt="f16", rot="none", lens=2048, desc="single FP8 decode, 2048 keys"),
    "c4": dict(b=32, hq=8, hkv=1, d=128, fmt="turbo4", mode=0, qdt="bf16", rot="hadamard", lens=32768, desc="TurboQuant-4 decode, one kv head of B=32 x 32768 keys per GPU"),
    "c5": dict(b=128, hq=32, hkv=8, d=128, fmt="mxfp8", mode=4, qdt="f16", rot="none", lens=16384, desc="MXFP8 decode, B=128 x 16384 keys, one layer"),
}


def seq_lens(w, rank=0):
    from oracle import oracle as O  # only the seeded generator of the reference is used here
    if w["lens"] == "uniform512-8192":
        # every rank gets the same multiset of lengths (weak scaling: the work per GPU is fixed), in its own order
        lens = (512 + O.u64s(2002, w["b"]) % np.uint64(7681)).astype(np.int32)
        return np.roll(lens, 7 * rank)
    return np.full(w["b"], w["lens"], np.int32)


def algorithmic_bytes(w, lens):
    qo = w["b"] * w["hq"] * w["d"] * 2 * 2  # queries read + outputs written, 16-bit
    return int(lens.astype(np.int64).sum()) * w["hkv"] * 2 * PAYLOAD[w["mode"]] + qo


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


def cpu_reference_step(w, lens, nseq, reps=1):
    """The reference's CPU path for `nseq` sequences of the batch; returns (seconds per pass, bytes)."""
    from oracle import oracle as O
    if os.environ.get("OMP_NUM_THREADS") == "1" and "LOCAL_RANK" in os.environ:
        # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm runs on one rank and may use the host's cores
        O.set_num_threads(len(os.sched_getaffinity(0)))
    d, hq, hkv = w["d"], w["hq"], w["hkv"]
    mode = w["mode"]
    bits = 4
    tab = O.codebook(d, 4) if mode == 0 else np.zeros(32, np.float32)
    lens = lens[:nseq]
    rows, qs = [], []
    for i, L in enumerate(lens):
        kx = O.normal(1002 + i, hkv * int(L) * d).reshape(-1, d)
        vx = O.normal(1003 + i, hkv * int(L) * d).reshape(-1, d)
        rows.append((O.quantize_rows(kx, mode, bits, tab), O.quantize_rows(vx, mode, bits, tab)))
        qs.append(O.round_to(O.normal(1001 + i, hq * d).reshape(1, 1, hq, d), w["qdt"]))
    t0 = time.perf_counter()
    for _ in range(reps):
        for (kw, vw), q, L in zip(rows, qs, lens):
            L = int(L)
            # TurboKvCache::keys_values: dequantize every cached row, cast to the cache dtype
            k = O.round_to(O.dequantize_rows(kw, d, mode, bits, tab), w["qdt"]).reshape(1, hkv, L, d).transpose(0, 2, 1, 3)
            v = O.round_to(O.dequantize_rows(vw, d, mode, bits, tab), w["qdt"]).reshape(1, hkv, L, d).transpose(0, 2, 1, 3)
            O.unfused_attention(q, np.ascontiguousarray(k), np.ascontiguousarray(v), d ** -0.5, wr=0)
    dt = (time.perf_counter() - t0) / reps
    sub = dict(w)
    sub["b"] = nseq
    return dt, algorithmic_bytes(sub, lens)


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


def run_reference(args, w, rank, world):
    if rank != 0:
        return
    from oracle import oracle as O
    O.build() if not (ROOT / "oracle" / "liboracle.so").exists() else None
    lens = seq_lens(w)
    nseq = min(w["b"], 8 if w["lens"] == "uniform512-8192" else max(1, 65536 // int(lens[0])))
    # about a minute of CPU work for the whole run: fewer sequences per step when many steps are asked for
    nseq = max(1, min(nseq, int(60.0 / max(args.steps + args.warmup, 1) / 0.17)))
    for _ in range(args.warmup):
        cpu_reference_step(w, lens, min(nseq, 2))
    times = []
    nbytes = 0
    for _ in range(args.steps):
        dt, nbytes = cpu_reference_step(w, lens, nseq)
        times.append(dt)
    t = float(np.mean(times))
    gbs = nbytes / t / 1e9
    cores = O.num_threads()
    sample = f"{nseq} of {w['b']} sequences of the batch per step ({int(lens[:nseq].sum())} keys x {w['hkv']} kv heads), dequantize + unfused attention"
    line = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": f"{args.workload}: {w['desc']}", "sample": sample},
            "tokens_per_s": nseq / t,
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_ours(args, w, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    import __graft_entry__ as G

    t_start = time.perf_counter()

    def stage(msg):
        if args.verbose:
            print(f"[bench rank {rank} +{time.perf_counter() - t_start:6.1f}s] {msg}", file=sys.stderr, flush=True)

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    stage("process group up")
    G.build()
    P = G.load_package()
    stage("library loaded")
    A = P._abi
    b, hq, hkv, d = w["b"], w["hq"], w["hkv"], w["d"]
    tdt = {"bf16": torch.bfloat16, "f16": torch.float16}[w["qdt"]]
    lens = seq_lens(w, rank)
    total_steps = args.steps + args.warmup + 8
    cap = int(lens.max()) + 2 * total_steps + 4
    kq = P.TurboQuantizer(P.QuantFormat.parse(w["fmt"]), d, w["rot"], 42, dev)
    vq = P.TurboQuantizer(P.QuantFormat.parse(w["fmt"]), d, w["rot"], 44, dev)
    rw = kq.row_words()
    # several distinct caches, cycled, so that no step finds its rows in L2 (each is larger than L2 anyway for c2 / c4 / c5)
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
        if args.workload == "c2":
            idx = torch.randperm(hkv * d, generator=g, device=dev)[: (hkv * d + 99) // 100]
            chan.view(-1)[idx] = 8
        for p0 in range(0, int(lens.max()), slab):
            t = min(slab, int(lens.max()) - p0)
            k = torch.randn((b, hkv, t, d), generator=g, device=dev, dtype=tdt) * chan
            v = torch.randn((b, hkv, t, d), generator=g, device=dev, dtype=tdt) * chan
            _kv_append(k, v, kc, vc, kq, vq, p0)
        caches.append((kc, vc))
    stage("caches filled")
    kv_len = torch.from_numpy(lens).to(dev)
    # the step's inputs (queries and the new token's keys and values) are packed into one pinned host buffer, so that
    # the end-to-end step pays for one host-to-device copy
    nq, nkv = b * hq * d, b * hkv * d
    step_host = torch.randn(nq + 2 * nkv, dtype=tdt).pin_memory()
    q_host = step_host[:nq].view(b, hq, 1, d)
    knew_host = step_host[nq:nq + nkv].view(b, hkv, 1, d)
    vnew_host = step_host[nq + nkv:].view(b, hkv, 1, d)
    step_dev = step_host.to(dev)
    out_host = torch.empty((b, hq, 1, d), dtype=tdt).pin_memory()
    q = step_dev[:nq].view(b, hq, 1, d)
    out = torch.empty((b, hq, 1, d), dtype=tdt, device=dev)
    gathered = torch.empty((world * b, hq, 1, d), dtype=tdt, device=dev) if world > 1 else None
    cfg = P.FlashAttnConfig(d ** -0.5).causal()

    # one prepared call per cache, each captured in a CUDA graph (attention + the all-gather of the outputs), so
    # that the host only replays: a step of tens of microseconds would otherwise be bound by the Python call path
    # N > 1: the outputs of all ranks are assembled on every rank inside the step. Default: by the attention's own
    # epilogue (peer stores over NVLink into symmetric memory, b200_tq_attention_gather); B200_BENCH_GATHER=nccl uses
    # an NCCL all-gather after the attention instead.
    peer_gather = None
    if world > 1 and os.environ.get("B200_BENCH_GATHER", "fused") != "nccl":
        try:
            peer_gather = P.OutputGather(b * hq, d, tdt, dev)
        except Exception as e:
            print(f"bench: symmetric memory for the fused gather is unavailable ({e}); using NCCL", file=sys.stderr)
        ok_all = torch.tensor([1 if peer_gather is not None else 0], device=dev)
        dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)
        if int(ok_all.item()) == 0:
            peer_gather = None
    if world == 1 and os.environ.get("B200_BENCH_SELF_GATHER") == "1":
        # diagnostic: the gather epilogue with a world of one (plain device buffers), to time its protocol alone
        class _Self:
            pass
        peer_gather = _Self()
        peer_gather.buf = torch.zeros((2, 1, b * hq, d), dtype=tdt, device=dev)
        peer_gather._flags = torch.zeros(4, dtype=torch.int32, device=dev)
        peer_gather._state = torch.zeros(2, dtype=torch.int32, device=dev)
        peer_gather._ptrs = torch.tensor([peer_gather.buf.data_ptr(), peer_gather._flags.data_ptr()], dtype=torch.int64, device=dev)
        peer_gather.args = A.PeerGather(peer_gather._ptrs.data_ptr(), peer_gather._ptrs.data_ptr() + 8, 1, 0,
                                        peer_gather._state.data_ptr(), peer_gather._state.data_ptr() + 4)
    # the timed steps stand for the layers of one decode step (lengths fixed before the step): each attention may take
    # its place on the GPU while the previous layer's last kernel ends (B200_TQ_AFTER_PREV)
    calls = [P.PackedAttention(q, kc, vc, kv_len, kq, vq, cfg, out=out, gather=peer_gather, after_prev=True, fresh_rows=0)
             for kc, vc in caches]

    def eager_step(i):
        calls[i % nbuf].run()
        if world > 1 and peer_gather is None:
            dist.all_gather_into_tensor(gathered, out)

    for i in range(nbuf):
        eager_step(i)
    torch.cuda.synchronize()
    stage("eager steps done")
    # CUDA graphs: one per cache (a single step), and one of `group` consecutive steps (cache after cache), so
    # that steps of a few microseconds are not bound by the host's replay rate
    graphs, long_graph = [], None
    group = nbuf * max(1, 16 // nbuf)
    use_graphs = os.environ.get("B200_BENCH_GRAPHS", "1") != "0"
    if use_graphs:
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

    stage(f"graphs captured: {len(graphs)}")

    def step(i):
        if graphs:
            graphs[i % nbuf].replay()
        else:
            eager_step(i)

    def run_steps(k):
        """Exactly k steps: whole groups through the long graph, the rest one by one."""
        i = 0
        while long_graph is not None and k - i >= group:
            long_graph.replay()
            i += group
        while i < k:
            step(i)
            i += 1

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    run_steps(args.warmup)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- device-resident timing: exactly K steps between two events on the launching stream
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    run_steps(args.steps)
    ev1.record()
    barrier()
    total_ms = ev0.elapsed_time(ev1)
    stage("timed region done")
    gather_note = "outputs all-gathered over NCCL"
    if peer_gather is not None and world > 1:
        # the gathered rows of the last step against an NCCL all-gather of the same outputs
        dist.all_gather_into_tensor(gathered, out)
        torch.cuda.synchronize()
        mine = peer_gather.gathered().reshape(gathered.shape)
        same = torch.tensor([1 if torch.equal(mine, gathered) else 0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        if int(same.item()) != 1:
            raise SystemExit("bench: the fused gather differs from the NCCL all-gather of the same outputs")
        gather_note = "outputs gathered on every rank by the attention epilogue (peer stores over NVLink; checked against NCCL)"
    per_step = [total_ms / args.steps]
    # ---- end to end through the public API with host buffers: H2D of the step's inputs, append of the new
    # token, attention, D2H of the outputs
    # A serving loop overlaps the copies of neighbouring steps with the kernels: inputs and outputs are double
    # buffered, the host-to-device copy of step i + 1 and the device-to-host copy of step i - 1 run on their own
    # streams beside the kernels of step i. Every step still copies its own inputs in and its own result out.
    lens_dev = kv_len.clone()
    in_dev = [step_dev, torch.empty_like(step_dev)]
    out_dev = [out, torch.empty_like(out)]
    out_hosts = [out_host, torch.empty_like(out_host).pin_memory()]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def e2e_steps(first, count):
        """Steps first .. first + count - 1 as a three-stage pipeline over the current stream and two copy streams."""
        main = torch.cuda.current_stream(dev)
        fork = torch.cuda.Event()
        fork.record(main)
        s_in.wait_event(fork)
        s_out.wait_event(fork)
        ev_in, ev_done, ev_out = {}, {}, {}
        for i in range(first, first + count):
            pb = i & 1
            kc, vc = caches[i % nbuf]
            qv = in_dev[pb][:nq].view(b, hq, 1, d)
            kn = in_dev[pb][nq:nq + nkv].view(b, hkv, 1, d)
            vn = in_dev[pb][nq + nkv:].view(b, hkv, 1, d)
            with torch.cuda.stream(s_in):
                if i - 2 in ev_done:
                    s_in.wait_event(ev_done[i - 2])       # the kernels of step i - 2 have read this input buffer
                in_dev[pb].copy_(step_host, non_blocking=True)
                ev_in[i] = torch.cuda.Event()
                ev_in[i].record(s_in)
            main.wait_event(ev_in[i])
            if i - 2 in ev_out:
                main.wait_event(ev_out[i - 2])            # the result of step i - 2 has left this output buffer
            # the device lengths are those at the start of this group of steps: step j appends at lens + j and attends
            # to lens + j + 1 keys (offsets in the call arguments), so no kernel sits between append and attention
            j = i - first
            _kv_append(kn, vn, kc, vc, kq, vq, lens_dev, pos_add=j)
            P.PackedAttention(qv, kc, vc, lens_dev, kq, vq, cfg, out=out_dev[pb], gather=peer_gather, kv_len_add=j + 1,
                              after_prev=True, fresh_rows=1).run()
            if world > 1 and peer_gather is None:
                dist.all_gather_into_tensor(gathered, out_dev[pb])
            ev_done[i] = torch.cuda.Event()
            ev_done[i].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[i])
                out_hosts[pb].copy_(out_dev[pb], non_blocking=True)
                ev_out[i] = torch.cuda.Event()
                ev_out[i].record(s_out)
        lens_dev.add_(count)                              # one length update per group of steps
        last = first + count - 1
        main.wait_event(ev_in[last])
        main.wait_event(ev_out[last])
        if last - 1 in ev_out:
            main.wait_event(ev_out[last - 1])

    e2e_steps(0, max(min(args.warmup, 3), nbuf))
    barrier()
    # the same calls captured once (copies and stream dependencies included): a serving loop replays its steps instead
    # of paying the host's call path every token
    e2e_group = nbuf * max(1, 8 // nbuf)
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
    barrier()
    e0.record()
    i = 0
    while i < args.steps:
        if e2e_graph is not None and args.steps - i >= e2e_group:
            e2e_graph.replay()
            i += e2e_group
        else:
            e2e_steps(i, 1)
            i += 1
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    e2e_graph = None
    stage("end-to-end region done")
    # max over ranks of the times, sum over ranks of the bytes
    (total_ms, e2e_ms, kern_ms), job_bytes = aggregate_over_ranks(
        [total_ms, e2e_ms, float(np.mean(per_step))], algorithmic_bytes(w, lens), world, dev)
    # the timed regions last milliseconds: keep the same step running (untimed) until the clock sampler has seen
    # about half a second of this load. Every rank runs the same number of steps (they hold a collective).
    extra = clock_sample_steps(total_ms / args.steps)
    for i in range(0, extra, 256):
        run_steps(min(256, extra - i))
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    stage("clock sampling done")
    if rank == 0:
        peaks = {}
        try:
            peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        except OSError:
            pass
        peak, peak_kind = (peaks["hbm_gbs"], "measured copy bandwidth (MEASURED_PEAKS.json)") if "hbm_gbs" in peaks else (6650.0, "fallback")
        ms = total_ms / args.steps
        value = job_bytes / (ms * 1e-3) / 1e9
        rank_bytes = algorithmic_bytes(w, lens)
        achieved = rank_bytes / (kern_ms * 1e-3) / 1e9
        cpu = None
        if world == 1 or rank == 0:
            nseq = min(b, 8 if w["lens"] == "uniform512-8192" else max(1, 65536 // int(lens[0])))
            from oracle import oracle as O
            cpu_reference_step(w, lens, min(2, nseq))
            dt, cb = cpu_reference_step(w, lens, nseq)
            cpu = {"value": cb / dt / 1e9, "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
                   "sample": f"{nseq} of {b} sequences, one pass ({dt:.2f} s): dequantize rows to {w['qdt']} + unfused attention"}
        # the decode grid, the combine grid, and with N > 1 the one-warp kernel that publishes the gathered step
        launches_per_step = 2 + (1 if (peer_gather is not None and world > 1) else 0)
        # dram__bytes_read.sum + dram__bytes_write.sum of one tq_decode_kernel launch, from the ncu capture of this same
        # workload (profiles/tq_decode_kernel_c2_mxfp4.md): 360.75 MB read + 7.54 MB written
        traffic, traffic_src = None, None
        if args.workload == "c2" and not args.uniform_len and world == 1:
            traffic, traffic_src = 368_288_000, "ncu capture of this workload, profiles/tq_decode_kernel_c2_mxfp4.md"
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 mma / f32 softmax",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: {w['desc']}", "batch_per_gpu": b, "hq": hq, "hkv": hkv, "head_dim": d,
                       "kv_format": w["fmt"], "rotation": w["rot"], "total_keys_per_gpu": int(lens.sum()),
                       "launch": (f"CUDA graph replay ({group} steps per graph)" if graphs else "eager C ABI calls") + ", attention launched as a programmatic dependent of the previous kernel (B200_TQ_AFTER_PREV)",
                       "l2": f"{nbuf} caches of {cache_bytes / 1e6:.0f} MB cycled (each step reads other rows than the last; L2 is 126 MB)",
                       "parallelism": f"batch shard x{world}, {gather_note}" if world > 1 else "single GPU"},
            "tokens_per_s": world * b / (ms * 1e-3),
            "pct_of_8000_gbs_nominal": 100.0 * value / (8000.0 * world),
            "e2e": {"value": job_bytes / (e2e_ms / args.steps * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": int(q_host.numel() + knew_host.numel() + vnew_host.numel()) * 2,
                    "d2h_bytes_per_step": int(out_host.numel()) * 2, "ms_per_step": e2e_ms / args.steps,
                    "tokens_per_s": world * b / (e2e_ms / args.steps * 1e-3)},
            "gpu_launches": args.steps * launches_per_step,
            "roofline": {"bound": "hbm", "kernel": "tq_decode_kernel (+ the combine kernel in the same timed call)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_kind, "traffic": traffic, "traffic_unit": "bytes per launch",
                         "traffic_source": traffic_src},
            "cpu_baseline": cpu, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # The captured graphs hold NCCL kernels of this communicator: release them, drain the device and meet the
        # other ranks before the communicator goes. The teardown itself runs beside a deadline, so that a rank
        # whose peers are already gone still exits.
        graphs.clear()
        long_graph = None
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        stage("tearing down the process group")
        th = threading.Thread(target=dist.destroy_process_group, daemon=True)
        th.start()
        th.join(timeout=20.0)
        sys.stdout.flush()
        sys.stderr.flush()
        # leave without the interpreter's own teardown of CUDA and NCCL objects, which can wait on a peer that is gone
        os._exit(0)


def run_prefill(args, rank, world, local_rank):
    """Workload c3: causal prefill of B=4 x S=4096 (Hq 32, Hkv 8, D 128, bf16) with the new K / V written into an
    NVFP4 cache in the same call. Metric: attention TFLOP/s (4 B Hq S^2 D / 2 flop per step); single GPU."""
    import torch

    import __graft_entry__ as G

    if args.impl == "reference" or rank != 0:
        if rank == 0:
            cpu, flops = cpu_prefill_sample()
            print(json.dumps({"impl": "reference", "metric": "prefill_attention_tflops", "value": cpu["value"], "unit": "TFLOP/s",
                              "n_gpus": args.gpus, "steps": 1, "warmup": 0, "higher_is_better": True, "config": {"workload": "c3 (sample)"},
                              "cpu_baseline": cpu, "e2e": {"value": cpu["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}),
                  flush=True)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    G.build()
    P = G.load_package()
    F = P.flash_attn
    b, s, hq, hkv, d = 4, 4096, 32, 8, 128
    nv = P.QuantFormat.parse("nvfp4")
    kq, vq = P.TurboQuantizer(nv, d, "none", 42, dev), P.TurboQuantizer(nv, d, "none", 44, dev)
    cfg = P.FlashAttnConfig(d ** -0.5).causal()
    nbuf = 3  # q/k/v/out sets cycled: 3 x 335 MB, so that no step finds its inputs in L2
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

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    # attention alone (the dominant kernel), for the roofline
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for i in range(args.steps):
        q, k, v = sets[i % nbuf]
        F.flash_attn_with_config(q, k, v, cfg)
    a1.record()
    torch.cuda.synchronize()
    attn_ms = a0.elapsed_time(a1) / args.steps
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
    torch.cuda.synchronize()
    n_e2e = max(2, min(args.steps, 5))
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / n_e2e
    for i in range(clock_sample_steps(ms, seconds=0.5, cap=400)):
        step(i)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    if P._abi.lib().b200_device_wait_status() != 0:
        raise SystemExit("bench: a bounded device wait ran out; the numbers are void")
    flops = 4.0 * b * hq * s * s * d / 2
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except OSError:
        pass
    peak, kind = (peaks["bf16_tflops"], "measured cuBLAS bf16 burst (MEASURED_PEAKS.json)") if "bf16_tflops" in peaks else (1590.0, "fallback")
    cpu, _ = cpu_prefill_sample()
    line = {"metric": "prefill_attention_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 mma / f32 softmax", "data": "synthetic",
            "config": {"workload": "c3: causal prefill B=4 S=4096 Hq=32 Hkv=8 D=128 bf16 + NVFP4 cache append",
                       "l2": f"{nbuf} input sets of 335 MB cycled (L2 is 126 MB)", "parallelism": "single GPU"},
            "tokens_per_s": b * s / (ms * 1e-3),
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(sum(t.numel() for t in sets[0])) * 2, "d2h_bytes_per_step": int(out_host.numel()) * 2},
            "gpu_launches": args.steps * 2,  # the attention kernel and the quantize-on-append kernel (K and V in one grid)
            "roofline": {"bound": "tensor", "kernel": "fa_prefill_sm100_kernel2 (attention alone)", "achieved": flops / (attn_ms * 1e-3) / 1e12,
                         "peak": peak, "unit": "TFLOP/s", "frac": flops / (attn_ms * 1e-3) / 1e12 / peak, "peak_source": kind,
                         # dram read + write of one launch at B = 1 (50.4 + 3.0 MB, part of q / k / v still in L2 from the
                         # call before), times the 4 batch entries of c3, whose blocks do not share data
                         "traffic": 4 * 53_400_000, "traffic_unit": "bytes per launch",
                         "traffic_source": "ncu capture at B=1 scaled by 4, profiles/fa_prefill_sm100_kernel2_b1_s4096.md"},
            "cpu_baseline": cpu, "clocks": clocks}
    print(json.dumps(line), flush=True)


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c3"])
    ap.add_argument("--verbose", action="store_true", help="print stage markers to stderr")
    ap.add_argument("--uniform-len", type=int, default=0, help="give every sequence this many keys (diagnostic)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "c3":
        return run_prefill(args, rank, world, local_rank)
    w = dict(WORKLOADS[args.workload])
    if args.uniform_len:
        w["lens"] = args.uniform_len
        w["desc"] += f" [every sequence {args.uniform_len} keys]"
    if args.impl == "reference":
        run_reference(args, w, rank, world)
    else:
        run_ours(args, w, rank, world, local_rank)


if __name__ == "__main__":
    main()
