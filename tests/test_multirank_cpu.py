"""The host logic of the multi-GPU benchmark path on two gloo ranks (CPU): every rank shards the
batch the same way the NCCL run does, the reductions give every rank the same totals, the number of
untimed steps (each holds a collective) is the same on all ranks, and the gathered outputs arrive in
rank order."""
import importlib.util
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _bench():
    spec = importlib.util.spec_from_file_location("bench", ROOT / "bench.py")
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    B = _bench()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = dict(B.WORKLOADS["c2"])
        lens = B.seq_lens(w, rank)
        mine = B.algorithmic_bytes(w, lens)
        times, total = B.aggregate_over_ranks([10.0 + rank, 5.0 - rank, 1.0], mine, world, torch.device("cpu"))
        steps = B.clock_sample_steps(times[0] / 100)
        out = torch.full((w["b"], 4), float(rank))
        gathered = torch.empty((world * w["b"], 4))
        dist.all_gather_into_tensor(gathered, out)
        q.put((rank, lens.tolist(), mine, times, total, steps, gathered[:: w["b"], 0].tolist()))
    finally:
        dist.destroy_process_group()


def test_two_ranks_agree_on_totals_and_step_counts():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, lens0, b0, t0, tot0, s0, g0), (r1, lens1, b1, t1, tot1, s1, g1) = res
    assert (r0, r1) == (0, 1)
    assert lens0 != lens1 and sorted(lens0) == sorted(lens1) and len(lens0) == 64  # own batch, same work (weak scaling)
    assert all(512 <= x <= 8192 for x in lens0 + lens1)
    assert t0 == t1 == [11.0, 5.0, 1.0]       # max over ranks
    assert tot0 == tot1 == float(b0 + b1)      # whole-job bytes
    assert s0 == s1                            # same number of collectives on every rank
    assert g0 == g1 == [0.0, 1.0]              # outputs assembled in rank order


def test_clock_sample_steps_is_bounded():
    B = _bench()
    assert B.clock_sample_steps(0.09) == 6666
    assert B.clock_sample_steps(1e-9) == 20000 and B.clock_sample_steps(1e6) == 50


def test_reference_arm_runs_on_rank_zero_only(capsys):
    B = _bench()

    class A:
        steps, warmup, gpus, workload = 1, 0, 2, "c1"
    B.run_reference(A, dict(B.WORKLOADS["c1"]), rank=1, world=2)
    assert capsys.readouterr().out == ""
