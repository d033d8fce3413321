"""Tensor-parallel NVFP4 linear on real GPUs: one process per GPU, NCCL
all-gather of the output slices.  Skipped with fewer than two GPUs.

The ranks run with NVLS and symmetric-memory multicast off (the kernels use plain
peer stores), a short process-group timeout, and bounded device-side waits, so a
rank that fails ends every rank on its own error path."""
import datetime
import os
import socket
import sys

import numpy as np
import pytest

from conftest import ROOT, REL_L2_TOL

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _init(rank, world, port):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))
    return torch, dist


def _worker(rank, world, port, cases, out_dir, mode):
    torch, dist = _init(rank, world, port)
    import mimfer_b200 as mm
    from mimfer_b200.tp import TpLinear
    rt = mm.Runtime.get(rank)
    for i, (M, K, N) in enumerate(cases):
        w = mm.make_weight(N, K, seed=i)
        lin = TpLinear(w, rank, world, rt=rt, mode=mode, push_rows=128)   # push mode: several row chunks
        x = rt.to_device_bf16(mm.make_activations(M, K, seed=100 + i))
        y = lin.forward(x, barrier=(i % 2 == 0))      # odd cases: barrier issued separately
        if i % 2:
            lin.barrier()
        rt.sync()
        assert rt.device_status() == 0
        np.save(os.path.join(out_dir, f"y{i}_{rank}.npy"), rt.from_device_bf16(y))
    if mode != "fused":
        dist.barrier()
        dist.destroy_process_group()
        return
    # the same linears as one captured step: refill the activations in place, replay
    from mimfer_b200.tp import TpStep
    M, K, N = cases[1]
    lins = [TpLinear(mm.make_weight(N, K, seed=40 + j), rank, world, rt=rt, mode=mode) for j in range(2)]
    xs = [rt.to_device_bf16(mm.make_activations(M, K, seed=1)) for _ in range(2)]
    step = TpStep(lins, xs)
    for j in range(2):
        xs[j].copy_(rt.to_device_bf16(mm.make_activations(M, K, seed=60 + j)))
    torch.cuda.synchronize()
    ys = step.replay()
    rt.sync()
    assert rt.device_status() == 0
    for j in range(2):
        np.save(os.path.join(out_dir, f"g{j}_{rank}.npy"), rt.from_device_bf16(ys[j]))
    dist.barrier()
    dist.destroy_process_group()


def _spawn_bounded(fn, args, world, limit_s=150, grace_s=90):
    """mp.spawn with a deadline.  Every wait of a rank is bounded (device-side waits give up
    after two seconds, the process group after sixty), so ranks end by themselves; past the
    deadline the test fails and gives them `grace_s` more to do so before asking the ones
    still alive to terminate."""
    import time
    import torch.multiprocessing as mp
    ctx = mp.spawn(fn, args=args, nprocs=world, join=False)
    deadline = time.time() + limit_s
    while True:
        try:
            if ctx.join(timeout=5):
                return
        except Exception as e:                      # a rank raised: the others follow on their own
            late = time.time() + grace_s
            while any(p.is_alive() for p in ctx.processes) and time.time() < late:
                time.sleep(1)
            pytest.fail(f"a rank failed: {e}")
        if time.time() > deadline:
            late = time.time() + grace_s
            while any(p.is_alive() for p in ctx.processes) and time.time() < late:
                time.sleep(1)
            for p in ctx.processes:
                if p.is_alive():
                    p.terminate()
            pytest.fail(f"ranks still running after {limit_s} s")


@pytest.mark.parametrize("mode", ["gather", "fused", "push"])
def test_two_gpu_tensor_parallel_matches_oracle(tmp_path, oracle, lib, mode):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import mimfer_b200 as mm
    from conftest import row_rel_l2
    # decode, decode, prefill kernel, prefill in several row chunks (push mode: 128 rows each, ragged tail)
    cases = [(1, 1024, 512), (32, 2048, 1024), (300, 512, 1040), (1100, 256, 4112)]
    world = 2
    _spawn_bounded(_worker, (world, _free_port(), cases, str(tmp_path), mode), world)
    for i, (M, K, N) in enumerate(cases):
        w = mm.make_weight(N, K, seed=i)
        x = mm.make_activations(M, K, seed=100 + i)
        want = oracle.gemm_f4(x, w.payload, w.scales, w.gs)
        ys = [np.load(tmp_path / f"y{i}_{r}.npy") for r in range(world)]
        assert np.array_equal(ys[0], ys[1])                          # every rank holds the full output
        assert row_rel_l2(ys[0], want) <= REL_L2_TOL
    M, K, N = cases[1]
    for j in range(2 if mode == "fused" else 0):                     # the captured step
        w = mm.make_weight(N, K, seed=40 + j)
        want = oracle.gemm_f4(mm.make_activations(M, K, seed=60 + j), w.payload, w.scales, w.gs)
        gs = [np.load(tmp_path / f"g{j}_{r}.npy") for r in range(world)]
        assert np.array_equal(gs[0], gs[1])
        assert row_rel_l2(gs[0], want) <= REL_L2_TOL


def _hazard_worker(rank, world, port, out_dir, captured):
    """Four steps on changing activations.  Rank 1 is slow to read: after every step's barrier
    it sleeps on its stream before copying the output away, while rank 0 goes straight on to
    the next step and stores that step's tiles into rank 1's memory."""
    torch, dist = _init(rank, world, port)
    import mimfer_b200 as mm
    from mimfer_b200.tp import TpLinear, TpStep
    rt = mm.Runtime.get(rank)
    M, K, N = 16, 1024, 2048
    lin = TpLinear(mm.make_weight(N, K, seed=7), rank, world, rt=rt, mode="fused")
    x = rt.to_device_bf16(mm.make_activations(M, K, seed=300))
    feeds = [rt.to_device_bf16(mm.make_activations(M, K, seed=300 + s)) for s in range(4)]
    torch.cuda.synchronize()
    step = TpStep([lin], [x]) if captured else None
    stream = rt.torch_stream()
    kept = []
    for s in range(4):
        with torch.cuda.stream(stream):
            x.copy_(feeds[s], non_blocking=True)
        if captured:
            y = step.replay()[0]
        else:
            y = lin.forward(x, barrier=True)
        with torch.cuda.stream(stream):
            if rank == 1:
                torch.cuda._sleep(int(60e6))           # tens of milliseconds: rank 0 is a step ahead by then
            kept.append(y.clone())
    rt.sync()
    assert rt.device_status() == 0
    for s, t in enumerate(kept):
        np.save(os.path.join(out_dir, f"h{s}_{rank}.npy"), rt.from_device_bf16(t))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("captured", [False, True])
def test_rank_that_runs_ahead_does_not_overwrite_a_slow_readers_output(tmp_path, oracle, lib, captured):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import mimfer_b200 as mm
    from conftest import row_rel_l2
    world = 2
    _spawn_bounded(_hazard_worker, (world, _free_port(), str(tmp_path), captured), world)
    M, K, N = 16, 1024, 2048
    w = mm.make_weight(N, K, seed=7)
    for s in range(4):
        want = oracle.gemm_f4(mm.make_activations(M, K, seed=300 + s), w.payload, w.scales, w.gs)
        for r in range(world):
            got = np.load(tmp_path / f"h{s}_{r}.npy")
            assert row_rel_l2(got, want) <= REL_L2_TOL, (s, r)


GROUP_CASES = [(1, 1024, 512), (16, 2048, 1024), (5, 512, 2064)]


def _group_worker(rank, world, port, out_dir):
    """Three decode linears of one step as one group launch per rank (TpGroupStep), replayed
    three times on changing activations; every rank saves its copy of every output."""
    torch, dist = _init(rank, world, port)
    import mimfer_b200 as mm
    from mimfer_b200.tp import TpGroupStep
    rt = mm.Runtime.get(rank)
    ws = [mm.make_weight(N, K, seed=20 + i) for i, (M, K, N) in enumerate(GROUP_CASES)]
    xs = [rt.to_device_bf16(mm.make_activations(M, K, seed=1)) for (M, K, N) in GROUP_CASES]
    feeds = [[rt.to_device_bf16(mm.make_activations(M, K, seed=400 + 10 * s + i))
              for i, (M, K, N) in enumerate(GROUP_CASES)] for s in range(3)]
    torch.cuda.synchronize()
    step = TpGroupStep(ws, xs, rank, world, rt)
    assert step.engines[0].n_group_launches() == 1
    stream = rt.torch_stream()
    for s in range(3):
        with torch.cuda.stream(stream):
            for x, f in zip(xs, feeds[s]):
                x.copy_(f, non_blocking=True)
        ys = step.replay()
        rt.sync()
        assert rt.device_status() == 0
        for i, y in enumerate(ys):
            np.save(os.path.join(out_dir, f"s{s}_{i}_{rank}.npy"), rt.from_device_bf16(y))
    step.close()
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_group_step_matches_oracle(tmp_path, oracle, lib):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import mimfer_b200 as mm
    from conftest import row_rel_l2
    world = 2
    _spawn_bounded(_group_worker, (world, _free_port(), str(tmp_path)), world)
    for s in range(3):
        for i, (M, K, N) in enumerate(GROUP_CASES):
            w = mm.make_weight(N, K, seed=20 + i)
            want = oracle.gemm_f4(mm.make_activations(M, K, seed=400 + 10 * s + i), w.payload, w.scales, w.gs)
            got = [np.load(tmp_path / f"s{s}_{i}_{r}.npy") for r in range(world)]
            assert np.array_equal(got[0], got[1])
            assert row_rel_l2(got[0], want) <= REL_L2_TOL, (s, i)
