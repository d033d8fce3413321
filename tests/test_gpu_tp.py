"""Tensor-parallel NVFP4 linear on real GPUs: one process per GPU, NCCL
all-gather of the output slices.  Skipped with fewer than two GPUs."""
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


def _worker(rank, world, port, cases, out_dir, mode):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import mimfer_b200 as mm
    from mimfer_b200.tp import TpLinear
    rt = mm.Runtime.get(rank)
    for i, (M, K, N) in enumerate(cases):
        w = mm.make_weight(N, K, seed=i)
        lin = TpLinear(w, rank, world, rt=rt, mode=mode)
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


def _spawn_bounded(fn, args, world, limit_s=150):
    """mp.spawn with a deadline: ranks that wait on each other forever are killed
    and the test fails, instead of holding the GPUs until the outer limit."""
    import time
    import torch.multiprocessing as mp
    ctx = mp.spawn(fn, args=args, nprocs=world, join=False)
    deadline = time.time() + limit_s
    while not ctx.join(timeout=5):
        if time.time() > deadline:
            for p in ctx.processes:
                p.kill()
            pytest.fail(f"ranks still running after {limit_s} s: killed")


@pytest.mark.parametrize("mode", ["gather", "fused"])
def test_two_gpu_tensor_parallel_matches_oracle(tmp_path, oracle, lib, mode):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import mimfer_b200 as mm
    from conftest import row_rel_l2
    cases = [(1, 1024, 512), (32, 2048, 1024), (300, 512, 1040)]    # decode, decode, prefill kernel
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
