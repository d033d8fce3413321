"""Tensor-parallel sharding and the all-gather layout, on CPU: world_size 2
over gloo.  The local op is the oracle here (the test's checker standing in
for the GPU kernel), so what is under test is the shard bounds, the gather and
the [tp][M][N/tp] -> [M][N] re-layout."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, M, K, N, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import mimfer_b200 as mm
    from mimfer_b200.tp import TpLinear
    from oracle.pyoracle import Oracle
    orc = Oracle()
    w = mm.make_weight(N, K, seed=0)
    x_bits = mm.make_activations(M, K, seed=1)

    def local_op(x, shard, y):
        bits = orc.gemm_f4(x.view(torch.int16).numpy().view(np.uint16), shard.payload, shard.scales,
                           shard.gs, threads=1)
        y.copy_(torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16))

    lin = TpLinear(w, rank, world, local_op=local_op)
    assert lin.shard.N == N // world and lin.shard.payload.shape == (N // world, K // 2)
    x = torch.from_numpy(x_bits.view(np.int16)).view(torch.bfloat16)
    y = lin.forward(x)
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y.view(torch.int16).numpy().view(np.uint16))
    dist.destroy_process_group()


@pytest.mark.parametrize("M", [1, 5])
def test_two_rank_all_gather_matches_single_rank(tmp_path, oracle, lib, M):
    import mimfer_b200 as mm
    K, N, world = 256, 96, 2
    mp.spawn(_worker, args=(world, _free_port(), M, K, N, str(tmp_path)), nprocs=world, join=True)
    w = mm.make_weight(N, K, seed=0)
    x = mm.make_activations(M, K, seed=1)
    want = oracle.gemm_f4(x, w.payload, w.scales, w.gs)
    for r in range(world):
        assert np.array_equal(np.load(tmp_path / f"y{r}.npy"), want)


def test_shard_bounds():
    from mimfer_b200.tp import shard_bounds
    assert shard_bounds(151936, 3, 8) == (56976, 75968)
    assert [shard_bounds(34816, r, 4) for r in range(4)] == [(0, 8704), (8704, 17408), (17408, 26112), (26112, 34816)]
    with pytest.raises(ValueError):
        shard_bounds(100, 0, 8)


def test_push_chunks_cover_the_rows_once_and_end_on_a_short_chunk():
    """Row chunks of the copy-engine form of the exchange: every row once, in order, chunks of
    the asked size, the last whole chunk halved so that little is left to push at the end."""
    from mimfer_b200.tp import push_chunks
    for M in (1, 32, 300, 512, 1024, 1100, 2048, 8192):
        for rows in (128, 512, 1024):
            chunks = push_chunks(M, rows)
            assert chunks[0][0] == 0 and sum(n for _, n in chunks) == M
            assert all(a + n == b for (a, n), (b, _) in zip(chunks, chunks[1:]))
            assert all(0 < n <= rows for _, n in chunks)
    assert push_chunks(8192, 1024)[-2:] == [(7168, 512), (7680, 512)]
    assert push_chunks(1100, 128)[-1] == (1024, 76)


def test_tensor_parallel_modes_are_checked():
    import mimfer_b200 as mm
    from mimfer_b200.tp import TpLinear
    w = mm.make_weight(64, 64, seed=0)
    with pytest.raises(ValueError):
        TpLinear(w, 0, 1, local_op=lambda x, s, y: None, mode="scatter")
    with pytest.raises(ValueError):
        TpLinear(w, 0, 1, local_op=lambda x, s, y: None, mode="push", push_rows=0)
