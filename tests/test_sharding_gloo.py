"""The multi-rank work distribution, run as two CPU processes over gloo: the LPT batch assignment is
the same on every rank and covers every problem once, and the row-block gather reassembles C.
The per-rank SpMM itself is replaced by the CPU oracle here (this is a test of the distribution
logic, not of the kernels; the GPU path is covered by the gpu-marked tests and by bench.py)."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import __graft_entry__ as entry
    from cases import csr_rowlen_normal, dense

    pkg = entry.load_package()
    oracle = entry.load_oracle()
    import importlib

    sharding = importlib.import_module(entry.PKG_NAME + ".sharding")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)

    # (a) batch: every rank derives the same assignment; together they cover each problem once
    weights = np.array([float(pkg.rand_u64(7, 1, i) % 1000 + 1) for i in range(101)])
    mine = sharding.my_problems(pkg, weights, rank, world)
    flags = torch.zeros(101, dtype=torch.int32)
    flags[torch.from_numpy(mine)] = 1
    dist.all_reduce(flags)
    assert bool((flags == 1).all()), "every problem must be owned by exactly one rank"
    load = torch.tensor([weights[mine].sum()], dtype=torch.float64)
    loads = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(loads, load)
    loads = np.array([float(x) for x in loads])
    assert loads.max() <= weights.sum() / world + weights.max()

    # (b) one SpMM, rows sharded by nonzero count, blocks gathered on every rank
    M, K, N = 300, 80, 24
    ro, ci = csr_rowlen_normal(pkg, M, K, 0.8, 5)
    vals = pkg.gen_dense_host(int(ci.size), 5, 2)
    B = dense(pkg, K, N, 5, 10)
    r0, r1, bounds = sharding.row_block(pkg, ro, rank, world)
    local_ro = sharding.rebase_offsets(ro, r0, r1)
    lo, hi = int(ro[r0]), int(ro[r1])
    c_local = oracle.spmm(vals[lo:hi], local_ro, ci[lo:hi], B, r1 - r0, N)
    full = sharding.gather_row_blocks(torch.from_numpy(c_local), bounds, N).numpy()
    ref = oracle.spmm(vals, ro, ci, B, M, N)
    assert full.shape == (M, N)
    assert np.array_equal(full.view(np.uint32), ref.view(np.uint32))
    nnz_per = np.diff(ro[bounds])
    assert nnz_per.max() - nnz_per.min() <= 2 * np.diff(ro).max()
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(result_dir, f"ok{rank}"), "w").write("ok")


@pytest.mark.parametrize("world", [2, 3])
def test_sharding_over_gloo(world, tmp_path):
    import torch.multiprocessing as mp

    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"ok{r}").exists()
