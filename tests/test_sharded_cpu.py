"""CPU, world_size 2 over gloo: the N-sharded path (slab arithmetic, per-rank call, optional all-gather
layout) with the oracle standing in for the GPU kernel as the per-rank compute."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, gs, b, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist

    from _util import make_oft_case
    from cute_mma_b200 import ops, sharded
    from oracle import oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, k = 24, 128
        A, R, B = make_oft_case(m, n, k, b, gs, seed=1)  # every rank builds the same full problem
        n0, n1 = sharded.my_slab(n, gs, lib=ops.load_library())
        G_first = n0 // gs if gs < n else 0
        c_local = np.zeros((m, n1 - n0), np.float16)

        def compute(m_, n_loc, k_, A_, ldA, B_, ldB, R_, ldR, C_, ldC, stream, group_size, reconn_sz):
            C_[:] = oracle.cpu_oft_tn(A_, R_, B_, m_, group_size, n_loc // group_size, k_, reconn_sz)

        R_slab = R[G_first * b:] if gs < n else R
        sharded.oft_tn_slab(m, n, k, A, k, B[n0:n1], k, R_slab[: max(1, (n1 - n0) // gs) * b], k, c_local, n1 - n0, n0, n1,
                            group_size=gs, reconn_sz=b, compute=compute)
        full = oracle.cpu_oft_tn(A, R, B, m, gs, n // gs, k, b)
        ok_local = np.array_equal(c_local.view(np.uint16), full[:, n0:n1].view(np.uint16))
        gathered = sharded.all_gather_c(torch.from_numpy(c_local.view(np.uint8)), world).numpy().view(np.float16)
        # rank-major [world][m][n_loc] -> [m][n]
        rebuilt = np.concatenate([gathered[r] for r in range(world)], axis=1)
        ok_gather = np.array_equal(rebuilt.view(np.uint16), full.view(np.uint16))
        q.put((rank, (n0, n1), bool(ok_local), bool(ok_gather)))
    except Exception as e:  # report instead of leaving the parent waiting for its timeout
        q.put((rank, repr(e), False, False))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n,gs,b", [(512, 512, 32), (512, 256, 16)])
def test_two_rank_sharded_product_matches_unsharded(n, gs, b):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n, gs, b, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=90) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    results.sort()
    assert [r[1] for r in results] == [(0, n // 2), (n // 2, n)]
    assert all(r[2] and r[3] for r in results), results
