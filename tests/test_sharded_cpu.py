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


def _host_runner_worker(rank, world, port, m, n, gs, b, q):
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
        k = 128
        A, R, B = make_oft_case(m, n, k, b, gs, seed=2)
        n0, n1 = sharded.my_slab(n, gs, lib=ops.load_library())
        calls = []

        def compute(m_, n_loc, k_, A_, ldA, B_, ldB, R_, ldR, C_, ldC, stream, group_size, reconn_sz):
            calls.append(m_)
            out = oracle.cpu_oft_tn(A_[:m_].numpy().view(np.float16), R_.numpy().view(np.float16), B_.numpy().view(np.float16),
                                    m_, group_size, n_loc // group_size, k_, reconn_sz)
            C_[:m_] = torch.from_numpy(out)

        runner = sharded.HostSlabRunner(m, n, k, n0, n1, group_size=gs, reconn_sz=b, device="cpu", compute=compute, chunks=2)
        r0, r1 = sharded.row_slice(m, world, rank)
        G_first = n0 // gs if gs < n else 0
        R_slab = R[G_first * b: G_first * b + runner.r_rows]
        hY = torch.zeros((m, n1 - n0), dtype=torch.float16)
        runner(torch.from_numpy(A[r0:r1]), torch.from_numpy(B[n0:n1]), torch.from_numpy(R_slab), hY)  # this rank only supplies ITS rows of X
        full = oracle.cpu_oft_tn(A, R, B, m, gs, n // gs, k, b)
        ok = np.array_equal(hY.numpy().view(np.uint16), full[:, n0:n1].view(np.uint16))
        h2d, d2h = runner.bytes_per_step()
        q.put((rank, bool(ok), (r0, r1), len(calls), h2d, d2h))
    except Exception as e:
        q.put((rank, repr(e), None, 0, 0, 0))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m,n,gs,b", [(512, 512, 512, 32), (300, 512, 256, 16)])
def test_two_rank_host_runner_uploads_x_once_and_matches(m, n, gs, b):
    """HostSlabRunner over gloo: each rank supplies only its rows of X, the all-gather rebuilds X on every rank
    (also when M is not a multiple of the world size), the chunked slab product equals the unsharded oracle."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_host_runner_worker, args=(r, 2, port, m, n, gs, b, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=90) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    results.sort()
    assert all(r[1] is True for r in results), results
    assert [r[2] for r in results] == [(0, (m + 1) // 2), ((m + 1) // 2, m)]
    assert all(r[3] == 2 for r in results)  # two row chunks per rank
    r_rows_total = (n // gs) * b if gs < n else 2 * b  # one group: both ranks hold the whole R
    assert sum(r[4] for r in results) == (m * 128 + n * 128 + r_rows_total * 128) * 2  # X crosses the host link once
    assert sum(r[5] for r in results) == m * n * 2
