"""N-sharded OFT product over the GPUs of one node: one process per GPU (torch.distributed).

The reference is single-GPU.  The product shards with no exchange in the compute: rank r owns the
rows [n0, n1) of the stored B[n][k] (a contiguous slab of W^T) and the same columns of C; A and R
are replicated.  The only collective is the optional all-gather of C over NCCL, which callers that
need the whole C on every GPU request explicitly.
"""
from __future__ import annotations

from . import ops


def my_slab(n: int, group_size: int | None = None, world: int | None = None, rank: int | None = None, lib=None):
    """Column range of this rank, read from torch.distributed when world/rank are not given."""
    if world is None or rank is None:
        import torch.distributed as dist

        world, rank = dist.get_world_size(), dist.get_rank()
    return ops.shard_range(n, n if group_size is None else group_size, world, rank, lib=lib)


def oft_tn_slab(m, n_total, k, A, ldA, B_slab, ldB, R_slab, ldR, C_slab, ldC, n0, n1, stream=None, *,
                group_size=None, reconn_sz=8, compute=None, lib=None) -> None:
    """This rank's share of C = (A.R).B^T: columns [n0, n1).

    B_slab points at row n0 of B (or at a private [n1-n0][k] copy), C_slab at column n0 of C (ldC = n_total)
    or at a private [m][n1-n0] buffer (ldC = n1-n0).  R_slab points at the first stored R row of the
    slab's first group.  ``compute`` (default: the CUDA kernel) exists so that the partition logic can be
    exercised on CPU ranks."""
    n_loc = n1 - n0
    if n_loc <= 0:
        return
    gs = n_total if group_size is None else group_size
    gs_loc = n_loc if gs >= n_total else gs   # a single group spans the whole slab
    fn = compute or ops.oft_tn
    kwargs = dict(group_size=gs_loc, reconn_sz=reconn_sz)
    if compute is None:
        kwargs["lib"] = lib
    fn(m, n_loc, k, A, ldA, B_slab, ldB, R_slab, ldR, C_slab, ldC, stream, **kwargs)


def all_gather_c(c_local, world: int | None = None):
    """Optional exchange: gathers the ranks' [m][n_loc] slabs (equal n_loc) into a rank-major
    [world][m][n_loc] tensor on every rank (contiguous, so a plain NCCL all-gather)."""
    import torch
    import torch.distributed as dist

    world = world or dist.get_world_size()
    m, n_loc = c_local.shape
    out = torch.empty((world * m, n_loc), dtype=c_local.dtype, device=c_local.device)  # concatenation along dim 0
    dist.all_gather_into_tensor(out, c_local.contiguous())
    return out.view(world, m, n_loc)
