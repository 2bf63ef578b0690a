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


def row_slice(m: int, world: int, rank: int) -> tuple[int, int]:
    """Rows of X that rank uploads in HostSlabRunner: equal slices of ceil(m / world) rows (the last ones may be
    short or empty), so that the all-gather of the slices is one contiguous collective."""
    per = (m + world - 1) // world
    r0 = min(m, rank * per)
    return r0, min(m, r0 + per)


class HostSlabRunner:
    """End-to-end N-sharded product from HOST buffers on the ranks of one node.

    Every rank needs all of X, but X crosses the host link only once per node: rank r uploads rows
    row_slice(m, world, r) of X from its (pinned) host buffer and the slices are all-gathered over NVLink
    (torch.distributed, NCCL on GPUs).  The slice goes up in ``chunks`` row chunks; as soon as chunk j of every
    rank is gathered, the rank's slab product runs on those world x chunk rows and their [rows][n_loc] piece of Y
    goes back to host memory while later chunks are still uploading, gathering and multiplying (four streams:
    upload, collective, product, download).  The slab of W^T and R go up right behind the first chunk of X.
    Device buffers are allocated once per runner; rows are independent, so the chunking changes no bit.
    ``compute`` / ``device`` exist so that the data movement can be exercised on CPU ranks over gloo with the
    oracle standing in for the kernel."""

    def __init__(self, m, n_total, k, n0, n1, *, group_size=None, reconn_sz=8, world=None, rank=None, device=None, compute=None,
                 lib=None, chunks=8):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.world = world if world is not None else dist.get_world_size()
        self.rank = rank if rank is not None else dist.get_rank()
        self.m, self.n_total, self.k, self.n0, self.n1 = m, n_total, k, n0, n1
        self.n_loc = n1 - n0
        gs = n_total if group_size is None else group_size
        self.gs_loc = self.n_loc if gs >= n_total else gs
        self.b = reconn_sz
        self.r_rows = max(1, self.n_loc // self.gs_loc) * reconn_sz
        self.device = torch.device(device if device is not None else "cuda")
        self.compute, self.lib = compute, lib
        self.per = (m + self.world - 1) // self.world                 # rows of X per rank (the last slices may be short)
        self.pc = max(8, ((self.per + chunks - 1) // chunks + 7) // 8 * 8)  # rows per chunk of a rank's slice
        self.n_chunks = (self.per + self.pc - 1) // self.pc
        f16 = torch.float16
        self.dSend = torch.zeros((self.n_chunks, self.pc, k), dtype=f16, device=self.device)             # my slice, chunked, zero padded
        self.dX = torch.empty((self.n_chunks, self.world * self.pc, k), dtype=f16, device=self.device)   # gathered: [chunk][rank][row]
        self.dW = torch.empty((self.n_loc, k), dtype=f16, device=self.device)
        self.dR = torch.empty((self.r_rows, k), dtype=f16, device=self.device)
        self.dY = torch.empty((self.n_chunks, self.world * self.pc, self.n_loc), dtype=f16, device=self.device)
        self.cuda = self.device.type == "cuda"
        if self.cuda:
            self.s_in, self.s_comm, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))

    def bytes_per_step(self):
        """(host-to-device, device-to-host) bytes this rank moves per call."""
        r0, r1 = row_slice(self.m, self.world, self.rank)
        return ((r1 - r0) * self.k + self.n_loc * self.k + self.r_rows * self.k) * 2, self.m * self.n_loc * 2

    def _rows_of(self, r: int, j: int) -> int:
        """Valid rows of chunk j of rank r's slice."""
        rows_r = min(self.per, max(0, self.m - r * self.per))
        return min(self.pc, max(0, rows_r - j * self.pc))

    # the four legs, each on the stream the caller has made current
    def _upload_chunk(self, hX_rows, j):
        rows = self._rows_of(self.rank, j)
        if rows > 0:
            self.dSend[j, :rows].copy_(hX_rows[j * self.pc: j * self.pc + rows], non_blocking=True)

    def _gather_chunk(self, j):
        if self.world > 1:
            self.dist.all_gather_into_tensor(self.dX[j], self.dSend[j])
        else:
            self.dX[j].copy_(self.dSend[j])

    def _product_chunk(self, j):
        torch = self.torch
        fn = self.compute or ops.oft_tn
        kwargs = dict(group_size=self.gs_loc, reconn_sz=self.b)
        if self.compute is None:
            kwargs["lib"] = self.lib
        stream = torch.cuda.current_stream(self.device).cuda_stream if self.cuda else None
        rows = self.world * self.pc
        fn(rows, self.n_loc, self.k, self.dX[j], self.k, self.dW, self.k, self.dR, self.k, self.dY[j], self.n_loc, stream, **kwargs)

    def _download_chunk(self, hY_slab, j):
        for r in range(self.world):
            rows = self._rows_of(r, j)
            if rows > 0:
                g0 = r * self.per + j * self.pc
                hY_slab[g0: g0 + rows].copy_(self.dY[j, r * self.pc: r * self.pc + rows], non_blocking=True)

    def __call__(self, hX_rows, hW_slab, hR_slab, hY_slab):
        """hX_rows: this rank's rows row_slice(m, world, rank) of X [rows][k]; hW_slab [n_loc][k]; hR_slab
        [r_rows][k]; hY_slab [m][n_loc] (written).  Host tensors, pinned for asynchronous copies.  Returns when
        hY_slab is complete."""
        torch = self.torch
        if not self.cuda:
            self.dW.copy_(hW_slab)
            self.dR.copy_(hR_slab)
            for j in range(self.n_chunks):
                self._upload_chunk(hX_rows, j)
                self._gather_chunk(j)
                self._product_chunk(j)
                self._download_chunk(hY_slab, j)
            return
        main = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_comm, self.s_out):
            s.wait_stream(main)
        ev_w = torch.cuda.Event()
        for j in range(self.n_chunks):
            ev_up, ev_g, ev_p = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
            with torch.cuda.stream(self.s_in):
                self._upload_chunk(hX_rows, j)
                ev_up.record(self.s_in)
                if j == 0:  # W and R right behind the first rows of X: the first product needs all three
                    self.dW.copy_(hW_slab, non_blocking=True)
                    self.dR.copy_(hR_slab, non_blocking=True)
                    ev_w.record(self.s_in)
            with torch.cuda.stream(self.s_comm):
                self.s_comm.wait_event(ev_up)
                self._gather_chunk(j)
                ev_g.record(self.s_comm)
            main.wait_event(ev_g)
            if j == 0:
                main.wait_event(ev_w)
            self._product_chunk(j)
            ev_p.record(main)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_p)
                self._download_chunk(hY_slab, j)
        self.s_out.synchronize()
        main.synchronize()
        self.s_in.synchronize()
        self.s_comm.synchronize()

    def leg_times(self, hX_rows, hW_slab, hR_slab, hY_slab) -> dict:
        """Milliseconds of each leg of one call run on its own, back to back on one stream (no overlap): what the
        overlapped call is made of.  GPU ranks only."""
        import time

        torch = self.torch

        def timed(fn):
            if self.world > 1:
                self.dist.barrier()
            torch.cuda.synchronize(self.device)
            t0 = time.perf_counter()
            fn()
            torch.cuda.synchronize(self.device)
            return (time.perf_counter() - t0) * 1e3

        def upload():
            for j in range(self.n_chunks):
                self._upload_chunk(hX_rows, j)
            self.dW.copy_(hW_slab, non_blocking=True)
            self.dR.copy_(hR_slab, non_blocking=True)

        return {"h2d_x_slice_w_r": timed(upload),
                "all_gather_x": timed(lambda: [self._gather_chunk(j) for j in range(self.n_chunks)]),
                "products": timed(lambda: [self._product_chunk(j) for j in range(self.n_chunks)]),
                "d2h_y_slab": timed(lambda: [self._download_chunk(hY_slab, j) for j in range(self.n_chunks)])}


class SlabProductAllGather:
    """The rank's slab product with the all-gather of Y overlapped: when the call returns, every rank holds
    all of Y, rank-major [world][m][n_loc] (the layout of all_gather_c).

    mode "copy_engines": the product runs in row chunks on the compute stream; as soon as a chunk of the rank's slab is written, copy
    streams push it into the same place of every peer's buffer over NVLink (contiguous device-to-device copies,
    i.e. copy engines, no SMs and no kernel that waits for another GPU).  The peers' buffers are symmetric memory
    (torch.distributed._symmetric_memory), mapped once at construction.  A host barrier at the end of the call tells a rank that
    its peers' chunks have landed.  At 8 GPUs the exchange (7/8 of Y leaving every GPU) takes longer than the
    product, so the step costs about the exchange instead of product + exchange.
    mode "stores" (default): one launch whose epilogue writes every tile straight into all GPUs' buffers (the direct peer-store
    epilogue: each warp transposes its rows in registers and writes whole 128-byte lines).  At 8 GPUs this is the
    faster of the two (6.2 ms per step against 8.2 ms; the NCCL all-gather alone takes 7.8 ms)."""

    def __init__(self, m, n_total, k, n0, n1, *, reconn_sz=8, world=None, rank=None, device=None, lib=None, chunks=4, copy_streams=3,
                 mode="stores"):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        if mode not in ("copy_engines", "stores"):
            raise ValueError("mode is 'copy_engines' or 'stores'")
        self.mode = mode
        self.world = world if world is not None else dist.get_world_size()
        self.rank = rank if rank is not None else dist.get_rank()
        self.m, self.k, self.n_loc, self.b, self.lib = m, k, n1 - n0, reconn_sz, lib
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        if (n1 - n0) * self.world != n_total:
            raise ValueError("SlabProductAllGather needs equal slabs on every rank")
        # Buffers the peers can write: torch's symmetric memory (driver-level shareable allocations mapped into every
        # rank's address space).  Legacy CUDA IPC handles also map, but copies into them ran at 37 GB/s here
        # against 770 GB/s into symmetric memory.
        import torch.distributed._symmetric_memory as symm_mem

        self.y_all = symm_mem.empty((self.world, m, self.n_loc), dtype=torch.float16, device=self.device)
        self._handle = symm_mem.rendezvous(self.y_all, dist.group.WORLD)
        self.peer_views = [self.y_all if r == self.rank else self._handle.get_buffer(r, (self.world, m, self.n_loc), torch.float16)
                           for r in range(self.world)]
        self.copy_streams = [torch.cuda.Stream(self.device) for _ in range(copy_streams)]
        self.chunk_rows = max(256, ((m + chunks - 1) // chunks + 255) // 256 * 256)
        dist.barrier()

    def __call__(self, dX, dW_slab, dR):
        torch, dist = self.torch, self.dist
        main = torch.cuda.current_stream(self.device)
        mine = self.y_all[self.rank]
        if self.mode == "stores":
            # One launch: the kernel's epilogue stores every tile into this rank's place of every GPU's buffer (plain
            # global stores over NVLink into the peers' symmetric memory; ops.oft_tn_gather).
            dsts = [mine] + [self.peer_views[(self.rank + p) % self.world][self.rank] for p in range(1, self.world)]
            ops.oft_tn_gather(self.m, self.n_loc, self.k, dX, self.k, dW_slab, self.k, dR, self.k, dsts, self.n_loc, main.cuda_stream,
                              group_size=self.n_loc, reconn_sz=self.b, lib=self.lib)
            main.synchronize()
            if self.world > 1:
                dist.barrier()  # every peer's stores into this rank's buffer are complete
            return self.y_all
        for s in self.copy_streams:
            s.wait_stream(main)
        i = 0
        for c0 in range(0, self.m, self.chunk_rows):
            rows = min(self.chunk_rows, self.m - c0)
            ops.oft_tn(rows, self.n_loc, self.k, dX[c0:], self.k, dW_slab, self.k, dR, self.k, mine[c0:], self.n_loc, main.cuda_stream,
                       group_size=self.n_loc, reconn_sz=self.b, lib=self.lib)
            done = torch.cuda.Event()
            done.record(main)
            for p in range(1, self.world):  # start with the next rank so that the ranks do not all write to one peer at once
                peer = (self.rank + p) % self.world
                s = self.copy_streams[i % len(self.copy_streams)]
                i += 1
                s.wait_event(done)
                dst = self.peer_views[peer][self.rank, c0: c0 + rows]
                ops.peer_copy_async(dst, dst.device.index, mine[c0:], self.device.index, rows * self.n_loc * 2, s.cuda_stream, lib=self.lib)
        for s in self.copy_streams:
            s.synchronize()
        main.synchronize()
        if self.world > 1:
            dist.barrier()  # every peer's copies into this rank's buffer are complete
        return self.y_all
