"""Column-block sharding of one large GEMM over the GPUs of a node.

The contraction needs no communication: rank r owns columns [col0, col0 + ncols) of
op(B) and of C, every rank holds all of A, and each rank runs an independent
m x ncols x k GEMM through the library's C ABI.  The only exchange step is optional:
reassembling the full C on every rank.  On GPUs that is fused into the GEMM: the full C
lives in symmetric memory (every rank maps every other rank's copy) and the epilogue of
the tensor-core kernel stores each finished chunk into all copies over NVLink
(`gemm_and_broadcast`, fp16); an all-gather of the column blocks (NCCL, or gloo for CPU
tensors) remains as the plain alternative.  The reference has no multi-device path
(device index hard-coded: src/gemm/benchmark.cc:54); this is new capability behind
the same GEMM call.

One process per GPU; torch.distributed provides the process group.
"""
from __future__ import annotations

import importlib
from dataclasses import dataclass

# the package re-exports a function called `gemm`; importing the submodule of that name must not hide it
_g = importlib.import_module(__package__)._bind_public()


@dataclass(frozen=True)
class ColumnShard:
    """Partition of the n columns of op(B)/C among `world` ranks."""
    n: int
    world: int
    rank: int
    align: int = 256

    @property
    def col0(self) -> int:
        return _g.shard_columns(self.n, self.world, self.rank, self.align)[0]

    @property
    def ncols(self) -> int:
        return _g.shard_columns(self.n, self.world, self.rank, self.align)[1]

    def block_of(self, rank: int) -> tuple[int, int]:
        return _g.shard_columns(self.n, self.world, rank, self.align)

    def blocks(self) -> list[tuple[int, int]]:
        return [self.block_of(r) for r in range(self.world)]

    # ---- operand placement -----------------------------------------------------------
    def b_window(self, transB: bool, k: int) -> dict:
        """Arguments for `gemm.fill` that generate this rank's block of B in place:
        a column window when B is stored k x n, a row window when stored n x k."""
        if transB:
            return dict(rows=self.ncols, cols=k, row0=self.col0, col0=0, total_rows=self.n)
        return dict(rows=k, cols=self.ncols, row0=0, col0=self.col0, total_rows=k)

    # ---- compute -----------------------------------------------------------------------
    def local_gemm(self, dtype, transA, transB, m, k, alpha, A, lda, B_block, ldb, beta, C_block, ldc,
                   kernelId=_g.KERNEL_AUTO, stream=None, col_begin: int = 0, col_count: int | None = None):
        """GEMM on this rank's block (or on columns [col_begin, col_begin + col_count) of it).
        B_block is this rank's part of B: k x ncols (ldb >= k) when transB is false, ncols x k
        (ldb >= ncols) when true; C_block is m x ncols."""
        cnt = self.ncols - col_begin if col_count is None else col_count
        if cnt <= 0:
            return
        esz = 4 if dtype in ("f32", _g.DTYPE_F32) else 2
        b_off = (col_begin if transB else col_begin * ldb) * esz
        c_off = col_begin * ldc * esz
        _g.gemm(dtype, transA, transB, m, cnt, k, alpha, A, lda, _g._addr(B_block) + b_off, ldb, beta,
                _g._addr(C_block) + c_off, ldc, kernelId, stream)

    # ---- exchange ------------------------------------------------------------------------
    def gather(self, C_block, C_full, m: int, group=None, col_begin: int = 0, col_count: int | None = None,
               async_op: bool = False):
        """All-gather columns [col_begin, col_begin + col_count) of every rank's block into the
        full column-major C (shape (n, m), leading dimension m).  All blocks must have the
        same width.  Works on any backend (NCCL for CUDA tensors, gloo for CPU tensors)."""
        import torch.distributed as dist
        widths = {nc for _, nc in self.blocks()}
        if len(widths) != 1:
            raise ValueError("gather needs equal column blocks; choose n divisible by world * align")
        cnt = self.ncols - col_begin if col_count is None else col_count
        outs = [C_full[c0 + col_begin:c0 + col_begin + cnt] for c0, _ in self.blocks()]
        src = C_block[col_begin:col_begin + cnt]
        if cnt == self.ncols and col_begin == 0 and C_full.is_contiguous():
            return dist.all_gather_into_tensor(C_full.view(-1), src.reshape(-1), group=group, async_op=async_op)
        return dist.all_gather(outs, src.contiguous(), group=group, async_op=async_op)

    def gemm_and_gather(self, dtype, transA, transB, m, k, alpha, A, lda, B_block, ldb, beta, C_block, C_full,
                        panels: int = 4, kernelId=_g.KERNEL_AUTO, group=None):
        """Local GEMM in `panels` column panels; the all-gather of panel p runs on a side
        stream while panel p+1 is being computed.  CUDA tensors, NCCL group."""
        import torch
        compute = torch.cuda.current_stream()
        comm = _side_stream()
        step = -(-self.ncols // panels)
        step = -(-step // self.align) * self.align if step > self.align else step
        begin = 0
        while begin < self.ncols:
            cnt = min(step, self.ncols - begin)
            self.local_gemm(dtype, transA, transB, m, k, alpha, A, lda, B_block, ldb, beta, C_block, m, kernelId,
                            compute, begin, cnt)
            done = torch.cuda.Event()
            done.record(compute)
            comm.wait_event(done)
            with torch.cuda.stream(comm):
                self.gather(C_block, C_full, m, group, begin, cnt)
            begin += cnt
        compute.wait_stream(comm)


    # ---- exchange fused into the GEMM -------------------------------------------------------
    def gemm_and_broadcast(self, transA, transB, m, k, alpha, A, lda, B_block, ldb, beta, C_sym: "SymmetricC",
                           kernelId=_g.KERNEL_AUTO, stream=None, barrier: bool = True):
        """fp16 GEMM on this rank's column block whose epilogue writes the block into the full
        C of every rank (C_sym).  With beta != 0 the old values are taken from this rank's
        copy.  `barrier`: wait (on the stream) until every rank's GEMM has finished, after
        which the whole of C is valid on this rank."""
        off = self.col0 * m * 2  # bytes to column col0 of the (n, m) fp16 array, leading dimension m
        mine = C_sym.ptrs[self.rank] + off
        peers = [p + off for r, p in enumerate(C_sym.ptrs) if r != self.rank]
        _g.gemm_bcast(transA, transB, m, self.ncols, k, alpha, A, lda, B_block, ldb, beta, mine, m, peers, kernelId,
                      stream)
        if barrier:
            C_sym.barrier()


    def gemm_and_multicast(self, transA, transB, m, k, alpha, A, lda, B_block, ldb, beta, C_sym: "SymmetricC",
                           kernelId=_g.KERNEL_AUTO, stream=None, barrier: bool = True):
        """The same exchange through the multicast address of the symmetric allocation: the epilogue writes
        every finished piece once (multimem.st) and NVSwitch delivers it to every rank's copy of C, this
        rank's included.  Needs `C_sym.multicast_ptr` (NVLink multicast support)."""
        if not C_sym.multicast_ptr:
            raise RuntimeError("this symmetric allocation has no multicast mapping")
        off = self.col0 * m * 2
        _g.gemm_mcast(transA, transB, m, self.ncols, k, alpha, A, lda, B_block, ldb, beta, C_sym.ptrs[self.rank] + off,
                      m, C_sym.multicast_ptr + off, kernelId, stream)
        if barrier:
            C_sym.barrier()

    # ---- the C-ABI multi-GPU entry points ---------------------------------------------------
    def gemm_sharded(self, transA, transB, m, k, alpha, A, lda, B_block, ldb, beta, C_full, gather_c: bool = True,
                     comm: int | None = None, kernelId=_g.KERNEL_AUTO, stream=None):
        """mmbo_gemm_f16_sharded: this rank's block of C_full (the whole m x n C on this GPU) is computed in
        place and, with gather_c, the blocks are exchanged through the caller's NCCL communicator."""
        if comm is None and gather_c and self.world > 1:
            comm = nccl_comm_ptr()
        _g.gemm_sharded(self.world, self.rank, comm, gather_c, transA, transB, m, self.n, k, alpha, A, lda, B_block,
                        ldb, beta, C_full, m, kernelId, stream)

    def gemm_sharded_host(self, transA, transB, m, k, alpha, hA, lda, hB_block, ldb, beta, hC_block, ldc,
                          comm: int | None = None, kernelId=_g.KERNEL_AUTO):
        """mmbo_gemm_f16_sharded_host: host operands; each rank uploads 1 / world of A and the GPUs exchange
        the shares over NVLink."""
        if comm is None and self.world > 1:
            comm = nccl_comm_ptr()
        _g.gemm_sharded_host(self.world, self.rank, comm, transA, transB, m, self.n, k, alpha, hA, lda, hB_block, ldb,
                             beta, hC_block, ldc, kernelId)


def bind_host_to_device(device_index: int) -> str:
    """Run this process on the CPU cores next to GPU `device_index` (NVML's ideal affinity for the device,
    intersected with the cores the process may use), so that pinned host buffers allocated afterwards live on
    that GPU's NUMA node and host <-> device copies of several ranks do not all cross the same socket link.
    Only this process's own CPU affinity changes; nothing of the GPU is touched.  Returns a short description
    of what was done (for a benchmark record); never raises."""
    import os
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
        ideal = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        pick = ideal & allowed
        if not pick:
            return "unchanged (no allowed core in the device's ideal set)"
        if pick == allowed:
            return f"unchanged (all {len(allowed)} allowed cores are local)"
        os.sched_setaffinity(0, pick)
        return f"{len(pick)} of {len(allowed)} allowed cores (local to GPU {device_index})"
    except Exception as e:  # no NVML, no affinity support: run where the launcher put us
        return f"unchanged ({type(e).__name__})"


def nccl_comm_ptr(group=None) -> int:
    """Address of the ncclComm_t behind a torch.distributed NCCL process group (what the C ABI's multi-GPU
    entry points take).  The communicator is created by the group's first collective; one is issued here."""
    import torch
    import torch.distributed as dist
    group = dist.group.WORLD if group is None else group
    dist.all_reduce(torch.zeros(1, device="cuda"), group=group)
    torch.cuda.synchronize()
    return int(group._get_backend(torch.device("cuda"))._comm_ptr())


class SymmetricC:
    """The full column-major C (n columns of m fp16 elements) allocated in symmetric memory:
    `tensor` is this rank's copy, `ptrs[r]` the address at which rank r's copy is mapped into
    this process.  Collective: every rank of `group` constructs it at the same time."""

    def __init__(self, n: int, m: int, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        group = dist.group.WORLD if group is None else group
        self.tensor = symm_mem.empty((n, m), dtype=torch.float16, device=torch.device("cuda", torch.cuda.current_device()))
        self._hdl = symm_mem.rendezvous(self.tensor, group)
        self.ptrs = [int(p) for p in self._hdl.buffer_ptrs]
        self.rank, self.world = self._hdl.rank, self._hdl.world_size
        # address of the same buffer in the NVLink multicast mapping (0: no multicast support here)
        self.multicast_ptr = int(getattr(self._hdl, "multicast_ptr", 0) or 0)

    def barrier(self):
        """All ranks' work queued so far on their current streams has finished (stream-ordered)."""
        self._hdl.barrier()


_SIDE = {}


def _side_stream():
    import torch
    dev = torch.cuda.current_device()
    if dev not in _SIDE:
        _SIDE[dev] = torch.cuda.Stream()
    return _SIDE[dev]
