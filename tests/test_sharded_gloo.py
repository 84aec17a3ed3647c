"""Host-side logic of the multi-GPU path on CPU ranks (gloo, world size 2): the column
partition tiles the matrix, every rank's operand window reproduces the matching slice
of the whole matrix, and the gather of the C blocks (whole block and panel by panel)
reassembles the full column-major C."""
import os
import socket
import sys
import pathlib

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, n: int, m: int, k: int, q):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from gemm_mmbo_b200.sharded import ColumnShard
        from oracle import oracle as O
        sh = ColumnShard(n, world, rank, align=64)
        blocks = sh.blocks()
        assert blocks[0][0] == 0 and sum(nc for _, nc in blocks) == n
        assert all(blocks[i][0] + blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
        # operand windows: this rank's block of B equals the slice of the whole B
        for tb in (False, True):
            w = sh.b_window(tb, k)
            whole = O.fill("f16", n if tb else k, k if tb else n, mat=O.MAT_B)
            mine = O.fill("f16", w["rows"], w["cols"], mat=O.MAT_B, row0=w["row0"], col0=w["col0"],
                          total_rows=w["total_rows"])
            want = whole[:, sh.col0:sh.col0 + sh.ncols] if tb else whole[sh.col0:sh.col0 + sh.ncols]
            assert np.array_equal(mine.view(np.uint16), want.view(np.uint16))
        # exchange: blocks of a known full C
        full = O.fill("f16", m, n, mat=O.MAT_C)                     # (n, m)
        mine = torch.from_numpy(full[sh.col0:sh.col0 + sh.ncols].copy())
        out = torch.zeros((n, m), dtype=torch.float16)
        sh.gather(mine, out, m)
        assert np.array_equal(out.numpy().view(np.uint16), full.view(np.uint16))
        out2 = torch.zeros((n, m), dtype=torch.float16)
        step = 64
        for b in range(0, sh.ncols, step):
            sh.gather(mine, out2, m, col_begin=b, col_count=min(step, sh.ncols - b))
        assert np.array_equal(out2.numpy().view(np.uint16), full.view(np.uint16))
        q.put((rank, "ok"))
    except Exception as e:  # report instead of hanging the peer
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_cpu_ranks_partition_and_gather():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 512, 96, 40, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=150) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
    assert results == {0: "ok", 1: "ok"}, results


def test_unequal_blocks_refuse_gather():
    sys.path.insert(0, str(ROOT))
    from gemm_mmbo_b200.sharded import ColumnShard
    sh = ColumnShard(1000, 3, 0, align=128)
    with pytest.raises(ValueError):
        sh.gather(torch.zeros((sh.ncols, 8)), torch.zeros((1000, 8)), 8)


def _absent_peer_worker(rank: int, world: int, port: int, q):
    """Rank 1 never enters the exchange; rank 0 must get an error after the group's
    time-out instead of waiting forever (failure made on the host, no GPU involved)."""
    import datetime
    import time
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        from gemm_mmbo_b200.sharded import ColumnShard
        sh = ColumnShard(256, world, rank, align=64)
        if rank == 1:
            time.sleep(12)  # absent from the collective
            q.put((rank, "absent"))
            return
        mine = torch.zeros((sh.ncols, 8), dtype=torch.float16)
        out = torch.zeros((256, 8), dtype=torch.float16)
        t0 = time.time()
        try:
            sh.gather(mine, out, 8)
            q.put((rank, "no error"))
        except Exception as e:  # gloo reports the time-out as a RuntimeError
            q.put((rank, f"error after {time.time() - t0:.0f}s: {type(e).__name__}"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.timeout(120)
def test_gather_reports_an_absent_rank_instead_of_hanging():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_absent_peer_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=90) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    assert results[1] == "absent"
    assert results[0].startswith("error after"), results


def test_broadcast_addresses_cover_every_copy(monkeypatch):
    """gemm_and_broadcast hands the GEMM this rank's window in its own copy of C and the same
    window in every other rank's copy (no GPU: the C ABI call is intercepted)."""
    sys.path.insert(0, str(ROOT))
    import importlib
    sharded = importlib.import_module("gemm_mmbo_b200.sharded")
    calls = []
    monkeypatch.setattr(sharded._g, "gemm_bcast", lambda *a: calls.append(a))

    class FakeC:
        ptrs = [0x10000000, 0x20000000, 0x30000000, 0x40000000]
        barriers = 0

        def barrier(self):
            FakeC.barriers += 1

    n, m, k, world = 4096, 512, 64, 4
    for rank in range(world):
        sh = sharded.ColumnShard(n, world, rank)
        sh.gemm_and_broadcast(False, True, m, k, 1.0, 111, m, 222, sh.ncols, 0.0, FakeC())
        (ta, tb, mm_, nn, kk, alpha, A, lda, B, ldb, beta, C, ldc, peers, kid, stream) = calls[-1]
        off = sh.col0 * m * 2
        assert (mm_, nn, kk, ldc) == (m, sh.ncols, k, m)
        assert C == FakeC.ptrs[rank] + off
        assert peers == [p + off for r, p in enumerate(FakeC.ptrs) if r != rank]
    assert FakeC.barriers == world
