"""Multi-GPU path on real devices (needs >= 2 GPUs, skipped otherwise): two ranks, one
per GPU, each computes its column block of C through the C ABI; the blocks are
all-gathered over NCCL (whole and panel-overlapped), or stored into every rank's copy of C
by the GEMM's own epilogue (symmetric memory), and compared with the oracle."""
import os
import pathlib
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import gemm_mmbo_b200 as mm
        from gemm_mmbo_b200.sharded import ColumnShard
        from oracle import oracle as O
        m, n, k = 1024, 2048, 520
        for ta, tb in ((False, False), (False, True)):
            sh = ColumnShard(n, world, rank)
            ra = k if ta else m
            A = torch.empty(((m if ta else k), ra), dtype=torch.float16, device="cuda")
            mm.fill("f16", A, ra, A.shape[0], ra, mat=0)
            w = sh.b_window(tb, k)
            B = torch.empty((w["cols"], w["rows"]), dtype=torch.float16, device="cuda")
            mm.fill("f16", B, w["rows"], w["cols"], w["rows"], mat=1, row0=w["row0"], col0=w["col0"],
                    total_rows=w["total_rows"])
            C = torch.full((sh.ncols, m), float("nan"), dtype=torch.float16, device="cuda")
            hA = O.fill("f16", ra, A.shape[0], mat=0)
            hB = O.fill("f16", n if tb else k, k if tb else n, mat=1)
            ref = O.gemm("f16", ta, tb, m, n, k, 1.0, hA, ra, hB, n if tb else k, 0.0, None, m)
            for panels in (1, 4):
                full = torch.zeros((n, m), dtype=torch.float16, device="cuda")
                if panels == 1:
                    sh.local_gemm("f16", ta, tb, m, k, 1.0, A, ra, B, w["rows"], 0.0, C, m)
                    sh.gather(C, full, m)
                else:
                    sh.gemm_and_gather("f16", ta, tb, m, k, 1.0, A, ra, B, w["rows"], 0.0, C, full, panels=panels)
                torch.cuda.synchronize()
                assert mm.device_status() == 0
                err = O.rel_frobenius("f16", m, n, full.cpu().numpy(), m, ref)
                assert err <= 2e-3, (ta, tb, panels, err)
        # the exchange fused into the GEMM: the epilogue stores this rank's block into every
        # rank's copy of C (symmetric memory), then a barrier; beta = 0 and beta != 0
        from gemm_mmbo_b200.sharded import SymmetricC
        ta, tb = False, True
        sh = ColumnShard(n, world, rank)
        A = torch.empty((k, m), dtype=torch.float16, device="cuda")
        mm.fill("f16", A, m, k, m, mat=0)
        w = sh.b_window(tb, k)
        B = torch.empty((w["cols"], w["rows"]), dtype=torch.float16, device="cuda")
        mm.fill("f16", B, w["rows"], w["cols"], w["rows"], mat=1, row0=w["row0"], col0=w["col0"],
                total_rows=w["total_rows"])
        hA, hB, hC = O.fill("f16", m, k, mat=0), O.fill("f16", n, k, mat=1), O.fill("f16", m, n, mat=2)
        sym = SymmetricC(n, m)
        for beta in (0.0, 0.5):
            if beta == 0.0:
                sym.tensor.fill_(float("nan"))
            else:
                mm.fill("f16", sym.tensor, m, n, m, mat=2)
            sym.barrier()
            sh.gemm_and_broadcast(ta, tb, m, k, 1.0, A, m, B, w["rows"], beta, sym)
            torch.cuda.synchronize()
            assert mm.device_status() == 0
            ref = O.gemm("f16", ta, tb, m, n, k, 1.0, hA, m, hB, n, beta, hC if beta else None, m)
            err = O.rel_frobenius("f16", m, n, sym.tensor.cpu().numpy(), m, ref)
            assert err <= 2e-3, ("fused", beta, err)
            sym.barrier()
        q.put((rank, "ok"))
    except Exception as e:
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gpu_ranks_sharded_gemm_and_gather(cuda):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=240) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
    assert results == {0: "ok", 1: "ok"}, results
