"""Multi-GPU path on real devices (needs >= 2 GPUs, skipped otherwise): two ranks, one per GPU.
Each rank computes its column block of C through the C ABI; the one optional exchange -- every rank
ends with the whole C -- is covered in every form the library has: NCCL all-gather from Python (whole
and panel-overlapped), the C ABI's own multi-GPU entry points (mmbo_gemm_f16_sharded with equal and
unequal blocks, mmbo_gemm_f16_sharded_host with A uploaded in shares and exchanged over NVLink), and
the exchange fused into the GEMM's epilogue (one store per peer; one multimem store through NVSwitch
where the system has NVLink multicast).  Everything is compared with the oracle.

A rank never enters a device-side barrier after a failure: both ranks agree on the host
(all-reduce of an ok flag) after every step that can fail, and stop together."""
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


class _Stop(Exception):
    pass


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    notes = []

    def agree(step, fn):
        """Runs fn on this rank; all ranks then agree whether everyone succeeded.  Returns fn's value, or
        raises _Stop on EVERY rank when any rank failed (so nobody walks into a barrier alone)."""
        ok, val, msg = 1.0, None, ""
        try:
            val = fn()
        except Exception as e:
            ok, msg = 0.0, f"{step}: {type(e).__name__}: {e}"
        t = torch.tensor([ok], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        if float(t.item()) != 1.0:
            raise _Stop(msg or f"{step}: the other rank failed")
        return val

    try:
        import gemm_mmbo_b200 as mm
        from gemm_mmbo_b200.sharded import ColumnShard, SymmetricC, nccl_comm_ptr
        from oracle import oracle as O
        m, n, k = 1024, 2048, 520

        def operands(ta, tb, n_cols, sh):
            ra = k if ta else m
            A = torch.empty(((m if ta else k), ra), dtype=torch.float16, device="cuda")
            mm.fill("f16", A, ra, A.shape[0], ra, mat=0)
            w = sh.b_window(tb, k)
            B = torch.empty((w["cols"], w["rows"]), dtype=torch.float16, device="cuda")
            mm.fill("f16", B, w["rows"], w["cols"], w["rows"], mat=1, row0=w["row0"], col0=w["col0"],
                    total_rows=w["total_rows"])
            hA = O.fill("f16", ra, A.shape[0], mat=0)
            hB = O.fill("f16", n_cols if tb else k, k if tb else n_cols, mat=1)
            return A, ra, B, w["rows"], hA, hB

        def check(full, ref, n_cols, what):
            torch.cuda.synchronize()
            assert mm.device_status() == 0, what
            err = O.rel_frobenius("f16", m, n_cols, np.ascontiguousarray(full.cpu().numpy()), m, ref)
            assert err <= 2e-3, (what, err)

        # 1. NCCL all-gather driven from Python: whole blocks, and panel by panel on a side stream
        for ta, tb in ((False, False), (False, True)):
            sh = ColumnShard(n, world, rank)
            A, ra, B, rb, hA, hB = operands(ta, tb, n, sh)
            ref = O.gemm("f16", ta, tb, m, n, k, 1.0, hA, ra, hB, n if tb else k, 0.0, None, m)
            C = torch.full((sh.ncols, m), float("nan"), dtype=torch.float16, device="cuda")
            for panels in (1, 4):
                full = torch.zeros((n, m), dtype=torch.float16, device="cuda")

                def run():
                    if panels == 1:
                        sh.local_gemm("f16", ta, tb, m, k, 1.0, A, ra, B, rb, 0.0, C, m)
                        sh.gather(C, full, m)
                    else:
                        sh.gemm_and_gather("f16", ta, tb, m, k, 1.0, A, ra, B, rb, 0.0, C, full, panels=panels)
                    check(full, ref, n, ("python gather", ta, tb, panels))
                agree(f"python gather {ta} {tb} {panels}", run)

        # 2. the C ABI's multi-GPU entry point on device operands: equal blocks (one ncclAllGather in place)
        #    and unequal blocks (1024 + 768 columns: a group of ncclBroadcast), beta = 0 and beta != 0
        comm = agree("communicator", nccl_comm_ptr)
        for n_cols, (ta, tb), beta in ((2048, (False, False), 0.0), (1792, (True, True), 0.5), (2048, (False, True), 0.5)):
            sh = ColumnShard(n_cols, world, rank)
            A, ra, B, rb, hA, hB = operands(ta, tb, n_cols, sh)
            hC = O.fill("f16", m, n_cols, mat=2)
            ref = O.gemm("f16", ta, tb, m, n_cols, k, 1.0, hA, ra, hB, n_cols if tb else k, beta, hC if beta else None, m)
            full = torch.full((n_cols, m), float("nan"), dtype=torch.float16, device="cuda")
            if beta:
                mm.fill("f16", full, m, n_cols, m, mat=2)

            def run():
                sh.gemm_sharded(ta, tb, m, k, 1.0, A, ra, B, rb, beta, full, True, comm)
                check(full, ref, n_cols, ("mmbo_gemm_f16_sharded", n_cols, ta, tb, beta))
            agree(f"mmbo_gemm_f16_sharded {n_cols}", run)

        # 3. ... and on host operands: every rank holds all of A on the host, uploads its share, the GPUs
        #    exchange the shares; B and C blocks travel in panels.  Checked on this rank's block.
        for (ta, tb), beta in (((False, True), 0.5), ((True, False), 0.0)):
            sh = ColumnShard(n, world, rank)
            A, ra, B, rb, hA, hB = operands(ta, tb, n, sh)
            hC = O.fill("f16", m, n, mat=2)
            ref = O.gemm("f16", ta, tb, m, n, k, 1.25, hA, ra, hB, n if tb else k, beta, hC if beta else None, m)
            hB_blk = np.ascontiguousarray(B.cpu().numpy())
            hC_blk = np.ascontiguousarray(hC[sh.col0:sh.col0 + sh.ncols]) if beta else \
                np.full((sh.ncols, m), np.nan, dtype=np.float16)

            def run():
                sh.gemm_sharded_host(ta, tb, m, k, 1.25, hA, ra, hB_blk, rb, beta, hC_blk, m, comm)
                assert mm.device_status() == 0
                err = O.rel_frobenius("f16", m, sh.ncols, hC_blk, m, np.ascontiguousarray(ref[sh.col0:sh.col0 + sh.ncols]))
                assert err <= 2e-3, ("mmbo_gemm_f16_sharded_host", ta, tb, beta, err)
            agree(f"mmbo_gemm_f16_sharded_host {ta} {tb}", run)

        # 4. the exchange fused into the GEMM: the epilogue writes this rank's block into every rank's copy
        #    of C (symmetric memory) -- one store per peer, or one multimem store through NVSwitch
        ta, tb = False, True
        sh = ColumnShard(n, world, rank)
        A, ra, B, rb, hA, hB = operands(ta, tb, n, sh)
        hC = O.fill("f16", m, n, mat=2)
        sym = agree("symmetric memory", lambda: SymmetricC(n, m))
        have_mc = agree("multicast?", lambda: bool(sym.multicast_ptr))
        mc = torch.tensor([1.0 if have_mc else 0.0], device="cuda")
        dist.all_reduce(mc, op=dist.ReduceOp.MIN)
        variants = ["peers"] + (["multicast"] if float(mc.item()) == 1.0 else [])
        notes.append("multicast " + ("tested" if len(variants) == 2 else "unavailable"))
        for variant in variants:
            for beta in (0.0, 0.5):
                def prepare():
                    if beta == 0.0:
                        sym.tensor.fill_(float("nan"))
                    else:
                        mm.fill("f16", sym.tensor, m, n, m, mat=2)
                    torch.cuda.synchronize()
                agree("prepare", prepare)
                sym.barrier()  # every copy is initialised before anyone stores into it

                def launch():
                    fn = sh.gemm_and_broadcast if variant == "peers" else sh.gemm_and_multicast
                    fn(ta, tb, m, k, 1.0, A, m, B, rb, beta, sym, barrier=False)
                agree(f"fused {variant} launch", launch)
                sym.barrier()  # both launches were accepted: the stream-ordered barrier cannot wait alone
                ref = O.gemm("f16", ta, tb, m, n, k, 1.0, hA, m, hB, n, beta, hC if beta else None, m)
                agree(f"fused {variant} beta={beta}", lambda: check(sym.tensor, ref, n, ("fused", variant, beta)))
                sym.barrier()
        torch.cuda.synchronize()
        dist.barrier()  # nobody leaves while a peer may still touch the shared mappings
        q.put((rank, "ok", notes))
    except _Stop as e:
        q.put((rank, f"stopped: {e}", notes))
    except Exception as e:
        q.put((rank, f"{type(e).__name__}: {e}", notes))
    finally:
        try:
            torch.cuda.synchronize()
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.timeout(420)
def test_two_gpu_ranks_sharded_gemm_and_gather(cuda):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    try:
        for p in procs:
            p.start()
        results = [q.get(timeout=360) for _ in range(world)]
        for p in procs:
            p.join(timeout=60)
    finally:
        for p in procs:  # never leave a child behind on a shared GPU
            if p.is_alive():
                p.terminate()
                p.join(timeout=10)
            if p.is_alive():
                p.kill()
    print("notes:", [r[2] for r in results])
    assert {r[0]: r[1] for r in results} == {0: "ok", 1: "ok"}, results
