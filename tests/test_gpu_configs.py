"""The five benchmark configurations (seeded synthetic inputs of the stated shapes and
distributions).  Sizes the oracle finishes in seconds are compared in full; the rest
are checked on sampled rows/columns computed by the oracle in binary64, against the
library's simplest kernel over the whole matrix, and through linearity."""
import numpy as np
import pytest

from helpers import Case, TOL, run_and_check

pytestmark = pytest.mark.gpu


def test_config1_sgemm_nn_1024(cuda, mm, oracle):
    """SGEMM NN, M=N=K=1024, ld=1024, alpha=1, beta=0, A,B ~ U[-1,1), C = 0."""
    case = Case(oracle, "f32", False, False, 1024, 1024, 1024, 1.0, 0.0)
    case.C[:] = 0.0
    for kid in (-1, 1, 2, 3, 4, 5, 6):
        run_and_check(cuda, mm, case, kid)


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_config3_sgemm_ragged_padded(cuda, mm, oracle, ta, tb):
    """SGEMM, M=4095 N=4097 K=1023, every ld = extent + 3, alpha=1.5, beta=-0.25."""
    case = Case(oracle, "f32", ta, tb, 4095, 4097, 1023, 1.5, -0.25, pad=(3, 3, 3))
    ref = case.reference()
    for kid in (-1, 1, 3, 5, 6):
        run_and_check(cuda, mm, case, kid, ref=ref)


def _device_operands(torch, mm, dtype, ta, tb, m, n, k, dist, scale, seed=1234):
    tdt = torch.float16 if dtype == "f16" else torch.float32
    ra, rb = (k if ta else m), (n if tb else k)
    ca, cb = (m if ta else k), (k if tb else n)
    A = torch.empty((ca, ra), dtype=tdt, device="cuda")
    B = torch.empty((cb, rb), dtype=tdt, device="cuda")
    C = torch.empty((n, m), dtype=tdt, device="cuda")
    mm.fill(dtype, A, ra, ca, ra, seed=seed, mat=0, dist=dist, scale=scale)
    mm.fill(dtype, B, rb, cb, rb, seed=seed, mat=1, dist=dist, scale=scale)
    mm.fill(dtype, C, m, n, m, seed=seed, mat=2, dist=dist, scale=scale)
    return A, B, C, ra, rb


def _sampled_check(torch, mm, oracle, dtype, ta, tb, m, n, k, alpha, beta, A, B, C0, C, ra, rb, nsamp=4096):
    """Oracle on sampled elements (always including the corners and tile seams)."""
    rng = np.random.default_rng(0)
    rows = rng.integers(0, m, nsamp)
    cols = rng.integers(0, n, nsamp)
    seams_r = [0, m - 1] + [x for x in (127, 128, 255, 256, m // 2) if x < m]
    seams_c = [0, n - 1] + [x for x in (127, 128, 255, 256, n // 2) if x < n]
    rows[:len(seams_r)] = seams_r
    cols[:len(seams_c)] = seams_c
    hA, hB, hC0 = A.cpu().numpy(), B.cpu().numpy(), C0.cpu().numpy()
    want = oracle.gemm_sampled(dtype, ta, tb, k, alpha, hA, ra, hB, rb, beta, hC0, m, rows, cols)
    got = C.cpu().numpy()[cols, rows].astype(np.float64)
    err = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert err <= TOL[dtype], err
    return err


def test_config2_hgemm_nt_8192(cuda, mm, oracle):
    """HGEMM NT, M=N=K=8192, alpha=1, beta=0.5, A,B,C ~ N(0, 0.5^2) as fp16."""
    torch = cuda
    m = n = k = 8192
    A, B, C0, ra, rb = _device_operands(torch, mm, "f16", False, True, m, n, k, 1, 0.5)
    C = C0.clone()
    mm.hgemm_NT(m, n, k, 1.0, A, ra, B, rb, 0.5, C, m)
    torch.cuda.synchronize()
    assert mm.device_status() == 0
    _sampled_check(torch, mm, oracle, "f16", False, True, m, n, k, 1.0, 0.5, A, B, C0, C, ra, rb)
    # whole matrix against the simplest kernel (itself checked against the oracle on
    # small shapes): both round an fp32 result to fp16, so they differ by rounding only
    Cs = C0.clone()
    mm.hgemm_NT(m, n, k, 1.0, A, ra, B, rb, 0.5, Cs, m, 0)
    torch.cuda.synchronize()
    d = (C.float() - Cs.float()).norm() / Cs.float().norm()
    assert float(d) <= 2e-3
    # linearity in alpha with beta = 0: scaling alpha by two scales every result that
    # is a normal fp16 number exactly (subnormal results round on a fixed grid instead)
    C1, C2 = torch.empty_like(C), torch.empty_like(C)
    mm.hgemm_NT(m, n, k, 0.25, A, ra, B, rb, 0.0, C1, m)
    mm.hgemm_NT(m, n, k, 0.5, A, ra, B, rb, 0.0, C2, m)
    torch.cuda.synchronize()
    normal = C1.abs() >= 2.0 ** -14
    assert torch.equal((C1 * 2)[normal], C2[normal])
    assert float((C1.float() * 2 - C2.float()).abs().max()) <= 2.0 ** -24


@pytest.mark.parametrize("m,n,k", [(65536, 128, 4096), (128, 65536, 4096), (8192, 8192, 256)])
def test_config4_hgemm_tn_skinny(cuda, mm, oracle, m, n, k):
    """HGEMM TN tall-skinny / short-wide set, alpha=1 beta=0, N(0,1)/sqrt(K) inputs."""
    torch = cuda
    A, B, C0, ra, rb = _device_operands(torch, mm, "f16", True, False, m, n, k, 1, 1.0 / np.sqrt(k))
    C = torch.full_like(C0, float("nan"))  # beta == 0: C must not be read
    mm.hgemm_TN(m, n, k, 1.0, A, ra, B, rb, 0.0, C, m)
    torch.cuda.synchronize()
    assert mm.device_status() == 0
    hA, hB = A.cpu().numpy(), B.cpu().numpy()
    ref = oracle.gemm("f16", True, False, m, n, k, 1.0, hA, ra, hB, rb, 0.0, None, m)
    err = oracle.rel_frobenius("f16", m, n, C.cpu().numpy(), m, ref)
    assert err <= TOL["f16"], err


def test_config5_hgemm_nn_32768_one_shard(cuda, mm, oracle):
    """HGEMM NN, M=N=K=32768, alpha=1, beta=0, U[-1,1): one rank's column block of an
    8-way partition (A replicated, B/C block of 4096 columns) on one GPU."""
    torch = cuda
    M = N = K = 32768
    col0, ncols = mm.shard_columns(N, 8, 5)
    assert (col0, ncols) == (5 * 4096, 4096)
    A = torch.empty((K, M), dtype=torch.float16, device="cuda")
    B = torch.empty((ncols, K), dtype=torch.float16, device="cuda")
    C = torch.full((ncols, M), float("nan"), dtype=torch.float16, device="cuda")
    mm.fill("f16", A, M, K, M, mat=0)
    mm.fill("f16", B, K, ncols, K, mat=1, col0=col0, total_rows=K)
    mm.hgemm_NN(M, ncols, K, 1.0, A, M, B, K, 0.0, C, M)
    torch.cuda.synchronize()
    assert mm.device_status() == 0
    rng = np.random.default_rng(1)
    nsamp = 512
    rows = rng.integers(0, M, nsamp)
    cols = rng.integers(0, ncols, nsamp)
    rows[:4] = [0, M - 1, 255, 256]
    cols[:4] = [0, ncols - 1, 127, 128]
    # operands of the sampled elements, generated by the oracle (same generator)
    want = np.empty(nsamp)
    for t in range(nsamp):
        a_row = oracle.fill("f16", 1, K, 1, mat=0, row0=int(rows[t]), total_rows=M)  # A[i, :]
        b_col = oracle.fill("f16", K, 1, K, mat=1, col0=col0 + int(cols[t]), total_rows=K)
        want[t] = float(a_row.astype(np.float64).reshape(-1) @ b_col.astype(np.float64).reshape(-1))
    got = C.cpu().numpy()[cols, rows].astype(np.float64)
    err = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert err <= TOL["f16"], err
    assert torch.isfinite(C).all()


def _harness(name):
    import pathlib
    exe = pathlib.Path(__file__).resolve().parents[1] / "gemm_mmbo_b200" / "_build" / name
    if not exe.exists():
        pytest.skip(f"{name} not built")
    return str(exe)


def test_cpp_harness_test_program(cuda):
    """The C++ test program (counterpart of the reference's test.cc) on the reference's
    default HPL shape and on an fp32 ragged shape; exit code 0 = matches cuBLAS and kernel 0."""
    import subprocess
    for argv in ([], ["4095", "4097", "1023", "--dtype", "f32", "--trans", "TN", "--alpha", "1.5", "--beta", "-0.25"]):
        r = subprocess.run([_harness("test_gemm"), *argv], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stdout + r.stderr
        assert "results match" in r.stdout


def test_cpp_harness_benchmark_program(cuda):
    """The C++ benchmark in the reference's positional form, all three arms."""
    import re
    import subprocess
    for typ in ("0", "1", "2"):
        r = subprocess.run([_harness("benchmark"), typ, "4224", "2048", "384", "4224", "2048", "4224"],
                           capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stdout + r.stderr
        m = re.search(r"time, tflops, efficiency = .*?([0-9.]+), ([0-9.]+), ([0-9.]+)%", r.stdout)
        assert m and float(m.group(2)) > 0.0, r.stdout
