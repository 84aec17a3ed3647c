"""Device-side operand generator against the oracle's: bit-exact, padding untouched."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,dist,scale", [("f32", 0, 1.0), ("f32", 1, 1.0), ("f16", 1, 0.5),
                                              ("f16", 0, 1.0), ("f16", 1, 0.015625), ("f32", 2, 1.0)])
def test_device_fill_bit_exact(cuda, mm, oracle, dtype, dist, scale):
    torch = cuda
    rows, cols, ld = 777, 130, 781
    tdt = torch.float32 if dtype == "f32" else torch.float16
    dev = torch.full((cols, ld), float("nan"), dtype=tdt, device="cuda")
    mm.fill(dtype, dev, rows, cols, ld, seed=99, mat=1, dist=dist, scale=scale)
    torch.cuda.synchronize()
    want = oracle.fill(dtype, rows, cols, ld, seed=99, mat=1, dist=dist, scale=scale)
    got = dev.cpu().numpy()
    v = np.uint32 if dtype == "f32" else np.uint16
    assert np.array_equal(got.view(v), want.view(v))


def test_device_fill_shard_window(cuda, mm, oracle):
    """A column block generated on its own equals the same columns of the whole matrix."""
    torch = cuda
    rows, cols = 512, 96
    whole = oracle.fill("f16", rows, cols, rows, seed=5, mat=2, dist=1, scale=1.0)
    dev = torch.empty((32, rows), dtype=torch.float16, device="cuda")
    mm.fill("f16", dev, rows, 32, rows, seed=5, mat=2, dist=1, scale=1.0, col0=64, total_rows=rows)
    torch.cuda.synchronize()
    assert np.array_equal(dev.cpu().numpy().view(np.uint16), whole[64:96].view(np.uint16))
