"""The tcgen05 building blocks (tensor-memory allocation, descriptors, kind::i8 MMA with A in shared memory and in
tensor memory, commit, tensor-memory loads) against numpy integer arithmetic."""
import ctypes as C
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("n,kblocks", [(16, 1), (64, 1), (64, 4), (96, 2), (128, 4), (256, 2)])
def test_umma_i8_matches_numpy(clib, mode, n, kblocks):
    rng = np.random.default_rng(n * 10 + kblocks + mode)
    K = 128 * kblocks
    a = rng.integers(0, 3, (128, K)).astype(np.uint8)
    a[5, :] = 255; a[9, 3] = 200                                       # A is unsigned: 255 must count as 255, not -1
    b = rng.integers(-127, 128, (n, K)).astype(np.int8)
    d = np.zeros((128, n), np.int32)
    rc = clib.gmoe_umma_selftest(a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), n, kblocks, mode, d.ctypes.data_as(C.c_void_p))
    assert rc == 0
    want = a.astype(np.int64) @ b.astype(np.int64).T
    bad = np.argwhere(d != want)
    assert bad.size == 0, f"{len(bad)} wrong, first {bad[:5].tolist()} got {d[tuple(bad[0])]} want {want[tuple(bad[0])]}"
