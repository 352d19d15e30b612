"""GPU: the permutation kernel against exact index algebra (integers stored as floats, no tolerance) --
the checking idea of cuTT's own tester (external/cutt/src/cutt_test.cpp:136-160)."""
import itertools

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run_transpose(engine, src: np.ndarray, extent, perm):
    import torch
    s = torch.from_numpy(src).cuda()
    d = torch.empty_like(s)
    engine.transpose(s.data_ptr(), d.data_ptr(), extent, perm, src.dtype.itemsize, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return d.cpu().numpy()


def expected(src, extent, perm):
    r = len(extent)
    nd = src.reshape(extent[::-1])                       # numpy sees reversed (row-major) mode order
    axes = [r - 1 - perm[r - 1 - i] for i in range(r)]   # dst mode i = src mode perm[i]
    return np.ascontiguousarray(nd.transpose(axes)).ravel()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_all_permutations_rank4(engine, dtype):
    extent = [12, 5, 8, 6]
    src = np.arange(int(np.prod(extent)), dtype=dtype)
    for perm in itertools.permutations(range(4)):
        got = run_transpose(engine, src, extent, list(perm))
        np.testing.assert_array_equal(got, expected(src, extent, list(perm)), err_msg=str(perm))


@pytest.mark.parametrize("extent,perm", [
    ([48, 8, 48, 48], [3, 2, 0, 1]),        # cfg4's A[e,f,b,a] -> [a,b,e,f]
    ([48, 8, 48], [0, 2, 1]),               # cfg4's B[c,f,d] -> [c,d,f]
    ([130, 70], [1, 0]), ([67, 3, 129], [2, 1, 0]), ([1, 7, 1, 9], [3, 0, 1, 2]),
    ([256, 1024, 16], [1, 0, 2]), ([33, 2, 3, 4, 5], [4, 2, 0, 3, 1]),
    # tile extents chosen per launch: one tile of 72, of 96; two of 52 / 50 (4-byte) or 56 / 52 (8-byte); 97 and 200
    ([72, 5, 3, 72], [3, 1, 2, 0]), ([96, 3, 96], [2, 1, 0]), ([100, 104], [1, 0]), ([97, 2, 200], [2, 1, 0]),
    ([8, 300], [1, 0]), ([300, 8], [1, 0]),
])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_selected_shapes(engine, extent, perm, dtype):
    src = np.arange(int(np.prod(extent)), dtype=dtype)
    np.testing.assert_array_equal(run_transpose(engine, src, extent, perm), expected(src, extent, perm))


def test_bad_permutation_is_rejected(engine):
    import torch
    s = torch.zeros(24, device="cuda")
    with pytest.raises(ValueError):
        engine.transpose(s.data_ptr(), s.data_ptr(), [2, 3, 4], [0, 0, 1], 4)
