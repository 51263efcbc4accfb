"""The grouping entry point that takes no work buffer (nsl_bucket_noalloc) against kc_bucket, through the C ABI.

Some callers cannot hand the library device work memory: they run inside a host that owns the allocator, or on a path
where cudaMalloc is not allowed.  For them the 2n+3 ints of offsets sit in an array inside the library.  Because that
array is shared by all calls and keeps the previous call's contents, the check runs two different groupings back to
back and compares each with kc_bucket's result exactly (integer outputs: bit-exact)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _noalloc(inds, n):
    import torch
    from nanoseedlm_b200 import lib as L
    inds = np.ascontiguousarray(inds, np.int32).ravel()
    P = inds.size
    mt = P // L.MMT_BN + n
    di = torch.from_numpy(inds).cuda()
    perm = torch.zeros(max(P, 1), dtype=torch.int32, device="cuda")
    tiles = torch.zeros(mt * 4, dtype=torch.int32, device="cuda")
    nt = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    L.load().nsl_bucket_noalloc(torch.cuda.current_stream().cuda_stream, di.data_ptr(), P, n, perm.data_ptr(),
                                tiles.data_ptr(), nt.data_ptr())
    torch.cuda.synchronize()
    L.check()
    n_t = int(nt.item())
    tl = tiles.cpu().numpy().reshape(mt, 4)
    return perm.cpu().numpy()[:P], [tuple(int(v) for v in tl[i, :3]) for i in range(n_t)], n_t


def test_two_calls_in_a_row_match_kc_bucket():
    from nanoseedlm_b200 import kernels
    rng = np.random.default_rng(5)
    cases = [(128, rng.integers(0, 128, 512 * 8)), (40, rng.integers(0, 40, 300) * rng.integers(0, 2, 300)),
             (1024, rng.integers(0, 1024, 64 * 10)), (1, np.zeros(200, np.int64)), (7, np.zeros(0, np.int64)),
             (16, rng.integers(0, 16, 33))]      # also: one expert only, and an empty pair list (no tiles)
    for n, inds in cases:   # back to back: the second and third calls find the previous call's offsets in the array
        perm, tiles, nt = _noalloc(inds, n)
        rperm, rtiles, rnt = kernels.kt_bucket(inds, n)
        assert nt == rnt and tiles == rtiles and np.array_equal(perm, rperm)


def test_more_experts_than_the_array_holds_is_refused():
    import torch
    from nanoseedlm_b200 import lib as L
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    L.load().nsl_bucket_noalloc(None, z.data_ptr(), 8, 1025, z.data_ptr(), z.data_ptr(), z.data_ptr())
    assert "at most 1024" in L.last_error()
