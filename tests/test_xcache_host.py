"""The expert cache's host logic (include/nslm_cache.h) without a GPU: every CUDA call it makes goes through a table of
function pointers, replaced here by fakes ("device" memory = host memory, copies = memmove, the admit kernel = a Python
function that queues jobs).  Failures are injected on the host: the n-th allocation fails, a copy fails.  Checked: nothing
leaks when creation fails part-way, a failed copy surfaces as -1 with a message and leaves the cache usable, and the
side-stream path issues one copy per run of consecutive units that go to consecutive slots."""
import ctypes as C

import numpy as np
import pytest


class Fake:
    """The NslCacheOps table backed by host memory, with counters and failure switches."""

    def __init__(self, L):
        self.L = L
        self.live = {}            # address -> buffer (keeps it alive)
        self.allocs = 0
        self.fail_alloc_at = None  # the n-th allocation (host or device, 1-based) fails
        self.fail_copy_at = None   # the n-th copy fails
        self.copies = []           # (dst, src, bytes, kind)
        self.jobs_for_next_admit = []
        self.admits = []
        vp, i, sz = C.c_void_p, C.c_int, C.c_size_t
        pp = C.POINTER(C.c_void_p)
        self.sigs = [("host_alloc", C.CFUNCTYPE(i, pp, sz, i), self.host_alloc), ("host_free", C.CFUNCTYPE(i, vp), self.free),
                     ("dev_ptr", C.CFUNCTYPE(i, pp, vp), self.dev_ptr), ("dev_alloc", C.CFUNCTYPE(i, pp, sz), self.dev_alloc),
                     ("dev_free", C.CFUNCTYPE(i, vp), self.free), ("copy_async", C.CFUNCTYPE(i, vp, vp, sz, i, vp), self.copy),
                     ("fill_async", C.CFUNCTYPE(i, vp, i, sz, vp), self.fill), ("stream_create", C.CFUNCTYPE(i, pp), self.make_handle),
                     ("stream_destroy", C.CFUNCTYPE(i, vp), self.ok1), ("stream_sync", C.CFUNCTYPE(i, vp), self.ok1),
                     ("event_create", C.CFUNCTYPE(i, pp), self.make_handle), ("event_destroy", C.CFUNCTYPE(i, vp), self.ok1),
                     ("event_record", C.CFUNCTYPE(i, vp, vp), self.ok2), ("event_sync", C.CFUNCTYPE(i, vp), self.ok1),
                     ("stream_wait", C.CFUNCTYPE(i, vp, vp), self.ok2),
                     ("admit", C.CFUNCTYPE(i, vp, C.POINTER(L.CachePool), i, vp, i, i), self.admit),
                     ("copy_kernel", C.CFUNCTYPE(i, vp, C.POINTER(L.CachePool), i), self.copy_kernel)]
        self.cfuncs = [t(f) for _, t, f in self.sigs]
        self.table = (C.c_void_p * len(self.cfuncs))(*[C.cast(f, C.c_void_p) for f in self.cfuncs])
        self.handles = 0

    def _alloc(self, p, n):
        self.allocs += 1
        if self.fail_alloc_at is not None and self.allocs == self.fail_alloc_at:
            return -1
        buf = (C.c_uint8 * max(int(n), 16))()
        addr = C.addressof(buf)
        self.live[addr] = buf
        p[0] = addr
        return 0

    def host_alloc(self, p, n, mapped): return self._alloc(p, n)
    def dev_alloc(self, p, n): return self._alloc(p, n)

    def free(self, p):
        return 0 if self.live.pop(p, None) is not None else -1

    def dev_ptr(self, d, h):
        d[0] = h
        return 0

    def copy(self, dst, src, n, kind, s):
        self.copies.append((dst, src, int(n), kind))
        if self.fail_copy_at is not None and len(self.copies) == self.fail_copy_at:
            return -1
        C.memmove(dst, src, n)
        return 0

    def fill(self, dst, v, n, s):
        C.memset(dst, v, n)
        return 0

    def make_handle(self, p):
        self.handles += 1
        p[0] = 0x1000 + self.handles
        return 0

    def ok1(self, a): return 0
    def ok2(self, a, b): return 0

    def admit(self, s, pool, sl, inds, count, flags):
        p = pool.contents
        jobs = self.jobs_for_next_admit
        self.admits.append((sl, count))
        C.cast(p.njobs, C.POINTER(C.c_int32))[0] = len(jobs)
        out = C.cast(p.jobs, C.POINTER(C.c_int32))
        for j, (u, slot) in enumerate(jobs):
            out[2 * j], out[2 * j + 1] = u, slot
        return 0

    def copy_kernel(self, s, pool, blocks):
        return 0


@pytest.fixture
def fake():
    from nanoseedlm_b200 import lib as L
    lib = L.load()
    f = Fake(L)
    lib.nsl_xcache_set_ops(C.cast(f.table, C.c_void_p))
    yield f, lib, L
    lib.nsl_xcache_set_ops(None)
    L.last_error()


LENS = np.array([[512, 512, 0, 128], [512, 512, 0, 128], [256, 256, 0, 64]], np.uint64)


def make(lib, layers=3, per_layer=8, slots=12):
    return lib.nsl_xcache_create(layers, per_layer, LENS.ctypes.data, slots)


def test_creation_that_fails_part_way_releases_everything(fake):
    f, lib, L = fake
    h = make(lib)
    assert h and not L.last_error()
    total = f.allocs
    lib.nsl_xcache_destroy(h)
    assert not f.live
    for k in range(1, total + 1):      # the k-th allocation fails
        f.allocs, f.fail_alloc_at = 0, k
        assert not make(lib)
        assert "cannot allocate" in L.last_error()
        assert not f.live, k
    f.fail_alloc_at = None


def test_side_stream_copies_one_per_run_and_the_bytes_arrive(fake):
    f, lib, L = fake
    h = make(lib)
    ub = lib.nsl_xcache_unit_bytes(h)
    assert ub == 2 * (512 + 512 + 256) + (256 + 256 + 256)      # every stream padded to 256 bytes
    for u in range(24):
        unit = np.ctypeslib.as_array(C.cast(lib.nsl_xcache_host_unit(h, u), C.POINTER(C.c_uint8)), (ub,))
        unit[:] = (np.arange(ub) * 7 + u) % 251
    assert lib.nsl_xcache_finish(h, None) == 0
    pool = C.cast(lib.nsl_xcache_pool(h), C.POINTER(L.CachePool)).contents
    vram = pool.vram
    f.copies.clear()
    f.jobs_for_next_admit = [(5, 3), (6, 4), (7, 5), (20, 9), (21, 11)]      # runs: units 5-7 -> slots 3-5; 20 -> 9; 21 -> 11
    assert lib.nsl_xcache_fetch(h, None, 1, None, 0, 1) == 0
    up = [c for c in f.copies if c[3] == 1]
    assert [(c[0] - vram, c[2]) for c in up] == [(3 * ub, 3 * ub), (9 * ub, ub), (11 * ub, ub)]
    got = np.ctypeslib.as_array(C.cast(vram, C.POINTER(C.c_uint8)), (12 * ub,))
    for u, s in f.jobs_for_next_admit:
        assert np.array_equal(got[s * ub:(s + 1) * ub], (np.arange(ub) * 7 + u) % 251)
    v = (C.c_uint64 * 5)()
    assert lib.nsl_xcache_stats(h, *[C.cast(C.byref(v, 8 * i), C.c_void_p) for i in range(5)]) == 0
    assert v[2] == 12 + 5 and v[4] == 3 and v[3] == 17 * ub      # the first fill's 12 units, then 5 in 3 runs
    lib.nsl_xcache_destroy(h)
    assert not f.live


def test_a_failed_copy_is_reported_and_the_cache_stays_usable(fake):
    f, lib, L = fake
    h = make(lib)
    assert lib.nsl_xcache_finish(h, None) == 0
    f.jobs_for_next_admit = [(2, 0), (9, 5)]
    f.fail_copy_at = len(f.copies) + 2      # the second run's copy fails
    assert lib.nsl_xcache_fetch(h, None, 0, None, 0, 1) == -1
    assert "copy of units 9..9" in L.last_error()
    f.fail_copy_at = None
    assert lib.nsl_xcache_fetch(h, None, 0, None, 0, 1) == 0
    f.jobs_for_next_admit = [(30, 1)]       # a job the tables cannot hold
    assert lib.nsl_xcache_fetch(h, None, 0, None, 0, 1) == -1 and "out of range" in L.last_error()
    assert lib.nsl_xcache_fetch(h, None, 7, None, 0, 0) == -1 and "layer 7" in L.last_error()
    lib.nsl_xcache_destroy(h)
    assert not f.live


def test_prefetch_admits_every_expert_of_the_next_layer(fake):
    f, lib, L = fake
    h = make(lib, layers=3, per_layer=4, slots=8)
    assert lib.nsl_xcache_finish(h, None) == 0
    f.jobs_for_next_admit = []
    for l in range(3):
        assert lib.nsl_xcache_layer_start(h, None, l, 1) == 0
    assert f.admits == [(0, 4), (1, 4), (2, 4)]      # layer 0 at its own start, then each next layer one layer ahead
    lib.nsl_xcache_destroy(h)
