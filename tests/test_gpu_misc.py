"""Router, grouping, SwiGLU, combines, packing and the expert cache against the oracle, through the C ABI."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_route_512_experts_top10_with_tie(oracle, golden):
    # reference: tests/test_qwen4_kernels.c:223-245: indices equal, first index 300, weights to 1e-5
    from nanoseedlm_b200 import kernels
    lg = golden["route_logits"]
    for fn in (kernels.kt_route, kernels.kt_route_cfg):
        ind, wt = fn(lg, 10)
        assert np.array_equal(ind, golden["route_ind"]) and ind[0, 0] == 300
        assert np.max(np.abs(wt - golden["route_wt"]) / golden["route_wt"]) < 1e-5


@pytest.mark.parametrize("T,E,k", [(1, 128, 8), (8, 128, 8), (512, 128, 8), (64, 512, 10), (3, 1024, 32), (5, 40, 1)])
def test_route_shapes(oracle, T, E, k):
    from nanoseedlm_b200 import kernels
    lg = oracle.normal(T * E + k, T * E).reshape(T, E)
    ind, wt = kernels.kt_route(lg, k)
    ri, rw = oracle.route(lg, k)
    assert np.array_equal(ind, ri)
    assert np.max(np.abs(wt - rw) / rw) < 1e-5


@pytest.mark.parametrize("n,rows,k", [(128, 512, 10), (64, 128, 8), (512, 64, 10), (1024, 3, 1), (4, 1, 1)])
def test_bucket_against_host_grouping(oracle, n, rows, k):
    # reference: tests/test_qwen4_engine.c:34-61 (half of the selections on expert 0)
    from nanoseedlm_b200 import kernels
    P = rows * k
    x = 12345
    inds = np.zeros(P, np.int32)
    for i in range(P):
        x = (x * 1664525 + 1013904223) & 0xFFFFFFFF
        inds[i] = ((x >> 8) % n) * ((x >> 4) & 1)
    perm, tiles, nt = kernels.kt_bucket(inds, n)
    rperm, rtiles = oracle.bucket(inds, n)
    assert np.array_equal(perm, rperm) and tiles == rtiles and nt == len(rtiles)


def test_swiglu_and_combines(oracle):
    from nanoseedlm_b200 import kernels
    n = 5000
    g = oracle.normal(1, n, bf16=True) * 3
    u = oracle.normal(2, n, bf16=True)
    assert np.array_equal(kernels.kt_swiglu(g, u).view(np.uint32), oracle.swiglu(g, u).view(np.uint32))
    T, d, k = 3, 300, 8
    D = oracle.normal(3, T * k * d)
    wt = np.abs(oracle.normal(4, T * k)) / 8
    sh = oracle.normal(5, T * d)
    sg = oracle.normal(6, T)
    got = kernels.kt_q4_moe_combine(D, wt, sh, sg, T, d, k)
    ref = oracle.q4_moe_combine(D, wt, sh, sg, T, d, k)
    assert np.max(np.abs(got - ref)) <= 1e-5 * np.max(np.abs(ref))
    Db, wb, shb, xb = (oracle.normal(s, m, bf16=True) for s, m in ((7, T * k * d), (8, T * k), (9, T * d), (10, T * d)))
    got = kernels.kt_moe_combine(Db, wb, shb, xb, T, d, k)
    ref = oracle.moe_combine(Db, wb, shb, xb, T, d, k).reshape(T, d)
    assert np.mean(got.reshape(T, d) == ref) > 0.99   # bf16 points; an f32 sum-order flip may move one ulp
    assert np.max(np.abs(got.reshape(T, d) - ref)) <= np.max(np.abs(ref)) / 64


def test_swiglu_packed_is_swiglu_as_bf16_bits(oracle):
    import torch
    from nanoseedlm_b200 import kernels, lib as L
    n = 6002
    g, u = oracle.normal(11, n, bf16=True) * 3, oracle.normal(12, n, bf16=True)
    gd, ud = kernels.dev(g), kernels.dev(u)
    out = torch.zeros(n, dtype=torch.int16, device="cuda")
    L.load().nsl_swiglu_packed(None, gd.data_ptr(), ud.data_ptr(), out.data_ptr(), n)
    torch.cuda.synchronize()
    want = (oracle.swiglu(g, u).view(np.uint32) >> 16).astype(np.uint16)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want)


def test_pack_input_bf16_any_length(oracle):
    """Round to nearest even, every element of any n (the reference's kernel packs whole groups of 8: engine/kernels_moe.cu:2196-2201)."""
    from nanoseedlm_b200 import kernels
    x = oracle.normal(11, 1003)
    u32 = x.view(np.uint32).astype(np.uint64)
    want = ((u32 + 0x7FFF + ((u32 >> 16) & 1)) >> 16).astype(np.uint16)
    assert np.array_equal(kernels.kt_pack_bf16(x), want)
