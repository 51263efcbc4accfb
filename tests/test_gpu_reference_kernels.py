"""This library's kernels against the REFERENCE'S OWN CUDA kernels on the same device buffers.

oracle/_ref/libnslm_ref_gpu.so is engine/kernels_moe.cu + engine/kernels_qwen4.cu of the reference, compiled unmodified for
sm_100a (oracle/Makefile); both libraries export the same kc_* / kq4_* entry points, so every call below is made twice with
identical arguments.  Two kinds of check:

  * direct: routing ids identical, mat-vec / GEMM / combine outputs within the bound the reference's own kernel tests use
    (one bf16 unit plus the f32 accumulation noise, tests/test_mova_kernels.c:27-30), at BASELINE config-1 sizes;
  * the suite's own oracle-based checks re-run with the kc_* / kq4_* names resolved to the reference's kernels: if the
    reference passes them, the expectations written in those tests (and the CPU oracle behind them) are the reference's
    behaviour, not this library's.

Skipped when the reference library was not built (it builds where the reference's sources and nvcc are)."""
import contextlib

import numpy as np
import pytest

from oracle import ref_gpu

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_gpu.available(), reason="oracle/_ref/libnslm_ref_gpu.so was not built")]


class _ReferenceFirst:
    """kc_* / kq4_* from the reference's library, everything else (nsl_*: error text, the stream table) from this one."""

    def __init__(self, mine, ref):
        self._mine, self._ref = mine, ref

    def __getattr__(self, name):
        if name.startswith(("kc_", "kq4_")):
            return getattr(self._ref, name)      # AttributeError if the reference has no such entry point
        return getattr(self._mine, name)


@contextlib.contextmanager
def reference_kernels():
    from nanoseedlm_b200 import lib as L
    mine = L.load()
    L._lib = _ReferenceFirst(mine, ref_gpu.lib())
    try:
        yield
    finally:
        L._lib = mine


def close(got, ref, what, units=1):
    """Within `units` bf16 units of the reference's value plus 1e-5 of the largest; returns the bit-identical fraction.
    gate + up + SwiGLU rounds g and u to bf16 before their product is rounded: a flip of either moves the result by up to two
    units (the reference's own test allows "one BF16 flip of g or u", tests/test_mova_kernels.c:213-215)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    tol = units * np.abs(ref) / 128.0 + 1e-5 * np.max(np.abs(ref)) + 1e-30
    bad = np.abs(got - ref) > tol
    assert not bad.any(), (what, int(bad.sum()), float(np.max(np.abs(got - ref) / tol)))
    return float(np.mean(got == ref))


def test_config1_decode_step_kernel_by_kernel(oracle):
    """BASELINE config 1 (d 2048, ff 512, top-8) at M = 8 with 24 experts: router, gate + up + SwiGLU, down, combine."""
    from nanoseedlm_b200 import kernels, moe
    d, ff, E, k, T = 2048, 512, 24, 8, 8
    h = moe.HostLayer(oracle, d, ff, E, seed=5)
    lay = moe.DeviceLayer.from_host(h)
    x = oracle.normal(3, T * d, bf16=True).reshape(T, d)
    logits = oracle.normal(4, T * E).reshape(T, E)
    ind, wt = kernels.kt_route_cfg(logits, k)
    a = kernels.kt_mv_gu(lay.gate, lay.up, ind.ravel(), k, x)
    dn = kernels.kt_mv_sel(lay.down, ind.ravel(), 1, a)
    sh, sg = np.zeros((T, d), np.float32), np.zeros(T, np.float32)
    out = kernels.kt_q4_moe_combine(dn, wt, sh, sg, T, d, k)
    with reference_kernels():
        rind, rwt = kernels.kt_route_cfg(logits, k)
        ra = kernels.kt_mv_gu(lay.gate, lay.up, rind.ravel(), k, x)
        rdn_same_in = kernels.kt_mv_sel(lay.down, rind.ravel(), 1, a)      # the down projection on identical inputs
        rdn = kernels.kt_mv_sel(lay.down, rind.ravel(), 1, ra)
        rout = kernels.kt_q4_moe_combine(rdn, rwt, sh, sg, T, d, k)
    assert np.array_equal(ind, rind)
    assert np.max(np.abs(wt - rwt) / rwt) < 1e-6
    same = [close(a, ra, "gate+up", units=2), close(dn, rdn_same_in, "down")]
    assert min(same) > 0.98, same      # all but rare bf16 rounding flips are bit-identical
    # the whole step: this library's fused launches (router in the gate+up kernel's prologue) against the reference's four
    m = moe.Moe(lay, k, T)
    fused, find = m.forward_host(x, logits)
    m.close()
    assert np.array_equal(find.reshape(T, k), rind)
    assert np.max(np.abs(fused - rout)) <= 2e-3 * np.max(np.abs(rout))      # bf16 flips of the activations pass through down
    assert np.mean(np.abs(fused - rout) <= 1e-5 * np.max(np.abs(rout))) > 0.9


@pytest.mark.parametrize("P", [1, 8, 64, 200])
def test_gather_lists_of_every_kernel_regime(oracle, P):
    """1, 8, 64 pairs (the pair kernel) and 200 (the grouped kernel) against the reference's one-block-per-(row tile, pair) grid."""
    from nanoseedlm_b200 import kernels, moe
    d, ff, E, k = 512, 128, 16, 4
    h = moe.HostLayer(oracle, d, ff, E, seed=8)
    lay = moe.DeviceLayer.from_host(h)
    rng = np.random.default_rng(P)
    sel = rng.integers(0, E, P).astype(np.int32)
    x = oracle.normal(P, ((P + k - 1) // k) * d, bf16=True).reshape(-1, d)
    a = kernels.kt_mv_gu(lay.gate, lay.up, sel, k, x)
    dn = kernels.kt_mv_sel(lay.down, sel, 1, a)
    with reference_kernels():
        ra = kernels.kt_mv_gu(lay.gate, lay.up, sel, k, x)
        rdn = kernels.kt_mv_sel(lay.down, sel, 1, a)
    close(a, ra, "gate+up", units=2)
    close(dn, rdn, "down")


def test_prompt_rows_grouping_and_grouped_gemm(oracle):
    """96 rows x top-4 over 8 experts: kc_bucket's permutation and tile table identical, the grouped GEMM within the bf16 bound."""
    from nanoseedlm_b200 import kernels, moe
    d, ff, E, k, T = 256, 128, 8, 4, 96
    h = moe.HostLayer(oracle, d, ff, E, seed=11)
    lay = moe.DeviceLayer.from_host(h)
    x = oracle.normal(5, T * d, bf16=True).reshape(T, d)
    ind, _ = kernels.kt_route(oracle.normal(6, T * E).reshape(T, E), k)
    perm, tiles, nt = kernels.kt_bucket(ind, E)
    y = kernels.kt_mm_grouped(lay.gate, T * k, k, perm, tiles, x, mode="dev")
    with reference_kernels():
        rperm, rtiles, rnt = kernels.kt_bucket(ind, E)
        ry = kernels.kt_mm_grouped(lay.gate, T * k, k, perm, tiles, x, mode="dev")
    assert np.array_equal(perm, rperm) and tiles == rtiles and nt == rnt
    close(y, ry, "grouped GEMM")


def test_decode_attention_reference_case(oracle):
    """GQA 8 / 2 (the reference's kernel serves groups of 4), three ragged rows, five splits, BF16 and 8-bit caches."""
    from nanoseedlm_b200 import kernels, lib as L
    from oracle import binding as B
    rng = np.random.default_rng(2)
    nh, nkv, NP, pos, kv0, ns = 8, 2, 640, [300, 299, 37], [0, 310, 600], 5
    q = B.bfr((rng.random((3, nh, 128), np.float32) * 2 - 1) * 2)
    g = B.bfr((rng.random((3, nh, 128), np.float32) * 2 - 1) * 3)
    Kc = B.f2bf((rng.random((NP, nkv, 128), np.float32) * 2 - 1) * 2)
    Vc = B.f2bf(rng.random((NP, nkv, 128), np.float32) * 2 - 1)
    a = L.AttnArgs(nh, nkv, (301 + 4) // 5, ns, float(1 / np.sqrt(128.0)))
    kq, ks, _ = B.kv_q8_cache(Kc)
    vq, vs, _ = B.kv_q8_cache(Vc)
    mine = [kernels.kt_attn(a, q, Kc, Vc, pos, kv0, g, None), kernels.kt_attn(a, q, kq, vq, pos, kv0, g, None, scales=(ks, vs))]
    with reference_kernels():
        ref = [kernels.kt_attn(a, q, Kc, Vc, pos, kv0, g, None), kernels.kt_attn(a, q, kq, vq, pos, kv0, g, None, scales=(ks, vs))]
    for o, r in zip(mine, ref):
        bound = np.abs(r) / 128 + 2e-6      # the reference test's bound (tests/test_mova_kernels.c:660-715)
        assert (np.abs(o - r) <= 2 * bound).all() and np.mean(np.abs(o - r) > bound) <= 1e-3


def test_reference_kernels_pass_this_suites_checks(oracle, golden):
    """The oracle-based expectations of this suite hold for the reference's own kernels."""
    import test_gpu_attn
    import test_gpu_cache
    import test_gpu_gemm
    import test_gpu_misc
    import test_gpu_mv
    with reference_kernels():
        test_gpu_misc.test_route_512_experts_top10_with_tie(oracle, golden)
        for T, E, k in ((1, 128, 8), (8, 128, 8), (64, 512, 10), (3, 1024, 32)):
            test_gpu_misc.test_route_shapes(oracle, T, E, k)
        for n, rows, k in ((128, 512, 10), (512, 64, 10), (4, 1, 1)):
            test_gpu_misc.test_bucket_against_host_grouping(oracle, n, rows, k)
        test_gpu_misc.test_swiglu_and_combines(oracle)
        for K in (256, 512, 4096):      # the reference's own K list (tests/test_mova_kernels.c:161)
            test_gpu_mv.test_mv_dense_tokens_add_and_batch_invariance(oracle, K)
        test_gpu_cache.test_cache_admit_copy_and_identical_results(oracle)
        test_gpu_gemm.test_mm_grouped_tile_table(oracle, False, "dev")
        test_gpu_attn.run_variant(0, 8, 2, 640, [300, 299, 37], [0, 310, 600], 5, (301 + 4) // 5, True, None, 21, strict=True)


def test_reference_kernels_pass_the_checks_either_side_of_the_path(oracle):
    """The same for the kernels around the seed products, at the sizes the reference's kernels serve: its router holds
    n <= 128 experts and top_k <= 16 (engine/kernels_moe.cu:742-772), its per-head mat-vec T <= 8 rows
    (engine/kernels_moe.cu:2437-2440), its GEMM K a multiple of 32 (engine/kernels_cuda.h:118)."""
    import test_gpu_decoder
    import test_gpu_gemm
    import test_gpu_mova
    import test_gpu_mv
    import test_gpu_q4
    from nanoseedlm_b200 import kernels, lib as L
    with reference_kernels():
        for d, n, k, T in ((512, 20, 4, 5), (2048, 128, 8, 8), (2048, 100, 8, 3)):
            test_gpu_mova.test_router(kernels, L, d, n, k, T)
        for n, k in ((100, 8), (64, 4), (1, 1)):
            test_gpu_mova.test_router_topk_ties_to_lowest_id(kernels, L, n, k)
        for O, I, T, gate in ((96, 128, 3, 0), (128, 192, 5, 1), (6144, 128, 2, 1), (33, 2048, 4, 0)):
            test_gpu_mova.test_heads_mv(kernels, O, I, T, gate)
        for O, I in ((96, 128), (128, 192)):
            test_gpu_mova.test_heads_deq_bit_exact(kernels, O, I)
        for R, K in ((24, 256), (24, 4096), (37, 2048), (1000, 64), (16, 8192)):
            test_gpu_q4.test_q4_dense_tokens_add_and_batch_invariance(R, K)
        for V, n in ((151936, 3), (1000, 5), (7, 2)):
            test_gpu_q4.test_argmax_ties_to_the_lowest_id_and_probability(V, n)
        for R, K in ((24, 256), (24, 512), (512, 2048), (24, 136)):
            test_gpu_mv.test_mv_gather(oracle, R, K)
        for R, K in ((24, 256), (512, 2048), (24, 72)):
            test_gpu_mv.test_mv_gate_up_swiglu(oracle, R, K)
        for exact in (False, True):
            for R, K, T in ((40, 128, 45), (128, 64, 16), (300, 512, 130)):
                test_gpu_gemm.test_mm_dense_residual(oracle, exact, R, K, T)
        test_gpu_decoder.test_small_kernels_alone(oracle)


@contextlib.contextmanager
def stream_table_24_bits():
    """The table the reference's hosts pass with MF_SEED4 tensors: lfsr_stream24 = the low 24 bits of the 32-bit table
    (nslm/lfsr.h:40-49; engine/qwen4_cuda.c:265)."""
    import torch
    from nanoseedlm_b200 import kernels
    g32 = kernels.stream_table()
    d = torch.cuda.current_device()
    kernels._table[d] = kernels.dev(g32.cpu().numpy().view(np.uint32) & np.uint32(0xFFFFFF))
    try:
        yield
    finally:
        kernels._table[d] = g32


def test_p3_format_against_the_reference_kernels_with_the_24_bit_table(oracle):
    """MF_SEED4 (P = 3): this library with the 24-bit table == this library with the 32-bit table, bit for bit (it reads no
    stream bit beyond 23 for this format), and within the bf16 bound of the reference's own P = 3 kernels, for the dense
    mat-vec (1 and 5 tokens), the gather and gate + up at the tuned kernel's shapes, and the grouped GEMM."""
    from nanoseedlm_b200 import kernels
    from oracle import binding as B
    R, K, S = 96, 512, 4
    mats = [B.Matrix3(R, K, 500 + s, eb=-20 - s % 2) for s in range(S)]
    mu = [B.Matrix3(R, K, 600 + s, eb=-21 + s % 2) for s in range(S)]
    w, wu = kernels.SeedWeight3(mats), kernels.SeedWeight3(mu)
    rng = np.random.default_rng(17)
    x = B.bfr(rng.standard_normal((6, K)).astype(np.float32))
    sel = rng.integers(0, S, 12)
    perm, tiles = [], []
    for s in range(S):
        st = len(perm)
        perm += [p for p in range(12) if sel[p] == s]
        if len(perm) > st:
            tiles.append((s, st, len(perm) - st))

    def run():
        return [kernels.kt_mv3(w, x[:1], 1), kernels.kt_mv3(w, x[:5], 5), kernels.kt_mv3_sel(w, sel, 2, x), kernels.kt_mv3_gu(w, wu, sel, 2, x),
                kernels.kt_mm_grouped(w, 12, 2, perm, tiles, x, mode="dev")]

    wide = run()
    with stream_table_24_bits():
        narrow = run()
        with reference_kernels():
            ref = run()
    for a, b in zip(wide, narrow):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    for i, (a, r) in enumerate(zip(narrow, ref)):
        close(a, r, f"P = 3 case {i}", units=2 if i == 3 else 1)
