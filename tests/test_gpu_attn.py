"""Decode attention over a BF16 or 8-bit KV cache (kc_attn) against a double-precision reference.

The first case is the reference's own kernel test (tests/test_mova_kernels.c:660-715): GQA 8/2, three rows at
positions 300, 299, 37 in sequence slots based at cache rows 0, 310, 600, five splits; bound |o - ref| <= |ref| / 128 + 2e-6,
met by EVERY output as in the reference's test.  The same strict bound holds for every other case here when there is no
output gate.  With the gate the attention value is rounded to bf16 twice (before and after the gate, as the reference
does): where f32 summation noise flips the first rounding the second can land one unit further, which happens to 1-2
outputs in 10,000 of the larger cases (up to 1.33 x the bound measured); those cases allow one output in a thousand beyond
the bound and none beyond twice it.  Every case also runs on the 8-bit cache built from the same values as the
reference's test builds it (tests/test_mova_kernels.c:584-604, 688)."""
import numpy as np
import pytest

from oracle import binding as B

pytestmark = pytest.mark.gpu


def run_case(nh, nkv, NP, pos, kv0, ns, chunk, gate=True, nv=None, seed=21, strict=False):
    for invariant in (0, 1):      # the step's keys dealt evenly to the blocks (default); a block per caller split
        run_variant(invariant, nh, nkv, NP, pos, kv0, ns, chunk, gate, nv, seed, strict=strict)
        run_variant(invariant, nh, nkv, NP, pos, kv0, ns, chunk, gate, nv, seed, q8=True, strict=strict)      # the 8-bit cache
        if gate:                  # the same without the output gate: one rounding, the strict bound
            run_variant(invariant, nh, nkv, NP, pos, kv0, ns, chunk, False, nv, seed)


def run_variant(variant, nh, nkv, NP, pos, kv0, ns, chunk, gate, nv, seed, q8=False, strict=False):
    from nanoseedlm_b200 import kernels, lib as L
    L.load().nsl_attn_batch_invariant(variant)
    rng = np.random.default_rng(seed)
    T = len(pos)
    q = B.bfr((rng.random((T, nh, 128), np.float32) * 2 - 1) * 2)
    g = B.bfr((rng.random((T, nh, 128), np.float32) * 2 - 1) * 3)
    Kc = B.f2bf((rng.random((NP, nkv, 128), np.float32) * 2 - 1) * 2)
    Vc = B.f2bf(rng.random((NP, nkv, 128), np.float32) * 2 - 1)
    scale = np.float32(1 / np.sqrt(128.0))
    a = L.AttnArgs(nh, nkv, chunk, ns, float(scale))
    if q8:      # the cache quantized per (row, head); the reference sees the values the kernel reads, bf16(code * scale)
        kq, ks, Kc = B.kv_q8_cache(Kc)
        vq, vs, Vc = B.kv_q8_cache(Vc)
        o = kernels.kt_attn(a, q, kq, vq, pos, kv0, g if gate else None, nv, scales=(ks, vs))
    else:
        o = kernels.kt_attn(a, q, Kc, Vc, pos, kv0, g if gate else None, nv)
    ref, _ = B.attn_decode(q, Kc, Vc, pos, kv0, nkv, scale, g if gate else None)
    L.load().nsl_attn_batch_invariant(0)      # back to the default
    bound = np.abs(ref) / 128 + 2e-6      # the reference's bound
    bad = np.abs(o - ref) > bound
    if strict or not gate:
        assert not bad.any(), (variant, q8, int(bad.sum()), float(np.max(np.abs(o - ref) / bound)))
    else:      # an output whose attention value sits on a bf16 rounding boundary can land one unit further after the gate's second rounding
        assert bad.mean() <= 1e-3, (variant, int(bad.sum()), float(np.max(np.abs(o - ref))))
        assert (np.abs(o - ref) <= 2 * bound).all(), (variant, float(np.max(np.abs(o - ref) / bound)))


def test_reference_case_gqa_8_over_2():
    run_case(8, 2, 640, [300, 299, 37], [0, 310, 600], 5, (301 + 4) // 5, strict=True)


@pytest.mark.parametrize("nh,nkv", [(16, 2), (4, 4), (32, 2), (3, 1)])
def test_group_sizes(nh, nkv):
    run_case(nh, nkv, 700, [511, 0, 33, 64], [0, 600, 620, 512], 4, 128, seed=nh)


def test_ragged_rows_as_the_reference_host_splits_them():
    """12 rows of very different lengths, 32 splits of >= 128 keys (engine/mova_cuda.c:1040-1045): in the balanced form a
    block's units span several rows and a long row's units many blocks."""
    rng = np.random.default_rng(3)
    pos = [2999, 0, 15, 16, 1500, 127, 128, 2047, 700, 31, 2998, 5]
    run_case(8, 2, 12 * 3008, pos, [3008 * i for i in range(12)], 32, 128, seed=9)
    run_variant(0, 16, 1, 6000, [5999], [0], 32, 188, True, None, 4)      # one row, one KV head: its units over 30 blocks


def test_a_row_alone_and_in_a_batch():
    """With nsl_attn_batch_invariant(1) a row's output is bit-identical whatever rows share the call (its keys are cut by its
    own position alone, as the reference cuts them: engine/kernels_moe.cu:887-952); the default balanced form cuts a row's
    keys by the whole step's load, so alone and batched agree only within the kernel's bound."""
    from nanoseedlm_b200 import kernels, lib as L
    rng = np.random.default_rng(12)
    nh, nkv, ns, chunk = 8, 2, 16, 128
    pos = [1900, 7, 640, 1203, 64, 1999]
    kv0 = [2000 * i for i in range(len(pos))]
    NP = 2000 * len(pos)
    q = B.bfr((rng.random((len(pos), nh, 128), np.float32) * 2 - 1) * 2)
    g = B.bfr((rng.random((len(pos), nh, 128), np.float32) * 2 - 1) * 3)
    Kc = B.f2bf((rng.random((NP, nkv, 128), np.float32) * 2 - 1) * 2)
    Vc = B.f2bf(rng.random((NP, nkv, 128), np.float32) * 2 - 1)
    a = L.AttnArgs(nh, nkv, chunk, ns, float(1 / np.sqrt(128.0)))
    ref, _ = B.attn_decode(q, Kc, Vc, pos, kv0, nkv, np.float32(1 / np.sqrt(128.0)), g)
    try:
        for on in (1, 0):
            L.load().nsl_attn_batch_invariant(on)
            batch = kernels.kt_attn(a, q, Kc, Vc, pos, kv0, g, None)
            for t in (0, 3, 5):
                alone = kernels.kt_attn(a, q[t:t + 1], Kc, Vc, pos[t:t + 1], kv0[t:t + 1], g[t:t + 1], None)
                if on:
                    assert np.array_equal(alone[0].view(np.uint32), batch[t].view(np.uint32)), t
                else:
                    assert (np.abs(alone[0] - batch[t]) <= 2 * (np.abs(ref[t]) / 128 + 2e-6)).all(), t
    finally:
        L.load().nsl_attn_batch_invariant(0)


def test_one_split_no_gate_and_two_segments():
    run_case(8, 2, 640, [300, 299, 37], [0, 310, 600], 1, 0, gate=False)
    run_case(8, 2, 640, [300, 299, 37], [0, 310, 600], 3, 64, nv=320, seed=5)      # positions >= 320 live in segment b


def test_refuses_other_cache_formats_and_groups():
    import torch
    from nanoseedlm_b200 import lib as L
    kv = L.KvView()
    kv.fmt = 2      # FP8: the MLA caches' format
    L.load().kc_attn(None, L.AttnArgs(8, 2, 64, 2, 0.1), None, kv, None, None, None, None, 1)
    with pytest.raises(RuntimeError, match="format 2"):
        L.check()
    kv.fmt = 0
    L.load().kc_attn(None, L.AttnArgs(64, 2, 64, 2, 0.1), None, kv, None, None, None, None, 1)
    with pytest.raises(RuntimeError, match="groups of"):
        L.check()
