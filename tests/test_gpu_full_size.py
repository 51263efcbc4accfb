"""Parity at the sizes the bench's numbers come from: BASELINE config 2 (hidden 2048, 128 experts of intermediate 512, top-8,
512 prompt rows -> 4096 pairs through the grouped tcgen05 GEMM, 32 K-steps per tile) and config 3 (512 experts, top-10,
64 rows through the expert-parallel step).  Everything is checked against the CPU oracle on oracle-generated weights,
through the C ABI; nothing here compares the CUDA path with itself."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

D, FF = 2048, 512


def bfr(a):
    a = np.asarray(a, np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def close_bf(got, ref, extra):
    return np.abs(got.astype(np.float64) - ref) <= np.abs(ref) / 128.0 + 1e-30 + extra


def stack(kernels, st, R, K):
    return kernels.SeedWeight(st["seeds"], st["coefs"], st["codes"], st["eb"], R, K)


def weights_f64(oracle, h, which, e, exact):
    w = oracle.decode_rows_f32(h.matrix(oracle, which, e))
    return (w if exact else bfr(w)).astype(np.float64)


@pytest.fixture(scope="module")
def cfg2(oracle):
    from nanoseedlm_b200 import moe
    E, k, M = 128, 8, 512
    h = moe.HostLayer(oracle, D, FF, E, seed=202)
    x = oracle.normal(2021, M * D, bf16=True).reshape(M, D)
    logits = oracle.normal(2022, M * E).reshape(M, E)
    ind, wt = oracle.route(logits, k)
    return {"h": h, "x": x, "logits": logits, "ind": ind, "wt": wt, "E": E, "k": k, "M": M}


def picked_tiles(tiles):
    """At least eight tile entries: the smallest and the largest pair count, one whose count is not a multiple of 16, and
    a spread of the others."""
    by_count = sorted(tiles, key=lambda t: t[2])
    odd = [t for t in tiles if t[2] % 16]
    pick = {by_count[0], by_count[-1]} | set(odd[:2]) | set(tiles[:: max(1, len(tiles) // 6)][:6])
    return sorted(pick)


@pytest.mark.parametrize("exact", [False, True])
def test_config2_grouped_gemm_tiles_against_oracle(oracle, cfg2, exact):
    """kc_bucket + kc_mm_grouped_dev at config-2 size (4096 pairs, 128 tile entries, K = 2048: the stage ring of the
    tcgen05 pipeline wraps ten times), gate projection, and the down projection (K = 512, 2048 rows: 16 row tiles per
    entry) on a bf16-valued activation matrix; picked tile entries against the oracle's decode and a double-precision
    product, both weight modes."""
    from nanoseedlm_b200 import kernels
    h, x, ind, k, E, M = (cfg2[n] for n in ("h", "x", "ind", "k", "E", "M"))
    P = M * k
    perm, tiles, nt = kernels.kt_bucket(ind, E)
    rperm, rtiles = oracle.bucket(ind, E)
    assert np.array_equal(perm, rperm) and tiles == rtiles and nt == len(rtiles) == E      # every expert is hit at this size
    assert sorted(perm.tolist()) == list(range(P))
    y = kernels.kt_mm_grouped(stack(kernels, h.gate, FF, D), P, k, perm, tiles, x, exact=exact, mode="dev")
    a_in = oracle.normal(2023, P * FF, bf16=True).reshape(P, FF)
    yd = kernels.kt_mm_grouped(stack(kernels, h.down, D, FF), P, 1, perm, tiles, a_in, exact=exact, mode="dev")
    chosen = picked_tiles(tiles)
    assert len(chosen) >= 8 and any(c % 16 for _, _, c in chosen)
    for e, start, count in chosen:
        pairs = perm[start:start + count]
        xs = x[pairs // k].astype(np.float64)
        w = weights_f64(oracle, h, "gate", e, exact)
        acc, mag = xs @ w.T, np.abs(xs) @ np.abs(w).T
        ok = close_bf(y[pairs], bfr(acc.astype(np.float32)).astype(np.float64), 64 * 1.2e-7 * mag)
        assert ok.all(), (e, count, np.argwhere(~ok)[:4])
        w = weights_f64(oracle, h, "down", e, exact)
        xs = a_in[pairs].astype(np.float64)
        acc, mag = xs @ w.T, np.abs(xs) @ np.abs(w).T
        ok = close_bf(yd[pairs], bfr(acc.astype(np.float32)).astype(np.float64), 64 * 1.2e-7 * mag)
        assert ok.all(), (e, count, np.argwhere(~ok)[:4])


def test_config2_layer_rows_against_oracle(oracle, cfg2):
    """The whole prompt path of the layer at config-2 size through the C host layer: routing identical to the oracle's for
    all 512 rows; four rows' outputs against the oracle composed with the prompt path's rounding points (seed weights
    rounded to bf16, every GEMM output stored as bf16, SwiGLU on those, plain-f32 combine in rank order)."""
    from nanoseedlm_b200 import moe
    h, x, logits, ind, wt, k, M = (cfg2[n] for n in ("h", "x", "logits", "ind", "wt", "k", "M"))
    layer = moe.DeviceLayer.from_host(h)
    m = moe.Moe(layer, k, M)
    out, got_ind = m.forward_host(x, logits)
    assert np.array_equal(got_ind, ind)
    for t in (0, 17, 255, 511):
        acc = np.zeros(D, np.float32)
        for j in range(k):
            e = int(ind[t, j])
            xt = x[t].astype(np.float64)
            g = bfr((weights_f64(oracle, h, "gate", e, False) @ xt).astype(np.float32))
            u = bfr((weights_f64(oracle, h, "up", e, False) @ xt).astype(np.float32))
            a = oracle.swiglu(g, u)
            dn = bfr((weights_f64(oracle, h, "down", e, False) @ a.astype(np.float64)).astype(np.float32))
            acc = acc + wt[t, j] * dn
        scale = np.max(np.abs(acc))
        assert np.max(np.abs(out[t] - acc)) <= 4e-3 * scale       # a bf16 flip of one intermediate moves an output by < 1 bf16 ulp
        assert np.mean(np.abs(out[t] - acc) <= 1e-5 * scale) > 0.85   # four bf16 stores in a row over K = 2048: more flips than at decode
    # and against the CPU reference forward (f32 weights, no rounding points): the prompt path's bf16 weights and stores
    ref, rind, _ = oracle.moe_layer(h, x[:2], logits[:2], k)
    assert np.array_equal(rind, ind[:2])
    assert np.max(np.abs(out[:2] - ref)) <= 2e-2 * np.max(np.abs(ref))
    m.close()


@pytest.fixture(scope="module")
def cfg3(oracle):
    from nanoseedlm_b200 import moe
    E, k, B = 512, 10, 64
    h = moe.HostLayer(oracle, D, FF, E, seed=303)
    x = oracle.normal(3031, B * D, bf16=True).reshape(B, D)
    logits = oracle.normal(3032, B * E).reshape(B, E)
    ref, ind, wt = oracle.moe_layer(h, x, logits, k)      # the CPU reference forward: double sums, no rounding points
    return {"h": h, "x": x, "logits": logits, "ref": ref, "ind": ind, "E": E, "k": k, "B": B}


@pytest.mark.parametrize("ranks", [1, 8])
def test_config3_expert_parallel_step_against_oracle(oracle, cfg3, ranks):
    """The expert-parallel step at config-3 size (512 experts, top-10, 64 rows) against oracle.moe_layer directly: with one
    rank (all experts local), and with eight ranks' windows in one process, every rank's producers issued before any
    rank's consumers on one stream.  f32 throughout (no bf16 rounding points), the 1e-3 bar, identical routing ids."""
    import torch
    from nanoseedlm_b200 import ep, lib, moe
    h, x, logits, ref, ind, E, k, B = (cfg3[n] for n in ("h", "x", "logits", "ref", "ind", "E", "k", "B"))
    t_loc, e_loc = B // ranks, E // ranks
    wins = ep.P2PWindow.local_group(ranks, t_loc, D, k)
    eps = [ep.ExpertParallelMoe(ep.CudaBackend(moe.DeviceLayer.from_host(h, r * e_loc, (r + 1) * e_loc), rounding=False), D, k, E, t_loc,
                                collectives="p2p", window=wins[r]) for r in range(ranks)]
    dx, dl = torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda()
    for step in range(2):      # twice: the second step runs on the counters and epochs the first one left
        for r, e in enumerate(eps):
            e.be.route_pack_dispatch(e, dx[r * t_loc:(r + 1) * t_loc], dl[r * t_loc:(r + 1) * t_loc])
        for e in eps:
            e.be.local_experts(e)
        for e in eps:
            e.be.reduce(e)
        torch.cuda.synchronize()
        out = np.concatenate([e.out.cpu().numpy() for e in eps])
        got_ind = np.concatenate([e.be.ind.cpu().numpy() for e in eps])
        assert np.array_equal(got_ind, ind)
        err = np.max(np.abs(out - ref)) / np.max(np.abs(ref))
        assert err <= 1e-3, err
        assert err <= 5e-5, err      # what f32 accumulation actually gives
    assert sum(int(e.be.count.item()) for e in eps) == B * k
    assert all(w.status() == 0 for w in wins)
    lib.check()
    for w in wins:
        w.close()
