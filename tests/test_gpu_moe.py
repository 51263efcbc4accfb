"""One MoE expert layer through the C host layer (include/nslm_moe.h) against the oracle.

Two comparisons: (1) with the engine's bf16 rounding points, against the oracle composed with the same points;
(2) f32 throughout, against the CPU reference forward's arithmetic (double sums, no rounding) at the 1e-3 relative bar
with identical top-k routing indices."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def engine_rounding_reference(oracle, h, x, logits, k):
    """route -> per pair a = mv_gu, D = bf16(down a) -> out = sum_j wt_j D_j (plain f32), as the engine's kernels round."""
    T = x.shape[0]
    ind, wt = oracle.route(logits, k)
    out = np.zeros((T, h.d), np.float32)
    for t in range(T):
        acc = np.zeros(h.d, np.float32)
        for j in range(k):
            e = int(ind[t, j])
            a = oracle.mv_gu(h.matrix(oracle, "gate", e), h.matrix(oracle, "up", e), x[t])
            D = oracle.mv(h.matrix(oracle, "down", e), a)[0]
            acc = acc + wt[t, j] * D
        out[t] = acc
    return out, ind


@pytest.mark.parametrize("d,ff,E,k,T", [(256, 64, 16, 4, 1), (256, 64, 16, 4, 8), (512, 128, 24, 8, 5), (2048, 512, 12, 8, 2)])
def test_moe_layer_decode_rows(oracle, d, ff, E, k, T):
    from nanoseedlm_b200 import moe
    h = moe.HostLayer(oracle, d, ff, E, seed=d + T)
    layer = moe.DeviceLayer.from_host(h)
    m = moe.Moe(layer, k, 8)
    x = oracle.normal(1 + T, T * d, bf16=True).reshape(T, d)
    logits = oracle.normal(2 + T, T * E).reshape(T, E)
    # (1) engine rounding points
    out, ind = m.forward_host(x, logits)
    ref, rind = engine_rounding_reference(oracle, h, x, logits, k)
    assert np.array_equal(ind, rind)
    scale = np.max(np.abs(ref))
    assert np.max(np.abs(out - ref)) <= 4e-3 * scale        # a bf16 flip of one intermediate moves an output by < 1 bf16 ulp
    assert np.mean(np.abs(out - ref) <= 1e-5 * scale) > 0.97
    # (2) f32 throughout vs the CPU reference forward
    m.set_rounding(False)
    out32, ind32 = m.forward_host(x, logits)
    ref64, rind64, _ = oracle.moe_layer(h, x, logits, k)
    assert np.array_equal(ind32, rind64)
    assert np.max(np.abs(out32 - ref64)) <= 1e-3 * np.max(np.abs(ref64))
    assert np.max(np.abs(out32 - ref64)) <= 2e-5 * np.max(np.abs(ref64))   # what f32 accumulation actually gives
    m.close()


def test_moe_full_size_config1_properties(oracle):
    """BASELINE config 1 at full size (hidden 2048, 128 experts of 512, top-8, M = 8): size-independent checks --
    routing equals the oracle's, the layer is linear in the routing weights' experts (a token routed alone equals the
    same token inside the batch, bit for bit), and one token's output equals the oracle's on its 8 experts."""
    import torch
    from nanoseedlm_b200 import moe
    d, ff, E, k, M = 2048, 512, 128, 8, 8
    gen = torch.Generator(device="cuda").manual_seed(7)
    layer = moe.DeviceLayer.random_on_device(d, ff, E, gen)
    m = moe.Moe(layer, k, M)
    x = oracle.normal(11, M * d, bf16=True).reshape(M, d)
    logits = oracle.normal(12, M * E).reshape(M, E)
    out, ind = m.forward_host(x, logits)
    rind, rwt = oracle.route(logits, k)
    assert np.array_equal(ind, rind)
    for t in (0, 5):
        o1, i1 = m.forward_host(x[t:t + 1], logits[t:t + 1])
        assert np.array_equal(i1[0], ind[t]) and np.array_equal(o1[0].view(np.uint32), out[t].view(np.uint32))
    # token 3 against the oracle on the experts it routes to (weights copied back from the device)
    t = 3
    acc = np.zeros(d, np.float32)
    for j in range(k):
        e = int(ind[t, j])
        mats = []
        for st, (R, K) in ((layer.gate, (ff, d)), (layer.up, (ff, d)), (layer.down, (d, ff))):
            mm = oracle.Matrix(R, K, 0, eb=st.eb[e])
            mm.seeds[:] = st.seeds[e].cpu().numpy().view(np.uint16)
            mm.coefs[:] = st.coefs[e].cpu().numpy().view(np.uint16)
            mm.codes[:] = st.codes[e].cpu().numpy()
            mats.append(mm)
        a = oracle.mv_gu(mats[0], mats[1], x[t])
        acc = acc + rwt[t, j] * oracle.mv(mats[2], a)[0]
    assert np.max(np.abs(out[t] - acc)) <= 4e-3 * np.max(np.abs(acc))
    m.close()


def test_pinned_forward_in_two_halves_with_two_handles(oracle):
    """submit + wait on two handles used alternately (two steps in flight) give forward_host's results bit for bit."""
    from nanoseedlm_b200 import moe
    d, ff, E, k, T = 256, 64, 16, 4, 6
    h = moe.HostLayer(oracle, d, ff, E, seed=91)
    layer = moe.DeviceLayer.from_host(h)
    ms = (moe.Moe(layer, k, 8), moe.Moe(layer, k, 8))
    xs = [oracle.normal(40 + i, T * d, bf16=True).reshape(T, d) for i in range(5)]
    ls = [oracle.normal(50 + i, T * E).reshape(T, E) for i in range(5)]
    want = [ms[0].forward_host(x, l)[0].copy() for x, l in zip(xs, ls)]
    got = []

    def submit(i):
        m = ms[i & 1]
        m.hx[:T], m.hlogits[:T] = xs[i], ls[i]
        m.submit_pinned(T)

    submit(0)
    for i in range(1, 5):
        submit(i)
        ms[(i - 1) & 1].wait()
        got.append(ms[(i - 1) & 1].hout[:T].copy())
    ms[0].wait()
    got.append(ms[0].hout[:T].copy())
    for g, w in zip(got, want):
        assert np.array_equal(g, w)
    for m in ms:
        m.close()


def test_full_batch_from_the_callers_pinned_block_and_both_result_paths(oracle):
    """nsl_moe_submit_block (rows then logits in the caller's pinned memory, one copy) and the pinned forms with the result
    stored by the combine kernel or brought by a copy: all bit-equal to forward_host."""
    import torch
    from nanoseedlm_b200 import moe
    d, ff, E, k, T = 256, 64, 16, 4, 8
    layer = moe.DeviceLayer.from_host(moe.HostLayer(oracle, d, ff, E, seed=93))
    m = moe.Moe(layer, k, T)
    x = oracle.normal(60, T * d, bf16=True).reshape(T, d)
    lg = oracle.normal(61, T * E).reshape(T, E)
    want = m.forward_host(x, lg)[0].copy()
    block = torch.cat([torch.from_numpy(x).reshape(-1), torch.from_numpy(lg).reshape(-1)]).pin_memory()
    for direct in (1, 0):
        m.set_direct_output(direct)
        m.hout[:] = 0
        m.forward_block(block)
        assert np.array_equal(m.hout[:T], want)
        m.hout[:] = 0
        m.hx[:T], m.hlogits[:T] = x, lg
        m.forward_pinned(T)
        assert np.array_equal(m.hout[:T], want)
        m.hout[:] = 0
        m.hx[:5], m.hlogits[:5] = x[:5], lg[:5]      # fewer rows than the layer holds: two copies
        m.forward_pinned(5)
        assert np.array_equal(m.hout[:5], want[:5])
    m.close()


def test_dependent_launches_change_nothing(oracle):
    """The decode path with programmatic dependent launches (the default) and with ordinary launches: the same bits,
    directly and replayed from a CUDA graph of several steps."""
    import torch
    from nanoseedlm_b200 import moe
    d, ff, E, k, T = 512, 128, 24, 8, 8
    h = moe.HostLayer(oracle, d, ff, E, seed=17)
    layer = moe.DeviceLayer.from_host(h)
    m = moe.Moe(layer, k, 8)
    xs = [oracle.normal(60 + i, T * d, bf16=True).reshape(T, d) for i in range(3)]
    ls = [oracle.normal(70 + i, T * E).reshape(T, E) for i in range(3)]
    m.set_dependent_launch(False)
    plain = [m.forward_host(x, l)[0].copy() for x, l in zip(xs, ls)]
    m.set_dependent_launch(True)
    for x, l, w in zip(xs, ls, plain):
        for _ in range(3):
            assert np.array_equal(m.forward_host(x, l)[0], w)
    dx = [torch.from_numpy(x).cuda() for x in xs]
    dl = [torch.from_numpy(l).cuda() for l in ls]
    outs = [torch.zeros(T, d, device="cuda") for _ in xs]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(3):
            m.forward_dev(dx[i], dl[i], outs[i], stream=stream.cuda_stream)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for rep in range(2):
                for i in range(3):
                    m.forward_dev(dx[i], dl[i], outs[i], stream=stream.cuda_stream)
        for o in outs:
            o.zero_()
        g.replay()
        stream.synchronize()
    for o, w in zip(outs, plain):
        assert np.array_equal(o.cpu().numpy(), w)
    m.close()


@pytest.mark.parametrize("d,ff,E,k", [(512, 128, 24, 8), (2048, 512, 40, 8), (256, 64, 16, 4)])
def test_the_decode_step_as_one_launch_gives_the_three_launches_bits(oracle, d, ff, E, k):
    """nsl_mv_step (router, gate + up + SwiGLU, down, combine as phases of one grid that wait on counters) against the three
    dependent launches: the same bits for every row count in turn (the counters are left clean whatever T was), with and
    without the bf16 rounding points, directly and replayed from a CUDA graph; no wait runs out."""
    import torch
    from nanoseedlm_b200 import moe
    h = moe.HostLayer(oracle, d, ff, E, seed=d + 3)
    layer = moe.DeviceLayer.from_host(h)
    m = moe.Moe(layer, k, 8)
    cases = []
    for T in (8, 1, 5, 8, 2, 1, 7):
        x = oracle.normal(90 + T, T * d, bf16=True).reshape(T, d)
        l = oracle.normal(95 + T, T * E).reshape(T, E)
        cases.append((x, l))
    for rounding in (True, False):
        m.set_rounding(rounding)
        m.set_one_launch(False)
        want = [(o.copy(), i.copy()) for o, i in (m.forward_host(x, l) for x, l in cases)]
        m.set_one_launch(True)
        for rep in range(3):
            for (x, l), (wo, wi) in zip(cases, want):
                o, i = m.forward_host(x, l)
                assert np.array_equal(i, wi)
                assert np.array_equal(o.view(np.uint32), wo.view(np.uint32))
        assert m.step_status() == 0
    m.set_rounding(True)
    x, l = cases[0]
    dx, dl, out = torch.from_numpy(x).cuda(), torch.from_numpy(l).cuda(), torch.zeros(8, d, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        m.forward_dev(dx, dl, out, stream=stream.cuda_stream)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for _ in range(4):
                m.forward_dev(dx, dl, out, stream=stream.cuda_stream)
        out.zero_()
        g.replay()
        stream.synchronize()
    m.set_one_launch(False)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), m.forward_host(x, l)[0].view(np.uint32))
    assert m.step_status() == 0
    m.close()


def test_one_launch_step_called_directly_its_status_word_and_refusals(oracle):
    """nsl_mv_step through its own entry point: the caller's sync block stays zero but for the status word; a status word
    that is already set (as after a wait that ran out) is left for the caller and does not wedge the next call; sizes it
    does not serve are refused with 0 and nothing launched."""
    import torch
    from nanoseedlm_b200 import kernels, lib as L, moe
    lib = L.load()
    d, ff, E, k, T = 512, 128, 24, 8, 6
    h = moe.HostLayer(oracle, d, ff, E, seed=31)
    layer = moe.DeviceLayer.from_host(h)
    m = moe.Moe(layer, k, 8)
    x = oracle.normal(7, T * d, bf16=True).reshape(T, d)
    logits = oracle.normal(8, T * E).reshape(T, E)
    want, wind = m.forward_host(x, logits)
    dx, dl = torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda()
    P = T * k
    A, D, out = torch.zeros(P, ff, device="cuda"), torch.zeros(P, d, device="cuda"), torch.zeros(T, d, device="cuda")
    ind, wt = torch.zeros(P, dtype=torch.int32, device="cuda"), torch.zeros(P, device="cuda")
    sync = torch.zeros(2 + T + P, dtype=torch.int32, device="cuda")
    G = kernels.stream_table()

    def call(dd=d, TT=T):
        return lib.nsl_mv_step(None, layer.gate.table.data_ptr(), layer.up.table.data_ptr(), layer.down.table.data_ptr(), dd, ff, dx.data_ptr(), d, E, k,
                               dl.data_ptr(), E, TT, ind.data_ptr(), wt.data_ptr(), A.data_ptr(), D.data_ptr(), out.data_ptr(), 0, sync.data_ptr(),
                               G.data_ptr())

    for _ in range(3):
        assert call() == 1
        torch.cuda.synchronize()
        assert not sync.cpu().numpy().any()
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
        assert np.array_equal(ind.cpu().numpy().reshape(T, k), wind)
    sync[0] = 1                      # the word a timed-out wait leaves behind
    assert call() == 1
    torch.cuda.synchronize()
    after = sync.cpu().numpy()
    assert after[0] == 1 and not after[1:].any()
    sync[0] = 0
    out.zero_()
    assert call() == 1
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert call(dd=d + 8) == 0 and call(TT=9) == 0      # not 64 * 2^j; more rows than a decode step has
    m.close()
