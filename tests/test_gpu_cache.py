"""The expert cache's admit and copy kernels (kc_cache_admit, kc_cache_copy) through the C ABI.

Checks, as the reference's engine tests do (tests/test_qwen4_engine.c:514-533: cache on / off give identical results):
the slot bookkeeping equals a host model of the policy (hits touched; misses in expert order take the least recently
used slot, lowest index on ties, never one touched by the same call), the slice tables point at the slots, the copied
bytes equal the host arena's, and the mat-vec kernels give bit-identical outputs through the cache and without it."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TICK0 = 0x40000000


class HostModel:
    def __init__(self, units, slots):
        self.unit_slot = [-1] * units
        self.slot_unit = [-1] * slots
        self.slot_last = [0] * slots
        self.tick = TICK0
        self.hits = self.misses = 0

    def admit(self, sl, per_layer, inds, protect_prev=False):
        prev = self.tick if protect_prev else None
        now = self.tick + 1
        need = sorted(set(int(i) for i in inds))
        miss = []
        for x in need:
            s = self.unit_slot[sl * per_layer + x]
            if s >= 0:
                self.slot_last[s] = now
                self.hits += 1
            else:
                miss.append(x)
        self.misses += len(miss)
        self.tick = now
        jobs = []
        for x in miss:
            cand = [(l, s) for s, l in enumerate(self.slot_last) if l != now and l != prev]
            if not cand:
                break
            _, s = min(cand)
            u = sl * per_layer + x
            if self.slot_unit[s] >= 0:
                self.unit_slot[self.slot_unit[s]] = -1
            self.slot_unit[s], self.unit_slot[u], self.slot_last[s] = u, s, now
            jobs.append((u, s))
        return jobs


def test_cache_admit_copy_and_identical_results(oracle):
    import torch
    from nanoseedlm_b200 import kernels, lib as L, moe
    lib = L.load()
    d, ff, E, NLAY, slots, k = 256, 64, 12, 2, 9, 4
    hl = [moe.HostLayer(oracle, d, ff, E, seed=40 + l) for l in range(NLAY)]
    resident = [moe.DeviceLayer.from_host(h) for h in hl]
    # unit layout: tensor i (gate, up, down), stream s (0 seeds, 1 coefs, 3 codes), offsets aligned to 256 bytes
    lens = [[ff * d // 8 * 2, ff * d // 8 * 2, 0, ff * d // 16]] * 2 + [[d * ff // 8 * 2, d * ff // 8 * 2, 0, d * ff // 16]]
    off, ub = [[0xFFFFFFFF] * 4 for _ in range(3)], 0
    for i in range(3):
        for s in range(4):
            if lens[i][s]:
                off[i][s] = ub
                ub += (lens[i][s] + 255) // 256 * 256
    units = NLAY * E
    arena = torch.zeros(units, ub, dtype=torch.uint8).pin_memory()
    an = arena.numpy()
    for l, h in enumerate(hl):
        for i, st in enumerate((h.gate, h.up, h.down)):
            for x in range(E):
                u = l * E + x
                an[u, off[i][0]:off[i][0] + lens[i][0]] = st["seeds"][x].view(np.uint8)
                an[u, off[i][1]:off[i][1] + lens[i][1]] = st["coefs"][x].view(np.uint8)
                an[u, off[i][3]:off[i][3] + lens[i][3]] = st["codes"][x]
    vram = torch.zeros(slots, ub, dtype=torch.uint8, device="cuda")
    tab_h = (L.WSlice * (NLAY * 3 * E))()
    for t in tab_h:
        t.eb = -22
    tab = torch.zeros(NLAY * 3 * E * C.sizeof(L.WSlice), dtype=torch.uint8, device="cuda")
    tab.copy_(torch.frombuffer(bytearray(bytes(tab_h)), dtype=torch.uint8))
    i32 = lambda n, v=0: torch.full((n,), v, dtype=torch.int32, device="cuda")
    unit_slot, slot_unit, slot_last = i32(units, -1), i32(slots, -1), i32(slots)
    tick, stats, jobs, njobs = i32(4), i32(4), i32(2 * E), i32(4)
    tick[0] = TICK0
    pool = L.CachePool()
    pool.unit_slot, pool.slot_unit, pool.slot_last = unit_slot.data_ptr(), slot_unit.data_ptr(), slot_last.data_ptr()
    pool.tick, pool.stats, pool.jobs, pool.njobs = tick.data_ptr(), stats.data_ptr(), jobs.data_ptr(), njobs.data_ptr()
    pool.vram, pool.host, pool.unit_bytes = vram.data_ptr(), arena.data_ptr(), ub
    pool.slots, pool.per_layer, pool.ntens, pool.tab = slots, E, 3, tab.data_ptr()
    for i in range(3):
        for s in range(4):
            pool.off[i][s] = off[i][s]
    model = HostModel(units, slots)
    G = kernels.stream_table()
    rng = np.random.default_rng(3)
    x = oracle.normal(9, 2 * d, bf16=True).reshape(2, d)
    xd = torch.from_numpy(x).cuda()
    wsz = C.sizeof(L.WSlice)
    for step in range(7):
        sl = step % NLAY
        inds = np.concatenate([rng.choice(E, k, replace=False) for _ in range(2)]).astype(np.int32)
        di = torch.from_numpy(inds).cuda()
        lib.kc_cache_admit(None, C.byref(pool), sl, di.data_ptr(), inds.size, 0)
        lib.kc_cache_copy(None, C.byref(pool), 8)
        torch.cuda.synchronize()
        L.check()
        want_jobs = model.admit(sl, E, inds)
        assert unit_slot.cpu().tolist() == model.unit_slot and slot_unit.cpu().tolist() == model.slot_unit
        assert int(njobs[0]) == len(want_jobs)
        assert [tuple(v) for v in jobs.cpu().numpy()[:2 * len(want_jobs)].reshape(-1, 2).tolist()] == want_jobs
        assert stats.cpu().tolist()[:2] == [model.hits, model.misses]
        for u, s in want_jobs:
            assert torch.equal(vram[s].cpu(), arena[u])
        # the routed experts through the cache's tables == through the all-resident layer, bit for bit
        P = inds.size
        gate_t, up_t, down_t = (tab.data_ptr() + ((sl * 3 + i) * E) * wsz for i in range(3))
        outs = []
        for (gt, ut, dt) in ((gate_t, up_t, down_t),
                             (resident[sl].gate.table.data_ptr(), resident[sl].up.table.data_ptr(), resident[sl].down.table.data_ptr())):
            A = torch.zeros(P, ff, device="cuda")
            Dx = torch.zeros(P, d, device="cuda")
            lib.kc_mv_gu(None, L.MF_SEED4P4, gt, ut, d, ff, xd.data_ptr(), d, A.data_ptr(), ff, di.data_ptr(), P, k, G.data_ptr())
            lib.kc_mv_sel(None, L.MF_SEED4P4, dt, ff, d, A.data_ptr(), ff, Dx.data_ptr(), d, di.data_ptr(), P, 1, G.data_ptr())
            torch.cuda.synchronize()
            outs.append(Dx.cpu().numpy())
        assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    assert model.hits > 0 and model.misses > slots   # both hits and evictions happened


def test_admit_stops_when_no_slot_may_be_replaced():
    import torch
    from nanoseedlm_b200 import lib as L
    lib = L.load()
    E, slots = 8, 3
    i32 = lambda n, v=0: torch.full((n,), v, dtype=torch.int32, device="cuda")
    unit_slot, slot_unit, slot_last = i32(E, -1), i32(slots, -1), i32(slots)
    tick, stats, jobs, njobs = i32(4), i32(4), i32(2 * E), i32(4)
    tick[0] = TICK0
    vram = torch.zeros(slots, 256, dtype=torch.uint8, device="cuda")
    tab = torch.zeros(E * C.sizeof(L.WSlice), dtype=torch.uint8, device="cuda")
    pool = L.CachePool()
    pool.unit_slot, pool.slot_unit, pool.slot_last = unit_slot.data_ptr(), slot_unit.data_ptr(), slot_last.data_ptr()
    pool.tick, pool.stats, pool.jobs, pool.njobs = tick.data_ptr(), stats.data_ptr(), jobs.data_ptr(), njobs.data_ptr()
    pool.vram, pool.host, pool.unit_bytes = vram.data_ptr(), 0, 256
    pool.slots, pool.per_layer, pool.ntens, pool.tab = slots, E, 1, tab.data_ptr()
    for s in range(4):
        pool.off[0][s] = 0xFFFFFFFF
    inds = torch.arange(5, dtype=torch.int32, device="cuda")   # five misses, three slots
    lib.kc_cache_admit(None, C.byref(pool), 0, inds.data_ptr(), 5, 0)
    torch.cuda.synchronize()
    assert int(njobs[0]) == 3 and sorted(slot_unit.cpu().tolist()) == [0, 1, 2]
