"""A .blk4 expert bank fed to the kernels through the library's ingestion (nsl_blk4_split + nsl_wslice_table): the
gather mat-vec over the ingested experts equals the oracle on the original matrices."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_blk4_bank_to_kernels(oracle):
    import torch
    from nanoseedlm_b200 import kernels, lib as L, moe
    E, R, K = 5, 48, 256
    mats = [oracle.Matrix(R, K, 700 + e, eb=-23 + e) for e in range(E)]
    cat = lambda f, dt: np.concatenate([getattr(m, f).ravel() for m in mats]).astype(dt)
    seeds, coefs, codes = cat("seeds", np.uint16), cat("coefs", np.uint16), cat("codes", np.uint8)
    bias = np.array([m.eb for m in mats], np.int32)
    img = np.zeros(L.load().nsl_blk4_bytes(E, R, K), np.uint8)
    assert L.load().nsl_blk4_join(img.ctypes.data, img.size, E, R, K, seeds.ctypes.data, coefs.ctypes.data, bias.ctypes.data,
                                  codes.ctypes.data) == 0
    bank = moe.ExpertStack.from_blk4(img, E, R, K)
    sel = np.array([4, 0, 2, 2, 1, 3, 4], np.int32)
    x = oracle.normal(9, sel.size * K, bf16=True).reshape(sel.size, K)
    xd, seld = kernels.dev(x), kernels.dev(sel)
    y = torch.zeros(sel.size, R, device="cuda")
    L.load().kc_mv_sel(None, L.MF_SEED4P4, C.c_void_p(bank.table.data_ptr()), K, R, C.c_void_p(xd.data_ptr()), K,
                       C.c_void_p(y.data_ptr()), R, C.c_void_p(seld.data_ptr()), sel.size, 1,
                       C.c_void_p(kernels.stream_table().data_ptr()))
    torch.cuda.synchronize()
    L.check()
    y = y.cpu().numpy()
    for p, e in enumerate(sel):
        ref = oracle.mv(mats[e], x[p])[0]
        y64, mag = oracle.matvec_f64(mats[e], x[p])
        assert np.all(np.abs(y[p] - ref) <= np.abs(ref) / 128 + 64 * 1.2e-7 * mag[0] + 1e-30)
