"""Generates tests/golden/seed4_p3_golden.npz from the REFERENCE's own C code (oracle/_ref/libnslm_ref.so): P = 3 block
decodes (nslm_decode_block) and rows through its weight reader (ns_row_f32, NS_SEED4).  Run it where the reference
tree exists; the fixture is committed.

    python tests/golden/make_golden_p3.py
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import binding as B  # noqa: E402


def main():
    R = B.ref()
    if R is None:
        raise SystemExit("oracle/_ref/libnslm_ref.so is missing: run `make -C oracle` where the reference tree exists")
    rng = np.random.default_rng(20261126)
    n = 4096
    seed = rng.integers(1, 65536, n).astype(np.uint16)
    nib = rng.integers(0, 65536, n).astype(np.uint16)
    bias = rng.integers(-30, -14, n).astype(np.int32)
    seed[:4] = [1, 65535, 0x8000, 0x7FFF]
    nib[:4] = [0x8880, 0x777F, 0x0000, 0xFFFF]
    bf16 = np.zeros((n, 8), np.uint16)
    for i in range(n):
        R.ref_decode3_block(C.c_uint16(int(seed[i])), C.c_uint16(int(nib[i])), int(bias[i]), bf16[i].ctypes.data_as(C.c_void_p))
    rows, K, eb = 5, 88, -20
    m = B.Matrix3(rows, K, 4242, eb=eb)
    row_f32 = np.zeros((rows, K), np.float32)
    for r in range(rows):
        R.ref_row3_f32(m.seeds.ctypes.data_as(C.c_void_p), m.nibs.ctypes.data_as(C.c_void_p), C.c_int32(eb), rows, K, r,
                       row_f32[r].ctypes.data_as(C.c_void_p))
    out = os.path.join(ROOT, "tests", "golden", "seed4_p3_golden.npz")
    np.savez_compressed(out, blk_seed=seed, blk_nib=nib, blk_bias=bias, blk_bf16=bf16, row_seeds=m.seeds, row_nibs=m.nibs,
                        row_shape=np.array([rows, K, eb], np.int32), row_f32=row_f32)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
