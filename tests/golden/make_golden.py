"""Generates tests/golden/seed4p4_golden.npz from the REFERENCE's own C code (oracle/_ref/libnslm_ref.so, built by
oracle/Makefile from the reference sources where they lie).  Run it in a container that has the reference tree; the
fixture it writes is committed and is what the tests read everywhere else.

    python tests/golden/make_golden.py
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
    rng = np.random.default_rng(20261125)
    u16p, f32p, i32p, u8p = (C.POINTER(t) for t in (C.c_uint16, C.c_float, C.c_int32, C.c_uint8))

    # 1. states and stream words of a few seeds
    st_seeds = np.array([1, 2, 0xACE1, 0x8000, 32767, 65535, 4660, 51966], np.uint16)
    states = np.zeros((len(st_seeds), 48), np.uint16)
    stream = np.zeros(len(st_seeds), np.uint32)
    for i, s in enumerate(st_seeds):
        R.ref_states(C.c_uint16(int(s)), 48, states[i].ctypes.data_as(u16p))
        stream[i] = R.ref_stream32(C.c_uint16(int(s)))

    # 2. block decodes (nslm4_decode_block): random blocks plus the extremes of every field
    n = 4096
    blk_seed = rng.integers(1, 65536, n).astype(np.uint16)
    blk_coef = rng.integers(0, 65536, n).astype(np.uint16)
    blk_e = rng.integers(-30, 1, n).astype(np.int32)
    blk_seed[:4] = [1, 65535, 0x8000, 0x7FFF]
    blk_coef[:4] = [0x8888, 0x7777, 0x0000, 0xFFFF]
    blk_bf16 = np.zeros((n, 8), np.uint16)
    for i in range(n):
        R.ref_decode_block(C.c_uint16(int(blk_seed[i])), C.c_uint16(int(blk_coef[i])), int(blk_e[i]),
                           blk_bf16[i].ctypes.data_as(u16p))

    # 3. whole rows through the reference weight reader (ns_row_f32), an odd block count so rows start mid-byte
    rows, K, eb = 7, 72, -21
    m = B.Matrix(rows, K, 31337, eb=eb)
    row_f32 = np.zeros((rows, K), np.float32)
    for r in range(rows):
        R.ref_row_f32(m.seeds.ctypes.data_as(u16p), m.coefs.ctypes.data_as(u16p), m.codes.ctypes.data_as(u8p),
                      C.c_int32(eb), rows, K, r, row_f32[r].ctypes.data_as(f32p))

    # 4. router: 512 experts, top 10, with the reference test's tie (experts 7 and 300 at 9.0)
    lg = rng.uniform(-4, 4, (3, 512)).astype(np.float32)
    lg[0, 7] = lg[0, 300] = 9.0
    r_ind = np.zeros((3, 10), np.int32)
    r_wt = np.zeros((3, 10), np.float32)
    for t in range(3):
        R.ref_route(512, 10, lg[t].ctypes.data_as(f32p), r_ind[t].ctypes.data_as(i32p), r_wt[t].ctypes.data_as(f32p))

    out = os.path.join(ROOT, "tests", "golden", "seed4p4_golden.npz")
    np.savez_compressed(out, st_seeds=st_seeds, states=states, stream=stream, blk_seed=blk_seed, blk_coef=blk_coef,
                        blk_e=blk_e, blk_bf16=blk_bf16, row_seeds=m.seeds, row_coefs=m.coefs, row_codes=m.codes,
                        row_shape=np.array([rows, K, eb], np.int32), row_f32=row_f32, route_logits=lg, route_ind=r_ind,
                        route_wt=r_wt)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
