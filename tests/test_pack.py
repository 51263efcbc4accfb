"""Ingestion of packed SEED4P4 weights (include/nslm_pack.h): host code, no GPU.

The .blk4 case is the reference's own known-answer test (tests/test_moe.c:121-137): 2 experts of 2 x 16, seeds 100 + k,
coefficient words 0x1000 + k, one code byte k per block, biases (-20, -19)."""
import ctypes as C

import numpy as np
import pytest


@pytest.fixture(scope="module")
def L():
    from nanoseedlm_b200 import lib
    lib.load()
    return lib


def reference_image(L):
    E, R, Cc, NB = 2, 2, 16, 2 * 16 // 8
    n = L.load().nsl_blk4_bytes(E, R, Cc)
    assert n == 56 + 12 * E + 5 * NB * E
    img = np.zeros(n, np.uint8)
    img[:8] = np.frombuffer(b"NSLMBLK4", np.uint8)
    img[8:20].view(np.uint32)[:] = (R, Cc, E)
    body = img[56:]
    body[:8].view(np.int32)[:] = (-20, -19)
    k = np.arange(NB * E)
    body[12 * E:12 * E + 2 * NB * E].view(np.uint16)[:] = 100 + k
    body[12 * E + 2 * NB * E:12 * E + 4 * NB * E].view(np.uint16)[:] = 0x1000 + k
    body[12 * E + 4 * NB * E:] = k
    return img, E, R, Cc, NB


def split(L, img, E, R, Cc, n=None):
    NB = R * Cc // 8
    s0, s1 = np.zeros(NB * E, np.uint16), np.zeros(NB * E, np.uint16)
    s2, s3 = np.zeros(E, np.int32), np.zeros(NB * E // 2, np.uint8)
    rc = L.load().nsl_blk4_split(img.ctypes.data, img.size if n is None else n, E, R, Cc, s0.ctypes.data, s1.ctypes.data,
                                 s2.ctypes.data, s3.ctypes.data)
    return rc, s0, s1, s2, s3


def test_blk4_known_answers(L):
    img, E, R, Cc, NB = reference_image(L)
    rc, s0, s1, s2, s3 = split(L, img, E, R, Cc)
    assert rc == 0
    assert s0[5] == 105 and s1[7] == 0x1007 and s2[1] == -19
    assert s3[0] == 0x10 and s3[3] == 0x76          # block 2j in the low nibble
    assert split(L, img, E, R, 2 * Cc)[0] == -1      # another shape
    assert split(L, img, E, R, Cc, n=img.size - 1)[0] == -1   # a short image
    bad = img.copy()
    bad[7] = ord("8")
    assert split(L, bad, E, R, Cc)[0] == -1           # another bank kind


def test_blk4_join_and_split_round_trip(L, oracle):
    E, R, Cc = 3, 8, 64
    mats = [oracle.Matrix(R, Cc, 50 + e, eb=-22 + e) for e in range(E)]
    seeds = np.concatenate([m.seeds.ravel() for m in mats]).astype(np.uint16)
    coefs = np.concatenate([m.coefs.ravel() for m in mats]).astype(np.uint16)
    codes = np.concatenate([m.codes.ravel() for m in mats]).astype(np.uint8)
    bias = np.array([m.eb for m in mats], np.int32)
    img = np.zeros(L.load().nsl_blk4_bytes(E, R, Cc), np.uint8)
    assert L.load().nsl_blk4_join(img.ctypes.data, img.size, E, R, Cc, seeds.ctypes.data, coefs.ctypes.data, bias.ctypes.data,
                                  codes.ctypes.data) == 0
    rc, s0, s1, s2, s3 = split(L, img, E, R, Cc)
    assert rc == 0 and np.array_equal(s0, seeds) and np.array_equal(s1, coefs) and np.array_equal(s2, bias)
    assert np.array_equal(s3, codes)


def test_wslice_table_addresses(L):
    S, R, Cc = 4, 6, 32
    nb = R * Cc // 8
    table = (L.WSlice * S)()
    bias = np.array([-20, -21, -19, -22], np.int32)
    rc = L.load().nsl_wslice_table(C.c_void_p(0x10000), C.c_void_p(0x20000), C.c_void_p(0x30000), bias.ctypes.data, S, R, Cc, table)
    assert rc == 0
    for i in range(S):
        assert table[i].p[0] == 0x10000 + 2 * nb * i and table[i].p[1] == 0x20000 + 2 * nb * i
        assert not table[i].p[2] and table[i].p[3] == 0x30000 + nb // 2 * i
        assert table[i].eb == bias[i] and table[i].gs == 0
    assert L.load().nsl_wslice_table(C.c_void_p(0x10000), C.c_void_p(0x20000), C.c_void_p(0x30000), bias.ctypes.data, S, 1, 8, table) == -1
    assert "multiple of 16" in L.last_error()
