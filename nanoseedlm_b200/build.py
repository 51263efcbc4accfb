"""Builds libnslm_b200.so (the CUDA kernels and their C ABI) in-tree with nvcc for sm_100a."""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libnslm_b200.so")
SOURCES = ["common.cu", "seed_mv.cu", "moe_misc.cu", "seed_gemm.cu", "moe_host.cu", "ep.cu", "ep_p2p.cu", "mova.cu", "q4_head.cu", "pack.cu", "attn.cu", "xcache.cu", "decoder_ops.cu", "decoder.cu", "dense_bf16.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-Xptxas", "-v"]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
    """Compile every .cu under csrc/ to an object (in parallel) and link the shared library.  Returns its path."""
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers += [os.path.join(HERE, "..", "include", h) for h in ("nslm_kernels.h", "nslm_moe.h", "nslm_ep.h", "nslm_pack.h", "nslm_cache.h", "nslm_decoder.h")]
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    procs, objs = [], []
    for src in SOURCES:
        sp = os.path.join(CSRC, src)
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [sp] + headers):
            log = open(obj + ".log", "w")
            procs.append((src, subprocess.Popen([_nvcc()] + NVCC_FLAGS + ["-c", sp, "-o", obj], stdout=log,
                                                stderr=subprocess.STDOUT), log))
    failed = []
    for src, p, log in procs:
        rc = p.wait()
        log.close()
        if rc != 0:
            failed.append(src)
    if failed:
        for src in failed:
            sys.stderr.write(open(os.path.join(objdir, src.replace(".cu", ".o")) + ".log").read())
        raise RuntimeError("nvcc failed for " + ", ".join(failed))
    if force or procs or _stale(LIB, objs):
        subprocess.run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + objs + ["-lcudart"],
                       check=True)
    if verbose:
        print("built", LIB)
    return LIB


if __name__ == "__main__":
    build_library(force="--force" in sys.argv, verbose=True)
