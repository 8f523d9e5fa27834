"""Builds the CUDA library in-tree with nvcc for sm_100a.

    python -m algebraic_transformer_b200.build [--force] [--verbose]

One shared object, `algebraic_transformer_b200/lib/libalg_b200.so`, holding every
kernel and the C ABI of include/alg_b200.h.  Objects are rebuilt when a source or a
header is newer than them.  No GPU is needed to build.
"""

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "build")
LIB = os.path.join(LIBDIR, "libalg_b200.so")

SOURCES = ["c_api.cu", "tmap.cu", "qk_prep.cu", "attn_mma.cu", "attn_sm100.cu", "head_mma.cu", "head_sm100.cu", "head_static.cu", "decode.cu", "prefill_ops.cu", "selftest.cu", "head_exchange.cu", "proj_sm100.cu", "attn_bwd_mma.cu", "attn_bwd_sm100.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "-Xptxas", "-v"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hs.append(os.path.join(ROOT, "include", "alg_b200.h"))
    return hs


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    nvcc = _nvcc()
    hdrs = _headers()
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, src.replace(".cu", ".o"))
        if force or _stale(o, [s] + hdrs):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        cmd = [nvcc] + NVCC_FLAGS + ["-c", s, "-o", o]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = o.replace(".o", ".ptxas.log")
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {s}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return o

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    objs = [os.path.join(OBJDIR, s.replace(".cu", ".o")) for s in SOURCES]
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                    "-Xcompiler", "-fPIC", "-cudart", "shared"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    build_xla_ffi(verbose)
    return LIB


def build_xla_ffi(verbose=False):
    """`lib/libalg_b200_xla.so`: the XLA typed-FFI handlers of csrc/xla_ffi.cc, linked against
    libalg_b200.so.  Needs the jaxlib headers (`jax.ffi.include_dir()`); returns None, leaving the
    rest of the package untouched, where JAX is not installed."""
    try:
        import jax
        inc = jax.ffi.include_dir()
    except Exception:
        return None
    src = os.path.join(CSRC, "xla_ffi.cc")
    out = os.path.join(LIBDIR, "libalg_b200_xla.so")
    if not _stale(out, [src, LIB] + _headers()):
        return out
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include") if os.path.isabs(_nvcc()) else "/usr/local/cuda/include"
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-I", inc, "-I", cuda_inc, src, "-o", out,
           "-L", LIBDIR, "-lalg_b200", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"xla_ffi.cc failed to build:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
