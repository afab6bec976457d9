"""In-tree build of the native libraries (no JIT cache, no pip install).

  libbt_b200.so            the CUDA kernels + C ABI (include/bt_b200.h), nvcc, sm_100a only
  libths_bytetransformer.so  the PyTorch operator / TorchScript class plugin (g++ against torch)

Run `python -m bytetransformer_b200.build` (add `--verbose` for ptxas resource usage).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
OBJ_DIR = os.path.join(PKG_DIR, "build")

CU_SOURCES = ["offsets.cu", "eltwise.cu", "embed_pool.cu", "gemm_sm100.cu", "mha_sm100.cu", "encoder.cu"]
CORE_LIB = os.path.join(LIB_DIR, "libbt_b200.so")
THS_LIB = os.path.join(LIB_DIR, "libths_bytetransformer.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found")
    return cand


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def source_hash() -> str:
    """Digest of the sources the core library is built from (first 12 hex digits of a SHA-256 over file
    names and contents).  It is compiled into `bt_version()`; a library whose digest differs from the
    sources beside it is rebuilt, whatever the file times say."""
    import hashlib
    h = hashlib.sha256()
    files = [os.path.join(CSRC, f) for f in CU_SOURCES] + [os.path.join(CSRC, "common.cuh"),
                                                         os.path.join(CSRC, "kernels.h"),
                                                         os.path.join(ROOT, "include", "bt_b200.h")]
    for f in sorted(files):
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:12]


def built_hash(lib_path: str = None) -> str:
    """The digest a built core library reports (text after 'src:' in bt_version()), or '' if it cannot be loaded."""
    import ctypes
    try:
        lib = ctypes.CDLL(lib_path or CORE_LIB)
        lib.bt_version.restype = ctypes.c_char_p
        v = lib.bt_version().decode()
    except (OSError, AttributeError):
        return ""
    return v.split("src:", 1)[1].strip() if "src:" in v else ""


def _run(cmd, verbose):
    if verbose:
        print("+", " ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), r.stdout))
    if verbose and r.stdout.strip():
        print(r.stdout)
    return r.stdout


def build_core(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "kernels.h"),
               os.path.join(ROOT, "include", "bt_b200.h")]
    objs = []
    procs = []
    digest = source_hash()
    stamp = os.path.join(OBJ_DIR, "source_hash.txt")
    stale = not os.path.exists(stamp) or open(stamp).read().strip() != digest
    for src in CU_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(o)
        # encoder.cu carries the digest: it is compiled again whenever any source changed
        if not force and _newer(o, [s] + headers) and not (stale and src == "encoder.cu"):
            continue
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
              ['-DBT_SOURCE_HASH="%s"' % digest, "-c", s, "-o", o]
        if verbose:
            print("+", " ".join(cmd), flush=True)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), out))
        if verbose and out.strip():
            print(out)
    if force or procs or not _newer(CORE_LIB, objs):
        _run([_nvcc(), "-shared", "-o", CORE_LIB] + objs +
             ["-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"], verbose)
    with open(stamp, "w") as fh:
        fh.write(digest + "\n")
    return CORE_LIB


def build_th_op(force: bool = False, verbose: bool = False) -> str:
    """The torch plugin: registers torch.ops.ByteTransformer.BertTransformer and the
    TorchScript class; calls the core library only through its C ABI."""
    import torch
    from torch.utils import cpp_extension as ce

    src = os.path.join(CSRC, "th_op", "ths_op.cc")
    hdr = os.path.join(ROOT, "include", "bt_b200.h")
    build_core(force=False, verbose=verbose)
    if not force and _newer(THS_LIB, [src, hdr, CORE_LIB]):
        return THS_LIB
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    inc = []
    for p in ce.include_paths():
        inc += ["-isystem", p]
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi,
           "-I", os.path.join(ROOT, "include"), "-isystem", cuda_inc] + inc + [src, "-o", THS_LIB,
           "-L", LIB_DIR, "-lbt_b200", "-Wl,-rpath,$ORIGIN",
           "-L", torch_lib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           "-Wl,-rpath," + torch_lib]
    _run(cmd, verbose)
    return THS_LIB


def build_all(force: bool = False, verbose: bool = False):
    return build_core(force, verbose), build_th_op(force, verbose)


if __name__ == "__main__":
    v = "--verbose" in sys.argv
    f = "--force" in sys.argv
    core = build_core(f, v)
    print("built", core)
    if "--no-th-op" not in sys.argv:
        print("built", build_th_op(f, v))
