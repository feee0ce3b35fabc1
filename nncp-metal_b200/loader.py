"""Builds (nvcc, sm_100a, in-tree) and loads libnncu.so and libnncp_host.so."""
import ctypes as C
import os
import shutil
import subprocess

from . import abi

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
HOST = os.path.join(PKG, "host")
LIB = os.path.join(PKG, "libnncu.so")
HOSTLIB = os.path.join(PKG, "libnncp_host.so")
CLI = os.path.join(PKG, "nncp-metal")   # the command-line tool (host/cli/nncp_metal_main.c)

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-ccbin", "/usr/bin/g++", "-Xcompiler", "-fPIC,-O2", "-shared"]


class LibraryMissing(RuntimeError):
    pass


def _nvcc():
    for c in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    return None


def _sources(d, exts):
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(exts))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
    """Compiles every .cu under csrc/ into libnncu.so and host/*.c into libnncp_host.so."""
    cu = _sources(CSRC, (".cu",))
    deps = cu + _sources(CSRC, (".cuh", ".h")) + [os.path.join(ROOT, "include", "nncu.h")]
    if force or _stale(LIB, deps):
        nvcc = _nvcc()
        if nvcc is None:
            raise LibraryMissing("nvcc not found and libnncu.so is not built")
        cmd = [nvcc] + NVCC_FLAGS + \
              ["-I", os.path.join(ROOT, "include"), "-I", CSRC] + \
              (["-Xptxas", "-v"] if verbose else []) + os.environ.get("NNCU_NVCC_EXTRA", "").split() + \
              ["-o", LIB] + cu
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
        if verbose:
            print(r.stderr)
    hc = _sources(HOST, (".c",)) if os.path.isdir(HOST) else []
    if hc and (force or _stale(HOSTLIB, hc + _sources(HOST, (".h",)) +
                               [os.path.join(ROOT, "include", "nncp_host.h"),
                                os.path.join(ROOT, "include", "nncp_metal_frontend.h")])):
        cmd = ["gcc", "-O2", "-fPIC", "-shared", "-Wall", "-I", os.path.join(ROOT, "include"),
               "-I", HOST, "-o", HOSTLIB] + hc + ["-lz", "-lm", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("gcc failed:\n" + r.stdout + r.stderr)
    cli_src = os.path.join(HOST, "cli", "nncp_metal_main.c")
    if os.path.exists(cli_src) and (force or _stale(CLI, [cli_src, HOSTLIB])):
        cmd = ["gcc", "-O2", "-Wall", "-I", os.path.join(ROOT, "include"), "-o", CLI, cli_src,
               "-L", PKG, "-l:libnncp_host.so", "-Wl,-rpath,$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("gcc failed:\n" + r.stdout + r.stderr)
    return LIB


DROPIN_DIR = os.path.join(HOST, "dropin")
DROPIN_BIN = os.path.join(DROPIN_DIR, "_build", "nncp_b200")


def build_dropin(reference_dir=None):
    """Builds the reference's own `nncp` command-line tool on this backend (host/dropin/Makefile):
    its unmodified nncp.c, compiled where it lies under `reference_dir` (default
    $NNCP_REFERENCE_DIR), with the Transformer class re-pointed at libnncu.so.  Returns the path
    of the binary, or None when no reference tree is available (a prebuilt binary is kept)."""
    ref = reference_dir or os.environ.get("NNCP_REFERENCE_DIR")
    if not ref or not os.path.isfile(os.path.join(ref, "nncp.c")) or not os.path.exists(LIB):
        return DROPIN_BIN if os.path.exists(DROPIN_BIN) else None
    r = subprocess.run(["make", "-C", DROPIN_DIR, "all", f"REF={ref}"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("drop-in build failed:\n" + r.stdout + r.stderr)
    return DROPIN_BIN if os.path.exists(DROPIN_BIN) else None


_lib = None


def library():
    """The bound libnncu.so.  Raises LibraryMissing when it has not been built: there is
    no other implementation to fall back to."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            raise LibraryMissing(f"{LIB} is not built; run __graft_entry__.build()")
        _lib = abi.bind(C.CDLL(LIB, mode=C.RTLD_GLOBAL))
        if _lib.nncu_abi_version() != 1:
            raise LibraryMissing("libnncu.so has a different ABI version")
    return _lib
