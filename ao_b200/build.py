"""Builds libao_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m ao_b200.build [--force] [--verbose]

The library has no Python or torch dependency; it is loaded with ctypes (ao_b200/_cabi.py).
"""
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libao_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O2", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr",
]


def _nvcc():
    for cand in (os.environ.get("AO_NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libao_b200.so cannot be built")


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale():
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, extra_flags=()):
    """Compiles every csrc/*.cu into one shared library; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(LIB_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    env = dict(os.environ)
    # the system compiler, not whatever $CC/$CXX point at
    ccbin = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else None
    objs, procs = [], []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        deps_newer = (not os.path.exists(obj)) or force or any(
            os.path.getmtime(d) > os.path.getmtime(obj)
            for d in [src] + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h")))
        if not deps_newer:
            continue
        cmd = [nvcc] + NVCC_FLAGS + list(extra_flags) + (["-ccbin", ccbin] if ccbin else []) + ["-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd))
        procs.append((src, subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src}:\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("building libao_b200.so failed")
    link = [nvcc, "-shared", "-o", LIB_PATH] + objs + (["-ccbin", ccbin] if ccbin else []) + ["-lcudart_static", "-ldl", "-lrt", "-lpthread"]
    subprocess.check_call(link, env=env)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
