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
    link = [nvcc, "-shared", "-o", LIB_PATH] + objs + (["-ccbin", ccbin] if ccbin else []) + [
        "-Xlinker", "-soname=libao_b200.so", "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
    subprocess.check_call(link, env=env)
    return LIB_PATH


TORCH_EXT_DIR = os.path.join(LIB_DIR, "torch_ext")
TORCH_EXT_PATH = os.path.join(TORCH_EXT_DIR, "ao_b200_torch.so")
TORCH_EXT_SRC = os.path.join(CSRC, "torch", "torch_binding.cpp")


def build_torch_binding(force=False, verbose=False):
    """Compiles csrc/torch/torch_binding.cpp (the TORCH_LIBRARY registration of torchao::quant_llm_linear,
    torchao::_weight_int4pack_mm, torchao::_convert_weight_to_int4pack) against the installed torch and links it to
    libao_b200.so; returns the path of ao_b200/lib/torch_ext/ao_b200_torch.so.  Host C++ only: no GPU needed."""
    lib_path = build(force=False, verbose=verbose)
    deps = [TORCH_EXT_SRC, lib_path, os.path.join(HERE, "..", "include", "ao_b200.h")]
    if not force and os.path.exists(TORCH_EXT_PATH) and all(os.path.getmtime(d) <= os.path.getmtime(TORCH_EXT_PATH) for d in deps[:1] + deps[2:]):
        return TORCH_EXT_PATH
    os.makedirs(TORCH_EXT_DIR, exist_ok=True)
    from torch.utils import cpp_extension
    cpp_extension.load(
        name="ao_b200_torch", sources=[TORCH_EXT_SRC], build_directory=TORCH_EXT_DIR, with_cuda=True,
        extra_cflags=["-O2", "-std=c++17"],
        # libao_b200.so is found by its soname: ao_b200/_torch_ops.py loads it before this library; the run path is
        # a second way in for C++ users of the binding
        extra_ldflags=[f"-L{LIB_DIR}", "-lao_b200", f"-Wl,-rpath,{LIB_DIR}"],
        is_python_module=False, verbose=verbose)
    assert os.path.exists(TORCH_EXT_PATH), TORCH_EXT_PATH
    return TORCH_EXT_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--torch" in sys.argv:
        print(build_torch_binding(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
