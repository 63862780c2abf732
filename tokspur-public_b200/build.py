"""In-tree build of the CUDA library (sm_100a only) with nvcc. No JIT cache: the .so sits beside the package."""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libtsp_moe.so")
STAMP = os.path.join(PKG, "build", "libtsp_moe.stamp")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for path in sources() + sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")) + \
            [os.path.join(ROOT, "include", "tsp_moe.h")]:
        with open(path, "rb") as f:
            h.update(os.path.relpath(path, ROOT).encode())
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu under csrc/ into libtsp_moe.so (object per file, then one link). Returns the path."""
    digest = _digest()
    if not force and os.path.exists(LIB) and os.path.exists(STAMP) and open(STAMP).read().strip() == digest:
        return LIB
    nvcc = _nvcc()
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
    procs = []
    objs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmd = [nvcc, *flags, "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-Xptxas", "-v" if verbose else "-warn-spills",
               "-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed for {src}:\n{out}\n")
        elif verbose or "warning" in out:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("CUDA build failed")
    subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs, "-lcudart"], check=True)
    with open(STAMP, "w") as f:
        f.write(digest)
    return LIB


EP_SRC = os.path.join(PKG, "csrc_ep")
EP_LIB = os.path.join(PKG, "libtsp_ep.so")
EP_STAMP = os.path.join(PKG, "build", "libtsp_ep.stamp")


def nccl_paths():
    """Include and library directories of NCCL (the copy that ships with torch), or None when there is none."""
    try:
        import nvidia.nccl as n
        root = os.path.dirname(n.__file__) if getattr(n, "__file__", None) else list(n.__path__)[0]
    except Exception:
        return None
    inc, lib = os.path.join(root, "include"), os.path.join(root, "lib")
    if os.path.exists(os.path.join(inc, "nccl.h")) and os.path.exists(os.path.join(lib, "libnccl.so.2")):
        return inc, lib
    return None


def build_ep(force: bool = False) -> str | None:
    """Compile csrc_ep/ into libtsp_ep.so (expert parallelism: needs NCCL and libtsp_moe.so). Returns the path, or None without NCCL."""
    paths = nccl_paths()
    if paths is None:
        return None
    build(force=False)
    srcs = sorted(os.path.join(EP_SRC, f) for f in os.listdir(EP_SRC) if f.endswith(".cu"))
    h = hashlib.sha256()
    for path in srcs + [os.path.join(ROOT, "include", "tsp_ep.h"), os.path.join(ROOT, "include", "tsp_moe.h")]:
        with open(path, "rb") as f:
            h.update(f.read())
    digest = h.hexdigest()
    if not force and os.path.exists(EP_LIB) and os.path.exists(EP_STAMP) and open(EP_STAMP).read().strip() == digest:
        return EP_LIB
    inc, lib = paths
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
    cmd = [_nvcc(), *flags, "-shared", "-I", os.path.join(ROOT, "include"), "-I", inc, "-o", EP_LIB, *srcs, "-L", PKG, "-ltsp_moe", "-L", lib,
           "-l:libnccl.so.2", "-lcudart", "-Xlinker", "-rpath=$ORIGIN", "-Xlinker", f"-rpath={lib}"]
    subprocess.run(cmd, check=True)
    os.makedirs(os.path.dirname(EP_STAMP), exist_ok=True)
    with open(EP_STAMP, "w") as f:
        f.write(digest)
    return EP_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_ep(force="--force" in sys.argv))
