"""Builds the C-ABI shared library of the sm_100a kernels, in-tree.

    python 2by4-pretrain_b200/build.py [--force] [--verbose]

Every ``csrc/*.cu`` is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` (nvcc cross-compiles
without a GPU) and linked into ``lib/libsparse24_b200.so``.  Object files are
cached under ``build/`` keyed by a hash of the source, the headers and the flags.
"""
import concurrent.futures
import glob
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")
LIB = os.path.join(LIBDIR, "libsparse24_b200.so")

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the sparse24_b200 kernels cannot be built")
    return exe


def _digest(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    return h.hexdigest()[:16]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def build(force=False, verbose=False):
    nvcc = _nvcc()
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    hdr_digest = _digest(headers, " ".join(NVCC_FLAGS))

    def compile_one(src):
        tag = _digest([src], hdr_digest)
        obj = os.path.join(OBJDIR, os.path.basename(src)[:-3] + "." + tag + ".o")
        log = obj[:-2] + ".log"
        if force or not os.path.exists(obj):
            stem = os.path.basename(src)[:-3] + "."
            for old in os.listdir(OBJDIR):  # drop objects and logs of earlier versions of this source
                if old.startswith(stem) and not old.startswith(stem + tag):
                    os.remove(os.path.join(OBJDIR, old))
            r = subprocess.run([nvcc] + NVCC_FLAGS + ["-c", src, "-o", obj], capture_output=True, text=True)
            with open(log, "w") as f:
                f.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose and os.path.exists(log):
            sys.stderr.write(open(log).read())
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, sources()))
    stamp = os.path.join(OBJDIR, "link.stamp")
    want = _digest(objs)
    if force or not os.path.exists(LIB) or not os.path.exists(stamp) or open(stamp).read() != want:
        r = subprocess.run([nvcc, "-shared", "-o", LIB] + objs, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        with open(stamp, "w") as f:
            f.write(want)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
