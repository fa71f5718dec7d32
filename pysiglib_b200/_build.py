"""Builds libcusig.so (sm_100a) from pysiglib_b200/csrc with nvcc, in-tree and incrementally.

    python -m pysiglib_b200._build [--force] [--jobs N]

The library is written to pysiglib_b200/lib/libcusig.so, the file name pySigLib's loader
looks for inside its CUDA plugin package (pysiglib/load_siglib.py:76-103).
"""
import argparse
import concurrent.futures
import hashlib
import os
import re
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_build")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libcusig.so")

NVCC_FLAGS = ["-std=c++17", "--expt-relaxed-constexpr", "-gencode", "arch=compute_100a,code=sm_100a",
              "-lineinfo", "-O3", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-DNDEBUG"]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _tile_parts():
    with open(os.path.join(CSRC, "tile_table.h")) as f:
        return int(re.search(r"#define SIG_TILE_PARTS (\d+)", f.read()).group(1))


def _units():
    """(object name, source, extra flags) for every translation unit."""
    units = [(n + ".o", n + ".cu", []) for n in ("abi", "dispatch", "runtime", "sig_generic", "sig_tile_dispatch", "microbench", "noalloc")]
    for k in range(_tile_parts()):
        units.append(("sig_tile_inst_%d.o" % k, "sig_tile_inst.cu", ["-DSIG_TILE_PART=%d" % k]))
    return units


def _stamp(dev=False):
    h = hashlib.sha256((" ".join(NVCC_FLAGS) + (" dev" if dev else "") +
                        os.environ.get("SIGB200_NO_PACKED_F32", "0")).encode())
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".h", ".cuh", ".cu")):
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(name.encode() + f.read())
    with open(os.path.join(HERE, "..", "include", "cusig_b200.h"), "rb") as f:
        h.update(f.read())
    return h.hexdigest()


def _compile(unit):
    obj, src, extra = unit
    extra = extra + _EXTRA
    cmd = [_nvcc()] + NVCC_FLAGS + extra + ["-c", os.path.join(CSRC, src), "-o", os.path.join(OBJ, obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, proc.stdout, proc.stderr))
    return obj


_EXTRA = []


def build(force=False, jobs=None, verbose=False, dev=None):
    """Compile every CUDA translation unit for sm_100a and link libcusig.so; returns its path.

    dev=True (or SIGB200_TILE_DEV=1) compiles only the development subset of the
    register-tile table (tile_table_dev.h) for quick iteration; the default is the full table."""
    if dev is None:
        dev = os.environ.get("SIGB200_TILE_DEV", "0") == "1"
    _EXTRA[:] = ["-DSIG_TILE_DEV"] if dev else []
    if os.environ.get("SIGB200_NO_PACKED_F32", "0") == "1":  # experiment switch: scalar FP32 rows
        _EXTRA.append("-DSIG_NO_PACKED_F32")
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    stamp, stamp_file = _stamp(dev), os.path.join(LIB_DIR, "stamp.txt")
    if not force and os.path.exists(LIB) and os.path.exists(stamp_file):
        with open(stamp_file) as f:
            if f.read().strip() == stamp:
                return LIB
    units = _units()
    jobs = jobs or min(len(units), os.cpu_count() or 4)
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs) as pool:
        for obj in pool.map(_compile, units):
            if verbose:
                print("compiled", obj, flush=True)
    link = [_nvcc(), "-shared", "-o", LIB] + [os.path.join(OBJ, u[0]) for u in units] + \
           ["-gencode", "arch=compute_100a,code=sm_100a"]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (proc.stdout, proc.stderr))
    with open(stamp_file, "w") as f:
        f.write(stamp)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--dev", action="store_true", help="compile only the development subset of the tile table")
    args = ap.parse_args()
    print(build(force=args.force, jobs=args.jobs, verbose=True, dev=True if args.dev else None))
