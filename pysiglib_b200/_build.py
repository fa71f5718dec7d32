"""Builds libcusig.so (sm_100a) from pysiglib_b200/csrc with nvcc, in-tree and incrementally
(an object is recompiled only when a file its preprocessor run reads has changed).

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
BENCH_LIB = os.path.join(LIB_DIR, "libsigb200_bench.so")  # FMA-peak probe; loaded by bench.py only

NVCC_FLAGS = ["-std=c++17", "--expt-relaxed-constexpr", "-gencode", "arch=compute_100a,code=sm_100a",
              "-lineinfo", "-O3", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-DNDEBUG",
              "-Xfatbin=-compress-all"]  # the several hundred tile variants compress about threefold


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _tile_parts():
    with open(os.path.join(CSRC, "tile_table.h")) as f:
        return int(re.search(r"#define SIG_TILE_PARTS (\d+)", f.read()).group(1))


def _units():
    """(object name, source, extra flags) for every translation unit."""
    units = [(n + ".o", n + ".cu", []) for n in ("abi", "dispatch", "runtime", "sig_generic", "sig_tile_dispatch", "sig_algebra", "sig_log", "sig_coef", "sig_chen", "sig_log_stream", "noalloc")]
    for k in range(_tile_parts()):
        units.append(("sig_tile_inst_%d.o" % k, "sig_tile_inst.cu", ["-DSIG_TILE_PART=%d" % k]))
    return units


def _stamp():
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for folder in (CSRC, os.path.join(CSRC, "bench")):
        for name in sorted(os.listdir(folder)):
            if name.endswith((".h", ".cuh", ".cu")):
                with open(os.path.join(folder, name), "rb") as f:
                    h.update(name.encode() + f.read())
    with open(os.path.join(HERE, "..", "include", "cusig_b200.h"), "rb") as f:
        h.update(f.read())
    return h.hexdigest()


def _unit_hash(unit):
    """Hash of one translation unit: its flags and the contents of every file of this
    repository that the preprocessor pulls in (nvcc -M), so that an edit recompiles only
    the objects that can see it."""
    obj, src, extra = unit
    cmd = [_nvcc()] + NVCC_FLAGS + extra + ["-M", os.path.join(CSRC, src)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc -M failed for %s:\n%s\n%s" % (src, proc.stdout, proc.stderr))
    root = os.path.realpath(os.path.join(HERE, ".."))
    deps = set()
    for tok in proc.stdout.split(":", 1)[-1].replace("\\\n", " ").split():
        path = os.path.realpath(tok)
        if path.startswith(root + os.sep):
            deps.add(path)
    h = hashlib.sha256((" ".join(NVCC_FLAGS + extra)).encode())
    for path in sorted(deps):
        with open(path, "rb") as f:
            h.update(os.path.relpath(path, root).encode() + f.read())
    return h.hexdigest()


def _compile(unit):
    """Compiles one unit unless its object is already up to date; returns (object, rebuilt)."""
    obj, src, extra = unit
    digest = _unit_hash(unit)
    obj_path, hash_path = os.path.join(OBJ, obj), os.path.join(OBJ, obj + ".hash")
    if not _FORCE[0] and os.path.exists(obj_path) and os.path.exists(hash_path):
        with open(hash_path) as f:
            if f.read().strip() == digest:
                return obj, False
    cmd = [_nvcc()] + NVCC_FLAGS + extra + ["-c", os.path.join(CSRC, src), "-o", obj_path]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, proc.stdout, proc.stderr))
    with open(hash_path, "w") as f:
        f.write(digest)
    return obj, True


_FORCE = [False]


def build(force=False, jobs=None, verbose=False):
    """Compile every CUDA translation unit for sm_100a and link libcusig.so; returns its path."""
    _FORCE[0] = bool(force)
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    stamp, stamp_file = _stamp(), os.path.join(LIB_DIR, "stamp.txt")
    if not force and os.path.exists(LIB) and os.path.exists(stamp_file):
        with open(stamp_file) as f:
            if f.read().strip() == stamp:
                return LIB
    units = _units()
    jobs = jobs or min(len(units), os.cpu_count() or 4)
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs) as pool:
        for obj, rebuilt in pool.map(_compile, units):
            if verbose:
                print("compiled" if rebuilt else "up to date", obj, flush=True)
    link = [_nvcc(), "-shared", "-o", LIB] + [os.path.join(OBJ, u[0]) for u in units] + \
           ["-gencode", "arch=compute_100a,code=sm_100a"]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (proc.stdout, proc.stderr))
    bench = [_nvcc(), "-shared", "-o", BENCH_LIB, os.path.join(CSRC, "bench", "fma_peak.cu"),
             os.path.join(CSRC, "bench", "fma_patterns.cu"), "-O3", "-lineinfo",
             "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
    proc = subprocess.run(bench, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("building the benchmark helper failed:\n%s\n%s" % (proc.stdout, proc.stderr))
    with open(stamp_file, "w") as f:
        f.write(stamp)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    args = ap.parse_args()
    print(build(force=args.force, jobs=args.jobs, verbose=True))
