"""Builds libnd4jb200.so (the CUDA kernels plus the C ABI) for sm_100a with nvcc.

Every (family, element type) pair is its own translation unit, so the build runs them in
parallel; object files go to libnd4j_b200/build/ and the shared library next to this file.
Usage: python -m libnd4j_b200.build [--force] [--ptxas-verbose]
"""
import concurrent.futures
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libnd4jb200.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    # no FMA contraction: +,-,*,/ sequences then round exactly like the reference's x86-64 build
    "-fmad=false",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-diag-suppress", "177",
]


def _sources():
    units = []
    for fam in range(7):
        for dt in range(3):
            units.append(("family_%d_%d" % (fam, dt), "family_tu.cu", ["-DND_FAMILY=%d" % fam, "-DND_DTYPE=%d" % dt]))
    units.append(("api", "api.cu", []))
    units.append(("native_ops", "native_ops.cu", []))
    units.append(("no_alloc", "no_alloc.cu", []))
    units.append(("utility_ops", "utility_ops.cu", []))
    units.append(("sort_ops", "sort_ops.cu", []))
    units.append(("special_transforms", "special_transforms.cu", []))
    units.append(("device_env", "device_env.cu", []))
    units.append(("comm", "comm.cu", []))
    units.append(("runtime", "runtime.cu", []))
    units.append(("shape_host", "shape_host.cpp", []))
    return [u for u in units if os.path.exists(os.path.join(CSRC, u[1]))]


def _digest():
    h = hashlib.sha256()
    for root in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        for name in sorted(os.listdir(root)):
            with open(os.path.join(root, name), "rb") as f:
                h.update(name.encode())
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile(unit, extra_flags):
    name, src, defs = unit
    obj = os.path.join(OUT, name + ".o")
    cmd = ["nvcc"] + NVCC_FLAGS + extra_flags + defs + ["-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (name, r.stdout, r.stderr))
    return obj, r.stderr


def build(force=False, ptxas_verbose=False, jobs=None):
    os.makedirs(OUT, exist_ok=True)
    stamp = os.path.join(OUT, "digest.txt")
    digest = _digest()
    if not force and os.path.exists(LIB) and os.path.exists(stamp) and open(stamp).read() == digest:
        return LIB
    extra = ["-Xptxas", "-v"] if ptxas_verbose else []
    units = _sources()
    jobs = jobs or min(len(units), os.cpu_count() or 4)
    objs, logs = [], []
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs) as ex:
        for obj, log in ex.map(lambda u: _compile(u, extra), units):
            objs.append(obj)
            logs.append(log)
    cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs + ["-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    with open(stamp, "w") as f:
        f.write(digest)
    if ptxas_verbose:
        with open(os.path.join(OUT, "ptxas.log"), "w") as f:
            f.write("\n".join(logs))
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, ptxas_verbose="--ptxas-verbose" in sys.argv)
    print(path)
