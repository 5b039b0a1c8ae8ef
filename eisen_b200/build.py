"""Builds libeisen_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libeisen_b200.so")
OBJ = os.path.join(HERE, "build")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "--extended-lambda", "-Xcompiler", "-fPIC,-O3", "-Xptxas", "-v"]


def sources():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith(".cu") or f.endswith(".cpp"):
                out.append(os.path.join(root, f))
    return sorted(out)


def headers_mtime():
    m = 0.0
    for root, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".h", ".cuh")):
                m = max(m, os.path.getmtime(os.path.join(root, f)))
    inc = os.path.join(os.path.dirname(HERE), "include", "eisen_b200.h")
    if os.path.exists(inc):
        m = max(m, os.path.getmtime(inc))
    return m


def build(verbose=False, force=False):
    os.makedirs(OBJ, exist_ok=True)
    hm = headers_mtime()
    objs = []
    procs = []
    for src in sources():
        rel = os.path.relpath(src, CSRC).replace(os.sep, "_")
        obj = os.path.join(OBJ, rel + ".o")
        objs.append(obj)
        if (not force) and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src), hm):
            continue
        cmd = [NVCC] + ARCH + COMMON + ["-x", "cu", "-c", src, "-o", obj]
        log = open(obj + ".log", "w")
        procs.append((src, subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT), obj + ".log"))
    failed = False
    for src, p, logp in procs:
        rc = p.wait()
        text = open(logp).read()
        if rc != 0:
            failed = True
            sys.stderr.write("nvcc failed for %s:\n%s\n" % (src, text))
        elif verbose:
            sys.stdout.write(text)
    if failed:
        raise RuntimeError("nvcc compilation failed")
    if procs or not os.path.exists(OUT):
        cmd = [NVCC] + ARCH + ["-shared", "-o", OUT] + objs + ["-lcuda" if False else "-lcudart_static", "-ldl", "-lpthread", "-lrt"]
        subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
