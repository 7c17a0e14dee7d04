"""Builds libseraph_b200.so in-tree with nvcc for sm_100a (plus gcc for the C host files).

    python -m seraph_b200.build            # build if sources are newer than the library
    python -m seraph_b200.build --force
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libseraph_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CUDA_INC = "/usr/local/cuda/include"


def _newer(srcs, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in srcs)


def build(force=False, verbose=False):
    cu = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    cc = sorted(glob.glob(os.path.join(CSRC, "*.c")))
    hdr = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    if not force and not _newer(cu + cc + hdr, OUT):
        return OUT
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for src in cu:
        o = os.path.join(objdir, os.path.basename(src) + ".o")
        objs.append(o)
        if force or _newer([src] + hdr, o):
            cmd = [NVCC, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v"] + ARCH + ["-c", src, "-o", o]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src in cc:
        o = os.path.join(objdir, os.path.basename(src) + ".o")
        objs.append(o)
        if force or _newer([src] + hdr, o):
            cmd = ["gcc", "-O2", "-std=gnu99", "-fPIC", "-Wall", "-I" + CUDA_INC, "-c", src, "-o", o]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = []
    for src, p in procs:
        out, _ = p.communicate()
        log.append(f"== {os.path.basename(src)}\n{out}")
        if p.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"compile failed: {src}")
    with open(os.path.join(objdir, "ptxas.log"), "a") as f:
        f.write("\n".join(log))
    if verbose:
        print("\n".join(log))
    link = [NVCC, "-shared", "-o", OUT] + objs + ["-lcudart", "-ldl", "-lm", "-Xlinker", "-Bsymbolic"]
    subprocess.run(link, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
