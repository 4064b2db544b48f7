"""Builds libznn_cuda.so (sm_100a only) in-tree with nvcc.

    python -m znn_b200.build [--force] [--verbose]

The shared object is written next to this file so that it travels with the
source tree; it is never installed into site-packages.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libznn_cuda.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "--expt-relaxed-constexpr"]

# (source, extra flags).  The row-wise and conv kernels keep the reference's
# unfused multiply-then-add rounding (see the headers of those files).
SOURCES = [
    ("runtime.cu", []),
    ("gemm_tc.cu", []),
    ("gemm_api.cu", []),
    ("attn_tc.cu", []),
    ("hostop.cu", []),
    ("rowops.cu", ["-fmad=false"]),
    ("conv.cu", ["-fmad=false"]),
    ("conv_tc.cu", []),
    ("dp.cu", []),
    ("host/graph.cpp", []),
    ("host/nn.cpp", []),
    ("host/capi.cpp", []),
    ("host/dataset.cpp", []),
]


def nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _deps_mtime():
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".hpp"))]
    hdrs += [os.path.join(CSRC, "host", f) for f in os.listdir(os.path.join(CSRC, "host")) if f.endswith(".hpp")]
    hdrs.append(os.path.join(os.path.dirname(HERE), "include", "znn_cuda.h"))
    hdrs.append(os.path.join(os.path.dirname(HERE), "include", "znn_host.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    hdr_m = _deps_mtime()
    objs = []
    rebuilt = False
    procs = []
    for src, extra in SOURCES:
        path = os.path.join(CSRC, src)
        if not os.path.exists(path):
            continue
        obj = os.path.join(OBJ, os.path.basename(src).rsplit(".", 1)[0] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(path), hdr_m):
            cmd = [nvcc()] + ARCH + COMMON + extra + ["-c", path, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
                print(" ".join(cmd), flush=True)
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
            rebuilt = True
    failed = []
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed.append((src, out))
        elif verbose or out.strip():
            print(out, flush=True)
    if failed:
        raise RuntimeError("nvcc failed:\n" + "\n".join(f"--- {s} ---\n{o}" for s, o in failed))
    if rebuilt or not os.path.exists(LIB):
        # NCCL is loaded with dlopen at run time (dp.cu), so only libdl is linked
        subprocess.check_call([nvcc(), "-shared", "-o", LIB] + objs + ARCH + ["-ldl"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
