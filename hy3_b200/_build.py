"""In-tree build of the two shared libraries for sm_100a with nvcc.

    python -m hy3_b200._build [--force] [--verbose]

  libhy3attn.so   the attention library: CUDA kernels + the C ABI of include/hy3_attn.h
  libhy3_gpu.so   the same objects plus hy3_gpu_dropin.cu: hy3_gpu_init / hy3_gpu_free / hy3_eval_gpu for the reference
                  engine (include/hy3_gpu_dropin.h).  It is compiled against the engine's own hy3.h, so it needs the
                  engine's checkout: HY3_REF, or a directory `reference` next to this repository.  Without one a
                  prebuilt libhy3_gpu.so is kept as it is.

Objects go to build/ (git-ignored), the libraries next to this file so that they travel with the source tree.  nvcc
cross-compiles without a GPU.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libhy3attn.so")
DROPIN_LIB = os.path.join(HERE, "libhy3_gpu.so")
SOURCES = ["append.cu", "decode.cu", "decode_umma.cu", "prefill.cu", "capi.cu", "selftest.cu"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC,-fvisibility=default", "-I", os.path.join(ROOT, "include")]


def _newer(src_list, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_list)


def build(force=False, verbose=False):
    nvcc = os.environ.get("NVCC", "nvcc")
    obj_dir = os.path.join(ROOT, "build", "hy3attn")
    lib_out = LIB
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(ROOT, "include", "hy3_attn.h"))
    objs, procs = [], []
    for s in SOURCES:
        src = os.path.join(CSRC, s)
        obj = os.path.join(obj_dir, s.replace(".cu", ".o"))
        objs.append(obj)
        if force or _newer([src] + headers, obj):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode or verbose:
            print("---- nvcc %s\n%s" % (s, out))
        failed |= bool(p.returncode)
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _newer(objs, lib_out):
        cmd = [nvcc, "-shared", "-o", lib_out] + objs + ["-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            print(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    build_dropin(objs, headers, nvcc, obj_dir, force, verbose)
    return lib_out


def reference_dir():
    """The reference engine's checkout (for its hy3.h), or None."""
    for d in (os.environ.get("HY3_REF"), os.path.join(os.path.dirname(ROOT), "reference")):
        if d and os.path.exists(os.path.join(d, "hy3.h")):
            return d
    return None


def build_dropin(attn_objs, headers, nvcc, obj_dir, force=False, verbose=False):
    ref = reference_dir()
    if ref is None:
        if not os.path.exists(DROPIN_LIB):
            print("hy3_b200._build: no reference checkout (HY3_REF) and no prebuilt %s: the drop-in backend is not built" % DROPIN_LIB)
        return None
    src = os.path.join(CSRC, "hy3_gpu_dropin.cu")
    obj = os.path.join(obj_dir, "hy3_gpu_dropin.o")
    if force or _newer([src, os.path.join(ref, "hy3.h")] + headers, obj):
        cmd = [nvcc] + NVCC_FLAGS + ["-I", ref] + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode or verbose:
            print("---- nvcc hy3_gpu_dropin.cu\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("nvcc failed")
    if force or _newer(attn_objs + [obj], DROPIN_LIB):
        # hy3_rope_get_params and forward_layer_* stay undefined: the engine the library is linked into provides them
        cmd = [nvcc, "-shared", "-o", DROPIN_LIB, obj] + attn_objs + ["-cudart", "static", "-lcublas"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            print(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return DROPIN_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
