"""In-tree build of libhy3attn.so (CUDA kernels + C ABI) for sm_100a with nvcc.

    python -m hy3_b200._build [--force] [--verbose]

Objects go to build/ (git-ignored), the shared library next to this file so that it
travels with the source tree.  nvcc cross-compiles without a GPU.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libhy3attn.so")
SOURCES = ["append.cu", "decode.cu", "prefill.cu", "capi.cu", "selftest.cu"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC,-fvisibility=default", "-I", os.path.join(ROOT, "include")]


def _newer(src_list, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_list)


def build(force=False, verbose=False, defines=(), lib_path=None):
    """defines: extra -D macros (tuning experiments build a second library beside the default one)."""
    global LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    tag = "".join("_" + d.replace("=", "") for d in defines)
    obj_dir = os.path.join(ROOT, "build", "hy3attn" + tag)
    lib_out = lib_path or (LIB if not defines else os.path.join(HERE, "libhy3attn%s.so" % tag))
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(ROOT, "include", "hy3_attn.h"))
    objs, procs = [], []
    for s in SOURCES:
        src = os.path.join(CSRC, s)
        obj = os.path.join(obj_dir, s.replace(".cu", ".o"))
        objs.append(obj)
        if force or _newer([src] + headers, obj):
            cmd = [nvcc] + NVCC_FLAGS + ["-D" + d for d in defines] + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
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
    return lib_out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                defines=tuple(a[2:] for a in sys.argv[1:] if a.startswith("-D"))))
