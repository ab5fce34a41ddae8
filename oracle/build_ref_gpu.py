"""TEST INFRASTRUCTURE ONLY: builds oracle/_ref_gpu/libfngine_ref_gpu.so, the reference's own GPU decode
kernels compiled for sm_100a.

The reference targets sm_120a only (its CMakeLists refuses other architectures) but the decode kernels
themselves (src/kernels/moe/moe_decode.cu, moe_format.cpp) use nothing specific to that architecture, so
they are compiled where they lie, unchanged, with nvcc for sm_100a, together with the C-linkage shim
oracle/ref_gpu_shim.cu. Used only by bench.py's `legacy` section to put the reference's kernels on the
same GPU beside this library's. No source is copied into this repository.

Usage: python oracle/build_ref_gpu.py [reference_root]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref_gpu")


def default_reference_root():
    return os.environ.get("FNGINE_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root=None, verbose=True):
    ref_root = ref_root or default_reference_root()
    src = os.path.join(ref_root, "src", "kernels", "moe", "moe_decode.cu")
    if not os.path.isfile(src):
        return None
    so = os.path.join(OUT, "libfngine_ref_gpu.so")
    inputs = [src, os.path.join(ref_root, "src", "kernels", "moe", "moe_format.cpp"), os.path.join(HERE, "ref_gpu_shim.cu")]
    if os.path.exists(so) and all(os.path.getmtime(so) >= os.path.getmtime(p) for p in inputs):
        return so
    os.makedirs(OUT, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++20", "--expt-relaxed-constexpr", "-Xcompiler",
             "-fPIC", "-I", os.path.join(ref_root, "src"), "-I", os.path.join(ref_root, "include"), "-I",
             os.path.join(ref_root, "third_party")]
    objs = []
    for p in inputs:
        obj = os.path.join(OUT, os.path.basename(p).rsplit(".", 1)[0] + ".o")
        cmd = [nvcc] + flags + ["-x", "cu", "-c", p, "-o", obj]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd, stdout=subprocess.DEVNULL if not verbose else None)
        objs.append(obj)
    subprocess.check_call([nvcc, "-shared", "-o", so] + objs + ["-cudart", "static"])
    return so


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None) or "reference checkout not present; nothing built")
