"""TEST INFRASTRUCTURE ONLY: builds oracle/_ref/libfngine_ref.so from the reference checkout.

The reference's CPU expert path is compiled where it lies (no source is copied into this
repository): third_party/ggml-iq/ggml-iq.c, src/cpu/iq_cpu.cpp, src/cpu/q8_cpu.cpp, and for the
production pool src/cpu/expert_pool.cpp, src/core/cpu_topology.cpp, src/core/exchange.cpp (these need
the CUDA headers for the bf16 type only), plus the C-linkage shims oracle/ref_shim.cpp and
oracle/ref_pool_shim.cpp. Flags follow the reference's own build
(third_party/ggml-iq/CMakeLists.txt, src/cpu/CMakeLists.txt:8-9): no fast-math, no FP contraction
for the quantizers. The instruction-set flags are spelled out instead of -march=native so the
library's requirements are explicit; oracle.py checks the host CPU before loading it.

Usage: python oracle/build_ref.py [reference_root]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
ISA = ("-mavx512f -mavx512bw -mavx512dq -mavx512vl -mavx512vnni -mavx512vbmi -mavx512vbmi2 "
       "-mavx512bitalg -mavx512vpopcntdq -mavx512bf16 -mavx2 -mfma -mf16c -mbmi -mbmi2 -mlzcnt "
       "-mpopcnt").split()
REQUIRED_CPU_FLAGS = ["avx512f", "avx512bw", "avx512dq", "avx512vl", "avx512_vnni", "avx512vbmi",
                      "avx512_vbmi2", "avx512_bitalg", "avx512_vpopcntdq", "avx512_bf16", "f16c",
                      "fma", "bmi2"]


def default_reference_root():
    """FNGINE_REFERENCE_ROOT, else the directory `reference` beside this repository."""
    return os.environ.get("FNGINE_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root=None, verbose=True):
    ref_root = ref_root or default_reference_root()
    if not os.path.isdir(os.path.join(ref_root, "src", "cpu")):
        return None
    os.makedirs(OUT, exist_ok=True)
    inc = ["-I", os.path.join(ref_root, "src"), "-I", os.path.join(ref_root, "include"),
           "-I", os.path.join(ref_root, "third_party")]
    objs = []

    def cc(cmd, src, obj):
        full = cmd + ["-fPIC", "-c", src, "-o", obj]
        if verbose:
            print(" ".join(full))
        subprocess.check_call(full)
        objs.append(obj)

    cc(["gcc", "-O2", "-std=c11", "-fno-fast-math", "-ffp-contract=off"] + inc,
       os.path.join(ref_root, "third_party/ggml-iq/ggml-iq.c"), os.path.join(OUT, "ggml-iq.o"))
    cc(["g++", "-O3", "-std=c++20"] + ISA + inc,
       os.path.join(ref_root, "src/cpu/iq_cpu.cpp"), os.path.join(OUT, "iq_cpu.o"))
    cc(["g++", "-O3", "-std=c++20", "-ffp-contract=off"] + ISA + inc,
       os.path.join(ref_root, "src/cpu/q8_cpu.cpp"), os.path.join(OUT, "q8_cpu.o"))
    cc(["g++", "-O2", "-std=c++20"] + ISA + inc,
       os.path.join(HERE, "ref_shim.cpp"), os.path.join(OUT, "ref_shim.o"))
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    if os.path.isfile(os.path.join(cuda_inc, "cuda_bf16.h")):  # the production pool (its headers use __nv_bfloat16)
        pool_inc = inc + ["-I", cuda_inc]
        cc(["g++", "-O3", "-std=c++20"] + ISA + pool_inc,
           os.path.join(ref_root, "src/cpu/expert_pool.cpp"), os.path.join(OUT, "expert_pool.o"))
        cc(["g++", "-O2", "-std=c++20"] + pool_inc,
           os.path.join(ref_root, "src/core/cpu_topology.cpp"), os.path.join(OUT, "cpu_topology.o"))
        cc(["g++", "-O2", "-std=c++20"] + pool_inc,
           os.path.join(ref_root, "src/core/exchange.cpp"), os.path.join(OUT, "exchange.o"))
        cc(["g++", "-O2", "-std=c++20"] + ISA + pool_inc,
           os.path.join(HERE, "ref_pool_shim.cpp"), os.path.join(OUT, "ref_pool_shim.o"))
    so = os.path.join(OUT, "libfngine_ref.so")
    subprocess.check_call(["g++", "-shared", "-o", so] + objs + ["-lm", "-lpthread"])
    with open(os.path.join(OUT, "REQUIRED_CPU_FLAGS"), "w") as f:
        f.write(" ".join(REQUIRED_CPU_FLAGS) + "\n")
    return so


if __name__ == "__main__":
    so = build(sys.argv[1] if len(sys.argv) > 1 else None)
    print(so or "reference checkout not present; nothing built")
