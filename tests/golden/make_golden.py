"""Regenerates tests/golden/*.npz from the reference's own CPU code.

Run only where oracle/_ref has been built from the reference checkout
(python oracle/build_ref.py): every array stored here is an output of the reference's functions
(ggml dequantizers/quantizers, cpu::decode_rows + cpu::gemm_decoded, cpu::silu_mul,
cpu::decode_rows_bf16 + cpu::gemm_bf16) on inputs that the tests regenerate from seeds.

Usage: python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from fngine_b200 import synth  # noqa: E402
from oracle import oracle as O  # noqa: E402
import patterns  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
IQ3_S, IQ4_NL = 21, 20


def main():
    ref = O.ref()
    if ref is None:
        raise SystemExit("oracle/_ref is not available on this machine")
    out = {}
    # dequantization: 2 rows of 2560 per format (seeds 11 / 12)
    for fmt, seed, name in ((IQ3_S, 11, "iq3s"), (IQ4_NL, 12, "iq4nl")):
        nb = 2 * 2560 // synth.BLOCK_ELEMS[fmt]
        rows = synth.fill_blocks(fmt, nb, 0, seed)
        out["dequant_" + name] = O.dequant_rows(fmt, rows, 2, 2560, lib=ref)
        out["dequant_bf16_" + name] = O.dequant_rows_bf16(fmt, rows, 2, 2560, lib=ref)
    # activation quantizers on the pattern set
    x = patterns.all_inputs()
    out["q8k"] = O.quantize_act(O.ACT_Q8_K, x, lib=ref, variant="avx")
    out["q80"] = O.quantize_act(O.ACT_Q8_0, x, lib=ref, variant="avx")
    # the ggml reference and the reference's AVX quantizers must agree before we pin to them
    assert np.array_equal(out["q8k"], O.quantize_act(O.ACT_Q8_K, x, lib=ref, variant="ref"))
    assert np.array_equal(out["q80"], O.quantize_act(O.ACT_Q8_0, x, lib=ref, variant="ref"))
    # SwiGLU
    g = (synth.normal(21, 4096) * 6).astype(np.float32)
    u = synth.normal(22, 4096).astype(np.float32)
    g[:8] = [0.0, -0.0, 100.0, -100.0, 88.0, -88.0, 1e-20, -1e-20]
    out["silu"] = O.silu_mul(g, u, lib=ref)
    # one expert, decode numerics, the benchmark shapes (IQ3_S x3, inter 512) and the IQ4_NL variant
    xs = synth.activations(31, 3)
    for fg, fd, inter, name in ((IQ3_S, IQ3_S, 512, "ffn_iq3s_512"), (IQ4_NL, IQ4_NL, 512, "ffn_iq4nl_512"),
                                (IQ3_S, IQ4_NL, 640, "ffn_iq3s_iq4nl_640")):
        blob = synth.expert_blob(fg, fd, inter, 41, 5)
        h, y = O.expert_ffn(fg, fd, 2560, inter, blob, xs, lib=ref)
        out[name + "_h"] = h
        out[name + "_y"] = y
    # prefill numerics (bf16 family), 2 tokens
    xb = synth.to_bf16_bits(xs[:2])
    blob = synth.expert_blob(IQ3_S, IQ3_S, 512, 41, 5)
    hb, yb = O.expert_ffn_bf16(IQ3_S, IQ3_S, 2560, 512, blob, xb, lib=ref)
    out["ffn_bf16_iq3s_512_h"] = hb
    out["ffn_bf16_iq3s_512_y"] = yb
    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
