"""Writes tests/golden/reference_vectors_formats.npz: outputs of the reference's own CPU code (oracle/_ref,
built by oracle/build_ref.py from the reference checkout) for the four expert formats beside IQ3_S and
IQ4_NL: IQ3_XXS, IQ2_S, IQ4_XS (gate/up) and Q2_0 (down). Dequantized rows by the vendored ggml
dequantizers, single-expert outputs by the AVX-512 expert tier, on seeded inputs of fngine_b200/synth.py.

Usage (only where the reference checkout and an AVX-512 host exist): python tests/golden/make_golden_formats.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from fngine_b200 import synth  # noqa: E402
from oracle import oracle as O  # noqa: E402

DEQUANT = ((O.IQ3_XXS, 13, "iq3xxs"), (O.IQ2_S, 14, "iq2s"), (O.IQ4_XS, 15, "iq4xs"), (O.Q2_0, 16, "q2_0"))
FFN = ((O.IQ3_XXS, O.IQ4_NL, 512, "ffn_iq3xxs_iq4nl_512"), (O.IQ2_S, O.IQ4_NL, 640, "ffn_iq2s_iq4nl_640"),
       (O.IQ4_XS, O.Q2_0, 512, "ffn_iq4xs_q2_0_512"))


def main():
    ref = O.ref()
    if ref is None:
        raise SystemExit("oracle/_ref is not available on this machine")
    out = {}
    for fmt, seed, name in DEQUANT:
        rows = synth.fill_blocks(fmt, 2 * 2560 // synth.BLOCK_ELEMS[fmt], 0, seed)
        out["dequant_" + name] = O.dequant_rows(fmt, rows, 2, 2560, lib=ref)
    xs = synth.activations(32, 2)
    for fg, fd, inter, name in FFN:
        h, y = O.expert_ffn(fg, fd, 2560, inter, synth.expert_blob(fg, fd, inter, 43, 6), xs, lib=ref)
        out[name + "_h"], out[name + "_y"] = h, y
    np.savez_compressed(os.path.join(HERE, "reference_vectors_formats.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
