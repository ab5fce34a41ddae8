"""Writes tests/golden/fp8row_vectors.npz: outputs of the reference's own FP8-row quantizer
(tools/fp8row.py quantize_rows, imported from the reference checkout) on seeded bf16 rows that cover its
special cases. Run where the checkout is present:

    python tests/golden/make_fp8row_golden.py [reference_root]

The committed .npz lets tests/test_oracle_pins.py hold this repository's restatement of the rule to the
reference's bits on machines without the checkout."""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from fngine_b200 import synth  # noqa: E402


def rows():
    k = 256
    r = synth.normal(4242, 12 * k).astype(np.float32).reshape(12, k)
    r[0] *= 1e-3                      # small values
    r[1] *= 37.0                      # large values
    r[2] = 0.0                        # all-zero row: scale 0, codes 0
    r[3] = 0.0
    r[3, 5] = 3.0                     # one non-zero element
    r[4] *= 1e-30
    r[5, :] = 448.0                   # exactly the E4M3 maximum
    r[6, ::2] = -r[6, 1::2]           # ties of sign
    r[7] = np.round(r[7] * 8) / 8     # many exact E4M3 grid points
    r[8] *= 2.0 ** -100              # tiny but normal (the reference refuses rows whose reciprocal scale overflows)
    r[9] *= 2.0 ** 100
    return synth.to_bf16_bits(r)


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FNGINE_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
    spec = importlib.util.spec_from_file_location("ref_fp8row", os.path.join(ref, "tools", "fp8row.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    w = rows()
    wt = torch.from_numpy(w.view(np.int16)).view(torch.bfloat16)
    codes, scales = mod.quantize_rows(wt)
    np.savez_compressed(os.path.join(HERE, "fp8row_vectors.npz"), weight=w, codes=codes.numpy(),
                        scales=scales.view(torch.int16).numpy().view(np.uint16))
    print("wrote fp8row_vectors.npz:", w.shape)


if __name__ == "__main__":
    main()
