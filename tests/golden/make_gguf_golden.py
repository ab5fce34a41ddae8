"""Generates tests/golden/tiny_experts.gguf (written by fngine_b200.pack.write_gguf from seeded bytes) and
tiny_experts_gguf.json: what the REFERENCE's reader (tools/gguf.py, GGUFFile) parses from that file. Run where
the reference checkout is available:

    python tests/golden/make_gguf_golden.py /path/to/reference

The test that uses the two files needs neither the reference nor this script."""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from fngine_b200 import pack, synth  # noqa: E402


def tensors():
    out, seed = [], 77
    # blk.0: IQ4_NL gate/up/down, hidden 64, inter 32; blk.1: IQ3_S gate/up with IQ4_NL down, hidden 256, inter 32
    for layer, (gu, dn, hidden, inter) in enumerate([(20, 20, 64, 32), (21, 20, 256, 32)]):
        n_experts = 2
        for k, (t, rows, cols) in (("gate", (gu, inter, hidden)), ("up", (gu, inter, hidden)), ("down", (dn, hidden, inter))):
            nb = n_experts * rows * pack.row_bytes(t, cols)
            seed += 1
            data = (synth.splitmix_words(seed, 0, (nb + 7) // 8).view(np.uint8))[:nb].copy()
            out.append(("blk.%d.ffn_%s_exps.weight" % (layer, k), [cols, rows, n_experts], t, data))
    out.append(("token_embd.weight", [8, 4], 0, np.arange(32, dtype=np.float32)))  # a non-expert tensor (F32)
    return out


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else None
    path = os.path.join(HERE, "tiny_experts.gguf")
    pack.write_gguf(path, tensors(), metadata={"general.architecture": "qwen4exp", "qwen4exp.block_count": 2})
    if ref is None:
        print("wrote", path, "(no reference path given: json not refreshed)")
        return
    sys.path.insert(0, os.path.join(ref, "tools"))
    from gguf import GGUFFile  # the reference's reader
    g = GGUFFile(path)
    doc = {"version": g.version, "alignment": g.alignment, "data_start": int(g.data_start),
           "metadata": {k: (v if isinstance(v, str) else int(v)) for k, v in g.metadata.items()},
           "tensors": [{"name": t.name, "ne": [int(d) for d in t.ne], "type_id": int(t.type_id), "type_name": t.type_name,
                        "offset": int(t.offset), "nbytes": int(t.nbytes),
                        "sha256": hashlib.sha256(bytes(g.tensor_bytes(t.name))).hexdigest()} for t in g.tensors.values()]}
    with open(os.path.join(HERE, "tiny_experts_gguf.json"), "w") as f:
        json.dump(doc, f, indent=1)
    print("wrote", path, "and tiny_experts_gguf.json:", len(doc["tensors"]), "tensors")


if __name__ == "__main__":
    main()
