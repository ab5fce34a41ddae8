"""Host-side ingestion of expert weights: the pack manifest + experts.bin and GGUF expert tensors
(src/io/pack.h:53-78, tools/convert.py:272-323, tools/gguf.py:68-100 of the reference). The GGUF reader is
pinned to what the reference's own reader parsed from the committed tiny file (tests/golden/)."""
import hashlib
import json
import os

import numpy as np
import pytest

from fngine_b200 import pack, synth

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
IQ4_NL, IQ3_S, IQ2_S = 20, 21, 22


def test_row_bytes_and_layout_known_answers():
    # block sizes of tools/iqformats.py:20-21 and the blob sizes of the model's two layouts
    assert [pack.row_bytes(t, 2560) for t in (18, 20, 21, 22, 23, 42)] == [980, 1440, 1100, 820, 1360, 720]
    a = pack.layer_info(IQ3_S, IQ4_NL, 2560, 640, 0)
    assert (a.gate_bytes, a.up_bytes, a.down_bytes, a.blob_bytes, a.blob_stride) == (704000, 704000, 921600, 2329600, 2330624)
    b = pack.layer_info(IQ3_S, IQ3_S, 2560, 512, 4096)
    assert (b.blob_bytes, b.blob_stride, b.offset) == (1689600, 1691648, 4096)
    with pytest.raises(pack.PackError):
        pack.row_bytes(IQ3_S, 640)  # not a multiple of 256
    with pytest.raises(pack.PackError):
        pack.row_bytes(12, 2560)    # Q4_K is not an expert format


def test_gguf_reader_agrees_with_the_reference_reader():
    doc = json.load(open(os.path.join(GOLD, "tiny_experts_gguf.json")))
    g = pack.GgufExperts(os.path.join(GOLD, "tiny_experts.gguf"))
    assert g.alignment == doc["alignment"] and g.data_start == doc["data_start"]
    assert list(g.tensors) == [t["name"] for t in doc["tensors"]]
    for t in doc["tensors"]:
        mine = g.tensors[t["name"]]
        assert (mine.ne, mine.type_id, mine.offset) == (t["ne"], t["type_id"], t["offset"])
        if t["type_id"] in pack.EXPERT_TYPES:
            assert mine.nbytes == t["nbytes"]
            assert hashlib.sha256(bytes(g.mm[mine.offset:mine.offset + mine.nbytes])).hexdigest() == t["sha256"]
        else:
            assert mine.nbytes is None
    assert g.layers() == [0, 1]
    info, n_experts, hidden, inter = g.layer_layout(1)
    assert (info.gu_type, info.down_type, n_experts, hidden, inter) == (IQ3_S, IQ4_NL, 2, 256, 32)
    assert info.gate_bytes == 32 * 110 and info.down_bytes == 256 * 18 and info.blob_stride == 12288
    # slot array: expert e = its slice of gate, then up, then down (tools/convert.py:292-318)
    slots = g.layer_bytes(1)
    for e in range(2):
        pos = 0
        for k, nb in (("gate", info.gate_bytes), ("up", info.up_bytes), ("down", info.down_bytes)):
            t = g.tensors["blk.1.ffn_%s_exps.weight" % k]
            assert np.array_equal(slots[e, pos:pos + nb], g.mm[t.offset + e * nb:t.offset + (e + 1) * nb])
            pos += nb
        assert not slots[e, pos:].any()
    assert np.array_equal(g.layer_bytes(1, first=1, count=1)[0], slots[1])


def test_gguf_errors(tmp_path):
    p = str(tmp_path / "bad.gguf")
    z = np.zeros(2 * 32 * 36, dtype=np.uint8)
    pack.write_gguf(p, [("blk.0.ffn_gate_exps.weight", [64, 32, 2], IQ4_NL, z),
                        ("blk.0.ffn_up_exps.weight", [256, 32, 2], IQ3_S, np.zeros(2 * 32 * 110, dtype=np.uint8)),
                        ("blk.0.ffn_down_exps.weight", [32, 64, 2], IQ4_NL, np.zeros(2 * 64 * 18, dtype=np.uint8))])
    g = pack.GgufExperts(p)
    with pytest.raises(pack.PackError, match="gate type"):
        g.layer_layout(0)
    with pytest.raises(pack.PackError, match="missing"):
        g.layer_layout(3)
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:len(raw) - 100])
    with pytest.raises(pack.PackError, match="past the end"):
        pack.GgufExperts(p)
    open(p, "wb").write(b"GGML" + raw[4:])
    with pytest.raises(pack.PackError, match="not a GGUF"):
        pack.GgufExperts(p)


def test_pack_round_trip_and_validation(tmp_path):
    d = str(tmp_path / "pack")
    gu, dn, inter = IQ3_S, IQ3_S, 256
    blobs = np.stack([synth.expert_blob(gu, dn, inter, 40, e, hidden=256) for e in range(4)])
    extra = np.stack([synth.expert_blob(IQ3_S, IQ4_NL, inter, 50, e, hidden=256) for e in range(4)])
    infos = pack.write_expert_pack(d, 256, inter, [(gu, dn, blobs), (IQ3_S, IQ4_NL, extra)])
    p = pack.ExpertPack.open(d)
    assert (p.n_experts, p.hidden, p.inter, len(p.layers)) == (4, 256, 256, 2)
    assert p.layers == infos and p.layers[1].offset == 4 * infos[0].blob_stride
    for e in range(4):
        assert np.array_equal(p.blob(0, e), blobs[e]) and np.array_equal(p.blob(1, e), extra[e])
    shard = p.layer_bytes(1, first=2, count=2)
    assert shard.shape == (2, infos[1].blob_stride) and np.array_equal(shard[1, :infos[1].blob_bytes], extra[3])
    assert p.supported(0) and p.supported(1)

    mpath = os.path.join(d, "manifest.json")
    good = json.load(open(mpath))

    def reopen(edit):
        man = json.loads(json.dumps(good))
        edit(man)
        json.dump(man, open(mpath, "w"))
        return pack.ExpertPack.open(d)

    with pytest.raises(pack.PackError, match=r"layers\[1\]\.gate_bytes"):
        reopen(lambda m: m["experts"]["layers"][1].__setitem__("gate_bytes", 1))
    with pytest.raises(pack.PackError, match=r"layers\[0\]\.blob_stride"):
        reopen(lambda m: m["experts"]["layers"][0].__setitem__("blob_stride", infos[0].blob_bytes))
    with pytest.raises(pack.PackError, match=r"layers\[1\]\.offset"):
        reopen(lambda m: m["experts"]["layers"][1].__setitem__("offset", 4096))
    with pytest.raises(pack.PackError, match="unsupported expert format"):
        reopen(lambda m: m["experts"]["layers"][0].update(gu_type="Q4_K", gu_type_id=12))
    with pytest.raises(pack.PackError, match="does not name"):
        reopen(lambda m: m["experts"]["layers"][0].update(gu_type_id=20))
    with pytest.raises(pack.PackError, match="fngine-pack"):
        reopen(lambda m: m.__setitem__("format", "other"))
    with pytest.raises(pack.PackError, match="n_layers"):
        reopen(lambda m: m["experts"].__setitem__("n_layers", 3))
    with pytest.raises(pack.PackError, match="missing field"):
        reopen(lambda m: m["experts"]["layers"][0].pop("offset"))
    with pytest.raises(pack.PackError, match=r"layers\[1\]\.offset"):
        reopen(lambda m: m["experts"].__setitem__("n_experts", 5))  # layer 0 would run into layer 1
    reopen(lambda m: None)  # the untouched manifest opens again
    bin_path = os.path.join(d, "experts.bin")
    os.truncate(bin_path, os.path.getsize(bin_path) - 4096)
    with pytest.raises(pack.PackError, match=r"layers\[1\]: needs .* bytes"):
        pack.ExpertPack.open(d)
    with pytest.raises(pack.PackError, match="cannot open"):
        pack.ExpertPack.open(str(tmp_path / "nowhere"))


def test_formats_the_kernels_do_not_decode_are_named(tmp_path):
    """An IQ2_S / Q2_0 layer is a valid pack layer the decode kernels take; Q2_0 as a gate/up format (or
    IQ2_S as a down format) is a valid description too, but loading it for the GPU is refused by name."""
    hidden, inter = 256, 256
    info = pack.layer_info(IQ2_S, 42, hidden, inter, 0)
    blobs = np.zeros((2, info.blob_bytes), dtype=np.uint8)
    info2 = pack.layer_info(IQ4_NL, IQ2_S, hidden, inter, 0)
    blobs2 = np.zeros((2, info2.blob_bytes), dtype=np.uint8)
    d = str(tmp_path / "pack")
    pack.write_expert_pack(d, hidden, inter, [(IQ2_S, 42, blobs), (IQ4_NL, IQ2_S, blobs2)])
    p = pack.ExpertPack.open(d)
    assert p.layers[0].gate_bytes == 256 * 82 and p.layers[0].down_bytes == 256 * 4 * 18
    assert p.supported(0) and not p.supported(1)
    with pytest.raises(pack.PackError, match="IQ4_NL gate/up with IQ2_S down"):
        p.load_layer(1, device="cpu")
