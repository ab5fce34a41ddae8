"""Expert weights from the reference's files: the `experts` section of a pack's manifest.json with its
experts.bin (src/io/pack.h:53-78, written by tools/convert.py:272-323 of the reference) and the expert
tensors `blk.N.ffn_{gate,up,down}_exps.weight` of a GGUF v3 file (tools/gguf.py:68-100). Both give, per
layer, 512 blobs `gate | up | down` of raw ggml blocks; `load_layer` puts them in HBM as the slot array
the kernels read (stride kept from the pack, 4096-aligned).

The decode kernels take gate/up in IQ3_S, IQ4_NL, IQ3_XXS, IQ2_S or IQ4_XS and down in IQ3_S, IQ4_NL or Q2_0
(IQ3_S and IQ4_NL through the streaming kernels, the others through plain ones). A layer in another
combination of the pack spec's formats is described and validated like the rest, and refused by `load_layer`
with a PackError that names it. Everything here is host code; device memory comes from torch."""
import json
import os
import struct
from collections import OrderedDict, namedtuple

import numpy as np

# ggml type id -> (name, block bytes, block elements): the expert formats of the pack spec (pack.h:53-61)
EXPERT_TYPES = {18: ("IQ3_XXS", 98, 256), 20: ("IQ4_NL", 18, 32), 21: ("IQ3_S", 110, 256), 22: ("IQ2_S", 82, 256),
                23: ("IQ4_XS", 136, 256), 42: ("Q2_0", 18, 64)}
TYPE_ID_OF = {v[0]: k for k, v in EXPERT_TYPES.items()}
GATE_UP_FORMATS = (18, 20, 21, 22, 23)  # what the GPU decode kernels take as gate/up ...
DOWN_FORMATS = (20, 21, 42)             # ... and as down
BLOB_ALIGN = 4096


class PackError(RuntimeError):
    """A manifest or file that does not describe what it should; the message names the field."""


def row_bytes(type_id, elements):
    """ggml_row_bytes (pack.h:63): bytes of one row of `elements` values."""
    if type_id not in EXPERT_TYPES:
        raise PackError("unknown ggml type id %r" % (type_id,))
    name, bb, be = EXPERT_TYPES[type_id]
    if elements <= 0 or elements % be:
        raise PackError("%d elements are not a multiple of the %s block (%d)" % (elements, name, be))
    return elements // be * bb


def align_up(v, a=BLOB_ALIGN):
    return (v + a - 1) // a * a


ExpertLayerInfo = namedtuple("ExpertLayerInfo", "gu_type down_type gate_bytes up_bytes down_bytes blob_bytes "
                                                "blob_stride offset")


def layer_info(gu_type, down_type, hidden, inter, offset):
    """The layout convert.py's expert_layout gives one layer (tools/convert.py:272-296)."""
    gb = inter * row_bytes(gu_type, hidden)
    db = hidden * row_bytes(down_type, inter)
    blob = 2 * gb + db
    return ExpertLayerInfo(gu_type, down_type, gb, gb, db, blob, align_up(blob), offset)


def _type_id(field, where):
    if isinstance(field, str):
        if field not in TYPE_ID_OF:
            raise PackError("%s: unsupported expert format %r" % (where, field))
        return TYPE_ID_OF[field]
    if field not in EXPERT_TYPES:
        raise PackError("%s: unsupported expert format id %r" % (where, field))
    return int(field)


class ExpertPack:
    """manifest.json + experts.bin of a pack directory (only the expert part of the manifest is read)."""

    def __init__(self, directory, n_experts, hidden, inter, layers, path):
        self.dir, self.n_experts, self.hidden, self.inter = directory, n_experts, hidden, inter
        self.layers, self.path = layers, path
        self._mm = None

    @classmethod
    def open(cls, directory):
        mpath = os.path.join(directory, "manifest.json")
        try:
            with open(mpath) as f:
                man = json.load(f)
        except OSError as e:
            raise PackError("cannot open %s: %s" % (mpath, e))
        except ValueError as e:
            raise PackError("%s is not JSON: %s" % (mpath, e))
        if man.get("format") != "fngine-pack":
            raise PackError("format: expected 'fngine-pack', found %r" % (man.get("format"),))
        try:
            ex = man["experts"]
            n_experts, hidden, inter = int(ex["n_experts"]), int(ex["hidden"]), int(ex["intermediate"])
            raw_layers = ex["layers"]
            fname = man["files"]["experts"]
        except (KeyError, TypeError, ValueError) as e:
            raise PackError("manifest: missing or malformed field %s" % (e,))
        if int(ex.get("n_layers", len(raw_layers))) != len(raw_layers):
            raise PackError("experts.n_layers: %r but %d layers listed" % (ex.get("n_layers"), len(raw_layers)))
        path = os.path.join(directory, fname)
        if not os.path.exists(path):
            raise PackError("files.experts: %s does not exist" % path)
        size = os.path.getsize(path)
        layers, end = [], 0
        for i, j in enumerate(raw_layers):
            where = "experts.layers[%d]" % i
            try:
                gu = _type_id(j.get("gu_type_id", j["gu_type"]), where + ".gu_type")
                dn = _type_id(j.get("down_type_id", j["down_type"]), where + ".down_type")
                if isinstance(j["gu_type"], str) and TYPE_ID_OF.get(j["gu_type"]) != gu:
                    raise PackError("%s.gu_type_id: %r does not name %r" % (where, gu, j["gu_type"]))
                if isinstance(j["down_type"], str) and TYPE_ID_OF.get(j["down_type"]) != dn:
                    raise PackError("%s.down_type_id: %r does not name %r" % (where, dn, j["down_type"]))
                got = ExpertLayerInfo(gu, dn, *(int(j[k]) for k in ("gate_bytes", "up_bytes", "down_bytes", "blob_bytes",
                                                                  "blob_stride", "offset")))
            except KeyError as e:
                raise PackError("%s: missing field %s" % (where, e))
            want = layer_info(gu, dn, hidden, inter, got.offset)
            for k in ("gate_bytes", "up_bytes", "down_bytes", "blob_bytes"):
                if getattr(got, k) != getattr(want, k):
                    raise PackError("%s.%s: %d, expected %d for %s/%s at hidden %d, intermediate %d" %
                                    (where, k, getattr(got, k), getattr(want, k), EXPERT_TYPES[gu][0],
                                     EXPERT_TYPES[dn][0], hidden, inter))
            if got.blob_stride % BLOB_ALIGN or got.blob_stride < got.blob_bytes:
                raise PackError("%s.blob_stride: %d is not a multiple of %d that holds %d bytes" %
                                (where, got.blob_stride, BLOB_ALIGN, got.blob_bytes))
            if got.offset % BLOB_ALIGN or got.offset < end:
                raise PackError("%s.offset: %d overlaps the previous layer or is not %d-aligned" %
                                (where, got.offset, BLOB_ALIGN))
            end = got.offset + n_experts * got.blob_stride
            if end > size:
                raise PackError("%s: needs %d bytes of %s, which has %d" % (where, end, fname, size))
            layers.append(got)
        return cls(directory, n_experts, hidden, inter, layers, path)

    # ------------------------------------------------------------------ bytes
    def _map(self):
        if self._mm is None:
            self._mm = np.memmap(self.path, dtype=np.uint8, mode="r")
        return self._mm

    def blob(self, layer, expert):
        """The gate | up | down bytes of one expert (a view of the mapped file)."""
        info = self.layers[layer]
        if not 0 <= expert < self.n_experts:
            raise PackError("expert %d out of range" % expert)
        o = info.offset + expert * info.blob_stride
        return self._map()[o:o + info.blob_bytes]

    def layer_bytes(self, layer, first=0, count=None):
        """Slot array [count][blob_stride] of experts first .. first + count - 1 (a view of the mapped file)."""
        info = self.layers[layer]
        count = self.n_experts - first if count is None else count
        if first < 0 or count < 0 or first + count > self.n_experts:
            raise PackError("experts %d..%d out of range" % (first, first + count))
        o = info.offset + first * info.blob_stride
        return self._map()[o:o + count * info.blob_stride].reshape(count, info.blob_stride)

    def supported(self, layer):
        info = self.layers[layer]
        return info.gu_type in GATE_UP_FORMATS and info.down_type in DOWN_FORMATS

    def load_layer(self, layer, first=0, count=None, device="cuda"):
        """The layer's experts (or the shard first .. first + count - 1 of them) as an ExpertLayer in HBM."""
        return _to_device(self.layers[layer], self.inter, self.layer_bytes(layer, first, count), "layer %d" % layer,
                          device)


def _to_device(info, inter, slots, what, device):
    import torch

    from . import moe
    if info.gu_type not in GATE_UP_FORMATS or info.down_type not in DOWN_FORMATS:
        raise PackError("%s: %s gate/up with %s down is in the pack spec but not decoded by the kernels "
                        "(gate/up: IQ3_S, IQ4_NL, IQ3_XXS, IQ2_S, IQ4_XS; down: IQ3_S, IQ4_NL, Q2_0)"
                        % (what, EXPERT_TYPES[info.gu_type][0], EXPERT_TYPES[info.down_type][0]))
    host = torch.from_numpy(np.array(slots, dtype=np.uint8, order="C")).reshape(-1)  # a writable copy of the mapped bytes
    dev = torch.empty(host.numel(), dtype=torch.uint8, device=device)
    dev.copy_(host.pin_memory() if torch.cuda.is_available() else host, non_blocking=False)
    return moe.ExpertLayer(dev, info.gu_type, info.down_type, inter, info.blob_stride)


def write_expert_pack(directory, hidden, inter, layers):
    """Writes manifest.json (the expert part, fields as tools/convert.py:516-528 of the reference) and
    experts.bin. layers: list of (gu_type id, down_type id, uint8 array [n_experts][blob_bytes])."""
    os.makedirs(directory, exist_ok=True)
    n_experts = len(layers[0][2])
    infos, off = [], 0
    for gu, dn, blobs in layers:
        info = layer_info(gu, dn, hidden, inter, off)
        blobs = np.asarray(blobs, dtype=np.uint8)
        if blobs.shape != (n_experts, info.blob_bytes):
            raise PackError("blobs of shape %r, expected %r" % (blobs.shape, (n_experts, info.blob_bytes)))
        infos.append(info)
        off += n_experts * info.blob_stride
    with open(os.path.join(directory, "experts.bin"), "wb") as f:
        for info, (_, _, blobs) in zip(infos, layers):
            padded = np.zeros((n_experts, info.blob_stride), dtype=np.uint8)
            padded[:, :info.blob_bytes] = blobs
            f.write(padded.tobytes())
    man = {"format": "fngine-pack", "version": 1, "files": {"experts": "experts.bin"},
           "experts": {"n_layers": len(infos), "n_experts": n_experts, "hidden": hidden, "intermediate": inter,
                       "layers": [{"gu_type": EXPERT_TYPES[i.gu_type][0], "down_type": EXPERT_TYPES[i.down_type][0],
                                   "gu_type_id": i.gu_type, "down_type_id": i.down_type, "gate_bytes": i.gate_bytes,
                                   "up_bytes": i.up_bytes, "down_bytes": i.down_bytes, "blob_bytes": i.blob_bytes,
                                   "blob_stride": i.blob_stride, "offset": i.offset} for i in infos]}}
    with open(os.path.join(directory, "manifest.json"), "w") as f:
        json.dump(man, f, indent=1)
    return infos


# ---------------------------------------------------------------------------------------------- GGUF
GgufTensor = namedtuple("GgufTensor", "name ne type_id offset nbytes")
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


class GgufExperts:
    """The expert tensors of a GGUF v3 file. Metadata values are parsed only far enough to be skipped,
    except `general.alignment`; a tensor of a type outside the expert formats is listed with nbytes None."""

    def __init__(self, path):
        self.path = path
        self.mm = np.memmap(path, dtype=np.uint8, mode="r")
        if self.mm.size < 24 or bytes(self.mm[:4]) != b"GGUF":
            raise PackError("%s: not a GGUF file" % path)
        self._pos = 4
        version = self._take("<I")
        if version != 3:
            raise PackError("%s: GGUF version %d, expected 3" % (path, version))
        n_tensors, n_kv = self._take("<Q"), self._take("<Q")
        self.alignment = 32
        for _ in range(n_kv):
            key = self._string()
            val = self._value(self._take("<I"))
            if key == "general.alignment":
                self.alignment = int(val)
        raw = []
        for _ in range(n_tensors):
            name = self._string()
            nd = self._take("<I")
            ne = [self._take("<Q") for _ in range(nd)]
            raw.append((name, ne, self._take("<I"), self._take("<Q")))
        self.data_start = align_up(self._pos, self.alignment)
        self.tensors = OrderedDict()
        for name, ne, t, off in raw:
            nb = None
            if t in EXPERT_TYPES:
                rows = 1
                for d in ne[1:]:
                    rows *= d
                nb = rows * row_bytes(t, ne[0])
                if self.data_start + off + nb > self.mm.size:
                    raise PackError("%s: tensor %s runs past the end of the file" % (path, name))
            self.tensors[name] = GgufTensor(name, ne, t, self.data_start + off, nb)

    def _take(self, fmt):
        n = struct.calcsize(fmt)
        if self._pos + n > self.mm.size:
            raise PackError("%s: truncated header" % self.path)
        v = struct.unpack_from(fmt, self.mm, self._pos)[0]
        self._pos += n
        return v

    def _string(self):
        n = self._take("<Q")
        if self._pos + n > self.mm.size:
            raise PackError("%s: truncated string" % self.path)
        s = bytes(self.mm[self._pos:self._pos + n]).decode("utf-8", "replace")
        self._pos += n
        return s

    def _value(self, vt):
        if vt == 8:
            return self._string()
        if vt == 9:
            et, n = self._take("<I"), self._take("<Q")
            if et in _SCALAR:
                self._pos += struct.calcsize(_SCALAR[et]) * n
                return None
            return [self._value(et) for _ in range(n)]
        if vt not in _SCALAR:
            raise PackError("%s: unknown metadata value type %d" % (self.path, vt))
        return self._take(_SCALAR[vt])

    def layers(self):
        """Indices N for which blk.N.ffn_{gate,up,down}_exps.weight are all present."""
        out = []
        for name in self.tensors:
            if name.startswith("blk.") and name.endswith(".ffn_gate_exps.weight"):
                n = int(name.split(".")[1])
                if all("blk.%d.ffn_%s_exps.weight" % (n, k) in self.tensors for k in ("up", "down")):
                    out.append(n)
        return sorted(out)

    def layer_layout(self, layer):
        """(ExpertLayerInfo, n_experts, hidden, inter) with the checks of tools/convert.py:275-289."""
        t = {k: self.tensors.get("blk.%d.ffn_%s_exps.weight" % (layer, k)) for k in ("gate", "up", "down")}
        for k, v in t.items():
            if v is None:
                raise PackError("blk.%d.ffn_%s_exps.weight is missing" % (layer, k))
            if v.type_id not in EXPERT_TYPES or len(v.ne) != 3:
                raise PackError("%s: not a 3-D tensor of an expert format" % v.name)
        if t["up"].type_id != t["gate"].type_id:
            raise PackError("layer %d: gate type %s != up type %s" % (layer, EXPERT_TYPES[t["gate"].type_id][0],
                                                                      EXPERT_TYPES[t["up"].type_id][0]))
        hidden, inter, n_experts = t["gate"].ne
        if t["up"].ne != [hidden, inter, n_experts] or t["down"].ne != [inter, hidden, n_experts]:
            raise PackError("layer %d: unexpected expert shapes %r %r %r" % (layer, t["gate"].ne, t["up"].ne, t["down"].ne))
        return layer_info(t["gate"].type_id, t["down"].type_id, hidden, inter, 0), n_experts, hidden, inter

    def layer_bytes(self, layer, first=0, count=None):
        """Slot array [count][blob_stride]: expert e's gate, up and down slices side by side, as
        write_experts does (tools/convert.py:297-318)."""
        info, n_experts, _, _ = self.layer_layout(layer)
        count = n_experts - first if count is None else count
        if first < 0 or count < 0 or first + count > n_experts:
            raise PackError("experts %d..%d out of range" % (first, first + count))
        out = np.zeros((count, info.blob_stride), dtype=np.uint8)
        pos = 0
        for k, nb in (("gate", info.gate_bytes), ("up", info.up_bytes), ("down", info.down_bytes)):
            t = self.tensors["blk.%d.ffn_%s_exps.weight" % (layer, k)]
            src = self.mm[t.offset + first * nb:t.offset + (first + count) * nb].reshape(count, nb)
            out[:, pos:pos + nb] = src
            pos += nb
        return out

    def load_layer(self, layer, first=0, count=None, device="cuda"):
        info, _, _, inter = self.layer_layout(layer)
        return _to_device(info, inter, self.layer_bytes(layer, first, count), "blk.%d" % layer, device)


def write_gguf(path, tensors, metadata=None, alignment=32):
    """A GGUF v3 file with the given tensors: list of (name, ne, ggml type id, bytes-like). Metadata: dict of
    str -> int (u32) or str. Enough of the format for expert tensors and for tests."""
    metadata = dict(metadata or {})
    metadata.setdefault("general.alignment", alignment)

    def s(x):
        b = x.encode("utf-8")
        return struct.pack("<Q", len(b)) + b

    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(metadata))
    for k, v in metadata.items():
        head += s(k) + (struct.pack("<I", 8) + s(v) if isinstance(v, str) else struct.pack("<II", 4, int(v)))
    infos, off = b"", 0
    offsets = []
    for name, ne, t, data in tensors:
        infos += s(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne) + struct.pack("<IQ", t, off)
        offsets.append(off)
        off = align_up(off + len(bytes(data)) if not isinstance(data, np.ndarray) else off + data.nbytes, alignment)
    start = align_up(len(head) + len(infos), alignment)
    with open(path, "wb") as f:
        f.write(head + infos)
        f.write(b"\0" * (start - len(head) - len(infos)))
        for (name, ne, t, data), o in zip(tensors, offsets):
            f.seek(start + o)
            f.write(data.tobytes() if isinstance(data, np.ndarray) else bytes(data))
        f.truncate(start + off)
