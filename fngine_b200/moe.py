"""Host-side mirror of the reference's routed-expert operator interface (decode path).

Function names and argument meaning follow src/kernels/moe/moe.h of the reference
(moe_select_publish / moe_hot_gate_up / moe_hot_down / moe_combine and the workspace helpers);
each call goes straight through the C ABI in include/fngine_b200.h. torch is used only to own
device memory and streams. Nothing here computes on the CPU.
"""
import ctypes as C

import numpy as np
import torch

from . import lib as L
from . import synth


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        assert t.is_cuda and t.is_contiguous()
        return t.data_ptr()
    return t


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _dtype_code(t):
    if t.dtype == torch.float32:
        return L.DT_F32
    if t.dtype == torch.bfloat16:
        return L.DT_BF16
    raise TypeError("activations must be float32 or bfloat16")


class ExpertLayer:
    """One layer's resident expert slot array (MoeExpertLayout, moe.h:62-76 of the reference)."""

    def __init__(self, slots, gate_up_format, down_format, inter, blob_stride=None):
        self.lib = L.load()
        self.slots = slots  # torch uint8 cuda tensor
        stride = blob_stride or self.lib.fb_moe_blob_bytes(gate_up_format, down_format, inter)
        self.layout = L.ExpertLayout()
        L.check(self.lib.fb_moe_expert_layout_make(slots.data_ptr(), stride, gate_up_format, down_format, inter,
                                                   C.byref(self.layout)), "expert_layout_make")
        self.n_slots = slots.numel() // stride
        self.blob_bytes = self.lib.fb_moe_blob_bytes(gate_up_format, down_format, inter)

    def with_slots(self, slots):
        return ExpertLayer(slots, self.layout.gate_up_format, self.layout.down_format, self.layout.inter,
                           self.layout.blob_stride)


def synth_layer(gate_up_format, down_format, inter, n_experts, seed, device="cuda", first_expert=0):
    """Seeded expert bytes generated on the device; synth.expert_blob() gives the same bytes on
    the host for any single expert. Slot s holds expert first_expert + s."""
    lib = L.load()
    stride = lib.fb_moe_blob_bytes(gate_up_format, down_format, inter)
    buf = torch.empty(n_experts * stride, dtype=torch.uint8, device=device)
    tables = {f: torch.from_numpy(synth.d_table(f).view(np.int16)).to(device) for f in {gate_up_format, down_format}}
    gu_bytes = 2 * inter * lib.fb_moe_row_bytes(gate_up_format, L.HIDDEN)
    nb_gu = gu_bytes // synth.BLOCK_BYTES[gate_up_format]
    nb_dn = (stride - gu_bytes) // synth.BLOCK_BYTES[down_format]
    fill_experts(buf, stride, gate_up_format, down_format, gu_bytes, nb_gu, nb_dn, n_experts, first_expert, seed, tables)
    return ExpertLayer(buf, gate_up_format, down_format, inter)


def synth_layer_of(gate_up_format, down_format, inter, experts, seed, device="cuda"):
    """The same seeded bytes for an arbitrary list of experts: slot s holds expert experts[s] (a placement's
    share of a layer). Consecutive ids are filled together."""
    lib = L.load()
    stride = lib.fb_moe_blob_bytes(gate_up_format, down_format, inter)
    experts = [int(e) for e in experts]
    buf = torch.empty(max(len(experts), 1) * stride, dtype=torch.uint8, device=device)
    tables = {f: torch.from_numpy(synth.d_table(f).view(np.int16)).to(device) for f in {gate_up_format, down_format}}
    gu_bytes = 2 * inter * lib.fb_moe_row_bytes(gate_up_format, L.HIDDEN)
    nb_gu = gu_bytes // synth.BLOCK_BYTES[gate_up_format]
    nb_dn = (stride - gu_bytes) // synth.BLOCK_BYTES[down_format]
    s = 0
    while s < len(experts):
        n = 1
        while s + n < len(experts) and experts[s + n] == experts[s] + n:
            n += 1
        fill_experts(buf[s * stride:], stride, gate_up_format, down_format, gu_bytes, nb_gu, nb_dn, n, experts[s], seed,
                     tables)
        s += n
    return ExpertLayer(buf, gate_up_format, down_format, inter)


def fill_experts(buf, stride, gate_up_format, down_format, gu_bytes, nb_gu, nb_dn, n_experts, first_expert, seed, tables):
    """Two launches for a whole slot array: the gate/up part and the down part of every expert."""
    lib = L.load()
    L.check(lib.fb_synth_fill_experts(gate_up_format, buf.data_ptr(), stride, n_experts, first_expert, nb_gu, seed,
                                      tables[gate_up_format].data_ptr(), _stream()), "synth_fill_experts")
    L.check(lib.fb_synth_fill_experts(down_format, buf.data_ptr() + gu_bytes, stride, n_experts, first_expert, nb_dn,
                                      seed ^ 0xD0, tables[down_format].data_ptr(), _stream()), "synth_fill_experts")


class DecodeWorkspace:
    """MoeDecodeWorkspace (moe.h:108-117 of the reference): caller-owned, allocated once."""

    def __init__(self, layer=None, device="cuda"):
        """layer=None makes a workspace that fits every layout (the reference's make_moe_decode_workspace takes
        no layout either); the stand-alone selection then quantizes x for both activation formats."""
        self.lib = L.load()
        n = self.lib.fb_moe_decode_workspace_bytes(layer.layout.inter if layer is not None else 640)
        self.buf = torch.zeros(n + 256, dtype=torch.uint8, device=device)
        base = (self.buf.data_ptr() + 255) & ~255
        self.ws = L.DecodeWorkspace()
        L.check(self.lib.fb_moe_decode_workspace_make(base, C.byref(layer.layout) if layer is not None else None,
                                                      C.byref(self.ws)), "decode_workspace_make")
        self.logits = torch.empty(L.DECODE_MAX_TOKENS * L.ROUTER_ROWS, dtype=torch.float32, device=device)

    def _view(self, ptr, nbytes):
        off = ptr - self.buf.data_ptr()
        return self.buf[off:off + nbytes]

    def work(self):
        """Host copy of the device work list."""
        raw = self._view(self.ws.work, C.sizeof(L.DecodeWork)).cpu().numpy().tobytes()
        return L.DecodeWork.from_buffer_copy(raw)

    def status(self):
        return int(self._view(self.ws.status, 4).view(torch.int32).item())

    def xq(self, tokens, act=L.ACT_Q8_K):
        """Planar activation rows of the step's tokens: the Q8_K rows, or (act = ACT_Q8_0) the Q8_0 rows."""
        both = self._view(self.ws.xq, 2 * L.DECODE_MAX_TOKENS * L.XQ_STRIDE).view(2, L.DECODE_MAX_TOKENS, L.XQ_STRIDE)
        return both[1 if act == L.ACT_Q8_0 else 0, :tokens].cpu().numpy()

    def hq(self, pairs):
        return self._view(self.ws.hq, L.DECODE_MAX_PAIRS * L.HQ_STRIDE).view(L.DECODE_MAX_PAIRS, L.HQ_STRIDE)[:pairs].cpu().numpy()

    def h(self, pairs):
        inter = self.ws.inter or 640
        return self._view(self.ws.h, L.DECODE_MAX_PAIRS * inter * 4).view(torch.float32).view(L.DECODE_MAX_PAIRS, inter)[:pairs].cpu().numpy()

    def partial(self, pairs):
        return self._view(self.ws.partial, L.DECODE_MAX_PAIRS * L.HIDDEN * 4).view(torch.float32).view(L.DECODE_MAX_PAIRS, L.HIDDEN)[:pairs].cpu().numpy()


def router_logits(w_router, x, logits, stride=L.ROUTER_ROWS):
    """linear_bf16 (513|512, 2560) StoreF32 of the reference (linear.h:20): logits fp32."""
    lib = L.load()
    tokens = x.shape[0]
    L.check(lib.fb_router_logits(_ptr(w_router), w_router.shape[0], _ptr(x), _dtype_code(x), tokens, _ptr(logits),
                                 stride, _stream()), "router_logits")


def moe_select_publish(router_logits_, x, slot_of, layer, seq, exchange, tokens, ws, routing_counts=None,
                       logits_stride=L.ROUTER_ROWS):
    lib = L.load()
    L.check(lib.fb_moe_select_publish(_ptr(router_logits_), logits_stride, _ptr(x), _dtype_code(x), _ptr(slot_of),
                                      layer, _ptr(seq), exchange, tokens, C.byref(ws.ws), _stream(),
                                      _ptr(routing_counts)), "moe_select_publish")


def moe_hot_gate_up(layer, tokens, ws):
    L.check(L.load().fb_moe_hot_gate_up(C.byref(layer.layout), tokens, C.byref(ws.ws), _stream()), "moe_hot_gate_up")


def moe_hot_down(layer, tokens, ws):
    L.check(L.load().fb_moe_hot_down(C.byref(layer.layout), tokens, C.byref(ws.ws), _stream()), "moe_hot_down")


def moe_hot_experts(layer, tokens, ws):
    """moe_hot_gate_up + moe_hot_down, one launch where the formats allow it."""
    L.check(L.load().fb_moe_hot_experts(C.byref(layer.layout), tokens, C.byref(ws.ws), _stream()), "moe_hot_experts")


def moe_combine(ws, y_shared, exchange, layer, seq, inj, X, y_out, tokens, timeout_cycles=0, ablate_direction=None,
                ablate_scale=0.0):
    L.check(L.load().fb_moe_combine(C.byref(ws.ws), _ptr(y_shared), exchange, layer, _ptr(seq), _ptr(inj), _ptr(X),
                                    _ptr(y_out), tokens, timeout_cycles, _ptr(ablate_direction), ablate_scale,
                                    _stream()), "moe_combine")


def moe_layer_decode(w_router, layer, x, ws, y_out):
    """Router projection -> select -> gate/up -> down -> combine for one layer (device tensors)."""
    L.check(L.load().fb_moe_layer_decode(_ptr(w_router), C.byref(layer.layout), _ptr(x), _dtype_code(x), x.shape[0],
                                         C.byref(ws.ws), _ptr(ws.logits), _ptr(y_out), _stream()), "moe_layer_decode")


class SharedExpert:
    """The shared expert of one layer as the reference registers it (src/kernels/linear/linear.h:11-12):
    gate_up = Fp8RowWeight (2 * inter_s, 2560) with the SwiGlu epilogue, down = Fp8RowWeight (2560, inter_s)
    with the SharedScale epilogue. Owns the workspaces and the two intermediate buffers."""

    def __init__(self, gate_up, down, max_tokens=16):
        from . import linear
        assert gate_up.n == 2 * down.k and down.n == gate_up.k
        self.gate_up, self.down = gate_up, down
        self.work_gu = linear.linear_fp8_decode_workspace(gate_up)
        self.work_dn = linear.linear_fp8_decode_workspace(down)
        self.h = torch.empty(max_tokens, down.k, dtype=torch.bfloat16, device=gate_up.codes.device)
        self.y = torch.empty(max_tokens, down.n, dtype=torch.float32, device=gate_up.codes.device)


def forward_moe_decode(w_router, shared, layer, x, ws, inj, X, y_out=None, aux_stream=None):
    """The decode branch of Forward::moe (src/model/forward.cpp:333,356-376 of the reference): router
    projection (513 rows, row 512 = the shared gate), select, the shared expert beside the routed
    experts on `aux_stream` (its down epilogue reads the shared-gate logit), gate/up, down, and the
    combine that adds y_shared and writes the residual streams X += inj * y. x: bf16 [T][2560]."""
    from . import linear
    T = x.shape[0]
    assert x.dtype == torch.bfloat16 and w_router.shape[0] == L.ROUTER_ROWS and T <= shared.h.shape[0]
    router_logits(w_router, x, ws.logits)
    moe_select_publish(ws.logits, x, None, 0, None, None, T, ws)
    cur = torch.cuda.current_stream()
    side = aux_stream if aux_stream is not None else cur
    if side is not cur:
        side.wait_stream(cur)
    with torch.cuda.stream(side):
        h, y_sh = shared.h[:T], shared.y[:T]
        linear.linear_fp8_decode(x, shared.gate_up, linear.swiglu(h), shared.work_gu)
        gate = ws.logits.view(-1)[L.ROUTER_ROWS - 1:]
        linear.linear_fp8_decode(h, shared.down, linear.shared_scale(y_sh, gate, L.ROUTER_ROWS), shared.work_dn)
    moe_hot_gate_up(layer, T, ws)
    moe_hot_down(layer, T, ws)
    if side is not cur:
        cur.wait_stream(side)
    moe_combine(ws, shared.y, None, 0, None, inj, X, y_out, T)


def moe_layer_decode_host(w_router, layer, x_host, ws, x_dev, y_dev, y_host):
    """Same with pinned HOST x / y: the copies in and out and the final wait are inside the call."""
    L.check(L.load().fb_moe_layer_decode_host(_ptr(w_router), C.byref(layer.layout), x_host.data_ptr(),
                                              _dtype_code(x_host), x_host.shape[0], C.byref(ws.ws), _ptr(ws.logits),
                                              _ptr(x_dev), _ptr(y_dev), y_host.data_ptr(), _stream()),
            "moe_layer_decode_host")


def moe_layer_decode_static(w_router, layer, x, y_out):
    """The decode layer with the library's built-in scratch (for callers that cannot allocate)."""
    L.check(L.load().fb_moe_layer_decode_static(_ptr(w_router), C.byref(layer.layout), _ptr(x), _dtype_code(x),
                                                x.shape[0], _ptr(y_out), _stream()), "moe_layer_decode_static")


def moe_layer_decode_static_status():
    """FB_STATUS_* word the last moe_layer_decode_static call on the current GPU left behind."""
    out = C.c_uint32(0xFFFFFFFF)
    L.check(L.load().fb_moe_layer_decode_static_status(C.byref(out), _stream()), "moe_layer_decode_static_status")
    return int(out.value)


def dequant_rows(fmt, rows, nrows, k):
    """Exact fp32 weights of `nrows` back-to-back rows (device uint8 tensor)."""
    lib = L.load()
    out = torch.empty(nrows, k, dtype=torch.float32, device=rows.device)
    L.check(lib.fb_dequant_rows(fmt, _ptr(rows), lib.fb_moe_row_bytes(fmt, k), nrows, k, _ptr(out), _stream()),
            "dequant_rows")
    return out


def quantize_act(act, x):
    """ggml activation blocks (block_q8_K / block_q8_0 bytes) of x [rows][k]."""
    lib = L.load()
    rows, k = x.shape
    out = torch.zeros(rows, lib.fb_act_row_bytes(act, k), dtype=torch.uint8, device=x.device)
    L.check(lib.fb_quantize_act(act, _ptr(x), _dtype_code(x), rows, k, _ptr(out), _stream()), "quantize_act")
    return out
