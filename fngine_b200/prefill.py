"""Host-side mirror of the reference's prefill MoE operators (moe_route, moe_grouped_gate_up,
moe_grouped_down, moe_prefill_combine; src/kernels/moe/moe.h:193-226 of the reference). Every call
goes through the C ABI; torch only owns device memory."""
import ctypes as C

import torch

from . import lib as L
from .moe import _ptr, _stream


class PrefillWorkspace:
    """MoePrefillWorkspace (moe.h:167-194 of the reference): caller-owned, sized for `capacity` tokens."""

    def __init__(self, capacity, inter, device="cuda"):
        self.lib = L.load()
        n = self.lib.fb_moe_prefill_workspace_bytes(capacity, inter)
        if n == 0:
            raise L.FbError("unsupported prefill workspace shape")
        self.buf = torch.zeros(n + 256, dtype=torch.uint8, device=device)
        base = (self.buf.data_ptr() + 255) & ~255
        self.ws = L.PrefillWorkspace()
        L.check(self.lib.fb_moe_prefill_workspace_make(base, capacity, inter, C.byref(self.ws)), "prefill_workspace_make")
        self.capacity, self.inter = capacity, inter

    def _view(self, ptr, nbytes):
        off = ptr - self.buf.data_ptr()
        return self.buf[off:off + nbytes]

    def ints(self, ptr, n):
        return self._view(ptr, 4 * n).view(torch.int32).cpu().numpy()

    def floats(self, ptr, n):
        return self._view(ptr, 4 * n).view(torch.float32).cpu().numpy()

    def meta(self):
        return self.ints(self.ws.meta, 3)

    def status(self):
        return int(self.ints(self.ws.status, 1)[0])

    def h(self, pairs):
        return self._view(self.ws.h, 2 * pairs * self.inter).view(torch.int16).cpu().numpy().view("uint16").reshape(pairs, self.inter)


def moe_route(router_logits, x, expert_blob, layer, seq, control, tokens, ws, logits_stride=None):
    stride = logits_stride or router_logits.shape[-1]
    L.check(L.load().fb_moe_route(_ptr(router_logits), stride, _ptr(x), _ptr(expert_blob), layer, _ptr(seq), control,
                                  tokens, C.byref(ws.ws), _stream()), "moe_route")


def moe_grouped_gate_up(layer, expert_blob, x, tokens, ws):
    assert x.dtype == torch.bfloat16
    L.check(L.load().fb_moe_grouped_gate_up(C.byref(layer.layout), _ptr(expert_blob), _ptr(x), tokens, C.byref(ws.ws),
                                            _stream()), "moe_grouped_gate_up")


def moe_grouped_down(layer, expert_blob, tokens, ws):
    L.check(L.load().fb_moe_grouped_down(C.byref(layer.layout), _ptr(expert_blob), tokens, C.byref(ws.ws), _stream()),
            "moe_grouped_down")


def moe_prefill_combine(ws, y_shared, control, layer, seq, inj, X, y_out, tokens, timeout_cycles=0,
                        ablate_direction=None, ablate_scale=0.0):
    L.check(L.load().fb_moe_prefill_combine(C.byref(ws.ws), _ptr(y_shared), control, layer, _ptr(seq), _ptr(inj),
                                            _ptr(X), _ptr(y_out), tokens, timeout_cycles, _ptr(ablate_direction),
                                            ablate_scale, _stream()), "moe_prefill_combine")


def moe_layer_prefill(router_logits, layer, x, ws, y_out):
    """route -> grouped gate/up -> grouped down -> combine for one layer (the prefill branch of
    Forward::moe, src/model/forward.cpp:334-353 of the reference, without the shared expert)."""
    tokens = x.shape[0]
    moe_route(router_logits, x, None, 0, None, None, tokens, ws)
    moe_grouped_gate_up(layer, None, x, tokens, ws)
    moe_grouped_down(layer, None, tokens, ws)
    moe_prefill_combine(ws, None, None, 0, None, None, None, y_out, tokens)
