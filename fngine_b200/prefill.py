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


def set_accumulation(fixed_point):
    """How the down projection hands results to the combine: True = 64-bit fixed-point per-token sums with
    integer atomics (the reference's scheme, moe.h:186-192), False = fp32 rows per pair added in ascending
    expert order. Process-wide; call it between layers, not inside one."""
    L.check(L.load().fb_moe_prefill_set_accumulation(1 if fixed_point else 0), "prefill_set_accumulation")


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


class SharedExpertPrefill:
    """The shared expert at prefill width: Fp8RowWeight gate_up (2 * inter_s, 2560) with the SwiGlu epilogue and
    down (2560, inter_s) with the SharedScale epilogue (src/kernels/linear/linear.h:11-12), exact activations.
    Owns the projection workspaces and the two intermediate buffers for up to `max_tokens` tokens."""

    def __init__(self, gate_up, down, max_tokens):
        from . import linear
        assert gate_up.n == 2 * down.k and down.n == gate_up.k
        self.gate_up, self.down = gate_up, down
        self.work_gu = linear.linear_fp8_workspace(gate_up, max_tokens)
        self.work_dn = linear.linear_fp8_workspace(down, max_tokens)
        self.h = torch.empty(max_tokens, down.k, dtype=torch.bfloat16, device=gate_up.codes.device)
        self.y = torch.empty(max_tokens, down.n, dtype=torch.float32, device=gate_up.codes.device)


def forward_moe_prefill(w_router, shared, layer, x, ws, inj, X, logits, y_out=None):
    """The prefill branch of Forward::moe (src/model/forward.cpp:333-353 of the reference): 513-row router
    projection (row 512 = the shared-expert gate), moe_route, the shared expert (linear_fp8 with the SwiGlu
    epilogue, then with SharedScale reading the shared-gate logit), grouped gate/up, grouped down, and the
    combine that adds y_shared and writes the residual streams X += inj * y. x: bf16 [T][2560];
    logits: fp32 scratch [T][513]."""
    from . import linear, moe
    T = x.shape[0]
    assert x.dtype == torch.bfloat16 and w_router.shape[0] == L.ROUTER_ROWS and T <= shared.h.shape[0]
    moe.router_logits(w_router, x, logits)
    moe_route(logits, x, None, 0, None, None, T, ws, logits_stride=L.ROUTER_ROWS)
    h, y_sh = shared.h[:T], shared.y[:T]
    linear.linear_fp8(x, shared.gate_up, linear.swiglu(h), shared.work_gu)
    gate = logits.view(-1)[L.ROUTER_ROWS - 1:]
    linear.linear_fp8(h, shared.down, linear.shared_scale(y_sh, gate, L.ROUTER_ROWS), shared.work_dn)
    moe_grouped_gate_up(layer, None, x, T, ws)
    moe_grouped_down(layer, None, T, ws)
    moe_prefill_combine(ws, y_sh, None, 0, None, inj, X, y_out, T)
