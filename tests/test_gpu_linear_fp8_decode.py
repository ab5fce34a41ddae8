"""GPU parity of the decode-width FP8-row projection (T <= 16, exact bf16 activations) through the C ABI.

Bars are the reference's own for its A16 path (tests/kernels/linear/test_linear.cpp:38-49,196-320):
against an fp64 dot product over the E4M3 weight values and the bf16 activations, times the row
scale, pushed through the epilogue in fp64,
  max(|got - ref| - allowance) <= 2e-3 * rms(ref), allowance = 1.001 * 2^-8 |ref| for bf16 outputs, 0 for fp32,
  and at least 99 % of the bf16 outputs equal bf16_rne(ref);
repeated calls are bitwise identical. The activation split that feeds the tensor core (three E5M2
pieces per value) is checked to be exact: scale * (p0 + p1 + p2) == x bit for bit."""
import numpy as np
import pytest

from fngine_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu
KTOL = 2e-3


def _torch():
    import torch
    assert torch.cuda.is_available()
    return torch


def bf16_tensor(torch, x):
    return torch.from_numpy(synth.to_bf16_bits(x).view(np.int16)).cuda().view(torch.bfloat16)


def make_weight(torch, seed, n, k, bf16_scales):
    from fngine_b200 import linear
    codes, scales = synth.fp8_row_weight(seed, n, k)
    wc, ws = torch.from_numpy(codes).cuda(), torch.from_numpy(scales).cuda()
    if bf16_scales:
        ws = ws.to(torch.bfloat16)
    return linear.Fp8RowWeight(wc, ws)


def exact_acc(torch, x, weight):
    """fp64 [T][n]: (x . W^T) * scale over the represented values."""
    tab = torch.from_numpy(O.e4m3_table().astype(np.float64)).cuda()
    out = torch.empty(x.shape[0], weight.n, dtype=torch.float64, device="cuda")
    xd = x.double()
    for r0 in range(0, weight.n, 4096):  # bounded fp64 temporaries
        w = tab[weight.codes[r0:r0 + 4096].long()]
        out[:, r0:r0 + 4096] = (xd @ w.T) * weight.scales[r0:r0 + 4096].double()[None, :]
    return out


def compare(torch, got, ref, bf16_out):
    got, ref = got.double().reshape(-1), ref.reshape(-1)
    rms = float(ref.pow(2).mean().sqrt())
    allowance = ref.abs() * (2.0 ** -8 * 1.001) if bf16_out else 0.0
    worst = float(((got - ref).abs() - allowance).max())
    assert bool(torch.isfinite(got).all())
    assert worst <= KTOL * rms, (worst, rms)
    if bf16_out:
        match = float((got.float() == ref.float().to(torch.bfloat16).float()).double().mean())
        assert match >= 0.99, match
        return worst / rms, match
    return worst / rms, 1.0


CASES = [
    # T, n, k, epilogue, bf16 row scales
    (1, 1280, 2560, "swiglu", True),          # moe.shared_gate_up
    (16, 1280, 2560, "swiglu", False),
    (9, 2560, 640, "shared_scale", True),     # moe.shared_down: five K blocks, every tile is shared by CTAs
    (5, 2560, 6144, "gr_write", True),        # gdn.out / qsa.o
    (16, 16384, 2560, "store_bf16", True),    # gdn.qkvz
    (3, 320, 10240, "store_f32", False),      # three row tiles, eighty K blocks each
    (7, 1000, 384, "store_bf16", False),      # ragged last row tile
    (16, 24832, 2560, "store_f32", True),     # a tenth of the vocabulary projection
    (2, 208, 256, "swiglu", False),           # 104 gate rows: ragged 64-row halves
    (4, 128, 128, "store_f32", True),         # one tile, one K block, one CTA
]


@pytest.mark.parametrize("T,n,k,kind,bf16_scales", CASES)
def test_linear_fp8_decode_matches_the_exact_product(T, n, k, kind, bf16_scales):
    torch = _torch()
    from fngine_b200 import linear
    weight = make_weight(torch, 300 + n + T, n, k, bf16_scales)
    x = bf16_tensor(torch, synth.activations(500 + T + k, T, hidden=k) * np.float32(1.7))
    work = linear.linear_fp8_decode_workspace(weight)
    acc = exact_acc(torch, x, weight)
    gen = torch.Generator(device="cpu").manual_seed(7 + T)
    if kind == "store_bf16":
        out = torch.full((T, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        make = lambda o: linear.store_bf16(o)
        ref, bf16_out = acc, True
    elif kind == "store_f32":
        out = torch.full((T, n), float("nan"), dtype=torch.float32, device="cuda")
        make = lambda o: linear.store_f32(o)
        ref, bf16_out = acc, False
    elif kind == "swiglu":
        out = torch.full((T, n // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
        make = lambda o: linear.swiglu(o)
        g, u = acc[:, :n // 2], acc[:, n // 2:]
        ref, bf16_out = g / (1.0 + torch.exp(-g)) * u, True
    elif kind == "shared_scale":
        logits = torch.randn(T, 513, generator=gen).cuda()
        out = torch.full((T, n), float("nan"), dtype=torch.float32, device="cuda")
        make = lambda o: linear.shared_scale(o, logits[:, 512:], 513)
        ref, bf16_out = acc * torch.sigmoid(logits[:, 512].double())[:, None], False
    else:
        inj = torch.randn(T, 4, generator=gen).cuda()
        x0 = torch.randn(T, 4, n, generator=gen).cuda()
        out = x0.clone()
        make = lambda o: linear.gr_write(o, inj)
        ref, bf16_out = inj.double()[:, :, None] * acc[:, None, :], False
    linear.linear_fp8_decode(x, weight, make(out), work)
    torch.cuda.synchronize()
    got = out.double() - x0.double() if kind == "gr_write" else out
    ratio, match = compare(torch, got, ref, bf16_out)
    print("fp8 decode T=%d %dx%d %s: worst excess / rms %.2e, bf16 rounding match %.4f" % (T, n, k, kind, ratio, match))
    # deterministic: a second call (fresh output) is bitwise identical
    out2 = x0.clone() if kind == "gr_write" else torch.empty_like(out)
    linear.linear_fp8_decode(x, weight, make(out2), work)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16 if out.dtype == torch.bfloat16 else torch.int32),
                       out2.view(torch.int16 if out.dtype == torch.bfloat16 else torch.int32))


def test_activation_pieces_are_exact():
    """scale[t] * (p0 + p1 + p2) reproduces the bf16 activations bit for bit over a 2^23 dynamic range
    inside a row; an all-zero token, a tiny token, and unused token slots left as zero rows."""
    torch = _torch()
    from fngine_b200 import linear
    T, n, k = 6, 256, 1024
    weight = make_weight(torch, 11, n, k, False)
    x = synth.activations(99, T, hidden=k) * np.exp2(np.linspace(-12, 4, k, dtype=np.float32))[None, :]
    x[2] = 0.0
    x[4] *= np.float32(1e-6)
    xb = bf16_tensor(torch, x)
    work = linear.linear_fp8_decode_workspace(weight)
    out = torch.empty(T, n, dtype=torch.float32, device="cuda")
    linear.linear_fp8_decode(xb, weight, linear.store_f32(out), work)
    torch.cuda.synchronize()
    raw = work.cpu().numpy()
    pieces = raw[:48 * k].reshape(3, 16, k)
    scales = raw[48 * k:48 * k + 64].view(np.float32)
    vals = (pieces.astype(np.uint16) << 8).view(np.float16).astype(np.float64)  # E5M2 = the top byte of binary16
    want = xb.float().cpu().numpy().astype(np.float64)
    got = vals.sum(axis=0)[:T] * scales[:T, None].astype(np.float64)
    # exact wherever the value's last mantissa bit is at least 2^-16 of the scaled range (guaranteed for
    # |x| >= 2^-23 of the row maximum); below that the dropped bits are under 2^-30 of the row maximum
    rowmax = np.abs(want).max(axis=1, keepdims=True)
    err = np.abs(got - want)
    assert np.all((err == 0) | (np.abs(want) < rowmax * 2.0 ** -23))
    assert np.all(err <= rowmax * 2.0 ** -30)
    assert (err == 0).mean() > 0.99
    assert not pieces[:, T:].any()
    assert np.all(np.log2(scales[[0, 1, 3, 4, 5]]) == np.round(np.log2(scales[[0, 1, 3, 4, 5]])))  # powers of two


def test_linear_fp8_decode_argument_errors():
    torch = _torch()
    import ctypes

    from fngine_b200 import lib as fblib
    lib = fblib.load()
    buf = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    epi = fblib.LinearEpilogue(fblib.EPI_STORE_BF16, 0, p, None, None)
    e = ctypes.byref(epi)
    assert lib.fb_linear_fp8_decode(p, 17, p, p, 0, 256, 256, e, p, 8 << 20, None) == 1   # more than 16 tokens
    assert lib.fb_linear_fp8_decode(p, 4, p, p, 0, 256, 100, e, p, 8 << 20, None) == 1    # k % 128
    assert lib.fb_linear_fp8_decode(p, 4, p, p, 0, 256, 256, e, p, 1024, None) == 1       # workspace too small
    assert b"workspace" in lib.fb_last_error_string()
    bad = fblib.LinearEpilogue(fblib.EPI_GR_WRITE, 0, p, None, None)
    assert lib.fb_linear_fp8_decode(p, 4, p, p, 0, 256, 256, ctypes.byref(bad), p, 8 << 20, None) == 1  # no inj
    bad = fblib.LinearEpilogue(9, 0, p, None, None)
    assert lib.fb_linear_fp8_decode(p, 4, p, p, 0, 256, 256, ctypes.byref(bad), p, 8 << 20, None) == 1  # bad kind
