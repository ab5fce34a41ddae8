"""GPU parity of the FP8-row dense projection above decode width (tcgen05 E4M3 GEMM) through the C ABI.

Two routes, as in the reference (src/kernels/linear/linear.h:27-37):

* exact (Auto / A16, the default): the bf16 activations are kept. Bar = the reference's own for its A16
  path (tests/kernels/linear/test_linear.cpp:8-11,38-49): against an fp64 product of the E4M3 weight
  values with the UNQUANTIZED bf16 activations, times the row scale, pushed through the epilogue,
  max(|got - ref| - allowance) <= 2e-3 rms(ref) with allowance = 1.001 * 2^-8 |ref| for bf16 outputs
  and 0 for fp32 outputs, and >= 99 % of bf16 outputs equal bf16_rne(ref). The benchmark shape is also
  held to the relative-L2 bar of 2e-2 against the fp32 reference on dequantized weights.
* A8 (on request): one E4M3 code per activation. Bar = the reference's for that path: the same rule
  against an oracle that applies the SAME per-token E4M3 quantization; its distance from the unquantized
  reference is mantissa-bound (about 2.6e-2 relative L2 for N(0,1) inputs, above the 2e-2 the exact
  route meets) and is only reported.
"""
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


def exact_acc(torch, a, weight):
    """fp64 [T][n]: (a . W^T) * scale over the represented values; a fp64 [T][k]."""
    tab = torch.from_numpy(O.e4m3_table().astype(np.float64)).cuda()
    out = torch.empty(a.shape[0], weight.n, dtype=torch.float64, device="cuda")
    for r0 in range(0, weight.n, 2048):  # bounded fp64 temporaries
        w = tab[weight.codes[r0:r0 + 2048].long()]
        out[:, r0:r0 + 2048] = (a @ w.T) * weight.scales[r0:r0 + 2048].double()[None, :]
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
    return worst / rms


def test_fp8_token_quantizer_bit_exact():
    torch = _torch()
    from fngine_b200 import linear
    x = synth.activations(61, 48) * np.linspace(0.01, 30, 48, dtype=np.float32)[:, None]
    x[5] = 0.0  # an all-zero token: scale 0, codes 0
    xb = synth.to_bf16_bits(x)
    codes, scales = linear.fp8_quantize_tokens(torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16))
    want_c, want_s = O.quantize_tokens_e4m3(xb)
    assert np.array_equal(codes.cpu().numpy(), want_c)
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), want_s.view(np.uint32))


def test_two_piece_split_is_bit_exact_and_lossless():
    """The exact route's activation pieces: bit-identical to the host statement, and scale * (hi + lo)
    gives the bf16 activation back - exactly for every element of at least 2^-9 of its row's scaled
    range (|v| >= 0.25 with the row maximum in [128, 256)), to 2^-10 of that range below."""
    torch = _torch()
    from fngine_b200 import linear
    x = synth.activations(62, 40) * np.logspace(-3, 3, 40, dtype=np.float32)[:, None]
    x[7] = 0.0
    x[9, :100] *= 1e-4  # tiny elements beside large ones
    xb = synth.to_bf16_bits(x)
    hi, lo, sc = linear.fp8_split_tokens(torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16))
    w_hi, w_lo, w_sc = O.split_tokens_e4m3x2(xb)
    assert np.array_equal(hi.cpu().numpy(), w_hi) and np.array_equal(lo.cpu().numpy(), w_lo)
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), w_sc.view(np.uint32))
    tab = O.e4m3_table().astype(np.float64)
    v = synth.bf16_bits_to_f32(xb).astype(np.float64)
    s = w_sc.astype(np.float64)[:, None]
    back = s * (tab[w_hi] + tab[w_lo])
    big = np.abs(v) >= 0.25 * s
    assert np.array_equal(back[big], v[big])
    assert np.all(np.abs(back - v) <= s * 2.0 ** -10)
    mx = np.abs(v).max(axis=1)
    live = mx > 0
    assert np.all((mx[live] / w_sc[live] >= 128) & (mx[live] / w_sc[live] < 256)) and np.all(w_sc[~live] == 0)


SHAPES = [(17, 256, 128, False), (64, 320, 640, True), (128, 1280, 2560, False), (300, 2560, 384, True),
          (512, 320, 256, False), (257, 192, 128, True)]


@pytest.mark.parametrize("T,N,K,bf16_scales", SHAPES)
def test_linear_fp8_exact_route(T, N, K, bf16_scales):
    """Auto (= exact activations) against the fp64 oracle on the unquantized bf16 activations."""
    torch = _torch()
    from fngine_b200 import linear
    weight = make_weight(torch, 900 + T, N, K, bf16_scales)
    x = bf16_tensor(torch, synth.activations(77 + T, T, hidden=K))
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    work = linear.linear_fp8_workspace(weight, T)
    linear.linear_fp8(x, weight, out, work)
    torch.cuda.synchronize()
    compare(torch, out, exact_acc(torch, x.double(), weight), True)
    out2 = torch.empty_like(out)
    linear.linear_fp8(x, weight, out2, work, path=linear.L.FP8_PATH_A16)  # A16 names the same route
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))  # and repeated calls are bitwise identical


@pytest.mark.parametrize("T,N,K,bf16_scales", [(1, 256, 128, False), (3, 512, 256, False)] + SHAPES)
def test_linear_fp8_a8_route(T, N, K, bf16_scales):
    """A8 against the fp64 oracle fed the same per-token E4M3 activation quantization."""
    torch = _torch()
    from fngine_b200 import linear
    weight = make_weight(torch, 900 + T, N, K, bf16_scales)
    x = bf16_tensor(torch, synth.activations(77 + T, T, hidden=K))
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    work = linear.linear_fp8_workspace(weight, T)
    linear.linear_fp8(x, weight, out, work, path=linear.L.FP8_PATH_A8)
    torch.cuda.synchronize()
    xq, xs = linear.fp8_quantize_tokens(x)
    tab = torch.from_numpy(O.e4m3_table().astype(np.float64)).cuda()
    ref = exact_acc(torch, tab[xq.long()] * xs.double()[:, None], weight)
    got = out.double()
    rms = ref.pow(2).mean().sqrt()
    excess = ((got - ref).abs() - 2.0 ** -8 * ref.abs()).max()
    assert torch.isfinite(got).all()
    assert float(excess) <= KTOL * float(rms), (float(excess), float(rms))
    out2 = torch.empty_like(out)
    linear.linear_fp8(x, weight, out2, work, path=linear.L.FP8_PATH_A8)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))


@pytest.mark.parametrize("T", [24, 300])
@pytest.mark.parametrize("kind", ["store_f32", "gr_write", "swiglu", "shared_scale"])
def test_linear_fp8_epilogues_above_decode_width(T, kind):
    """The other epilogues of linear.h:64-103 on the GEMM path (the shapes the reference registers:
    gdn.out GrWrite 2560 x 6144, shared gate/up SwiGlu 1280 x 2560, shared down SharedScale 2560 x 640),
    exact route, against the fp64 oracle pushed through the same epilogue."""
    torch = _torch()
    from fngine_b200 import linear
    n, k = {"store_f32": (1024, 2560), "gr_write": (2560, 6144), "swiglu": (1280, 2560),
            "shared_scale": (2560, 640)}[kind]
    weight = make_weight(torch, 1300 + T, n, k, True)
    x = bf16_tensor(torch, synth.activations(88 + T, T, hidden=k))
    acc = exact_acc(torch, x.double(), weight)
    work = linear.linear_fp8_workspace(weight, T)
    g = torch.Generator(device="cuda").manual_seed(T)
    if kind == "store_f32":
        out = torch.full((T, n), float("nan"), dtype=torch.float32, device="cuda")
        epi, ref, bf = linear.store_f32(out), acc, False
    elif kind == "gr_write":
        inj = torch.randn(T, 4, device="cuda", generator=g)
        x0 = torch.randn(T, 4, n, device="cuda", generator=g)
        out = x0.clone()
        epi, bf = linear.gr_write(out, inj), False
        ref = x0.double() + inj.double()[:, :, None] * acc[:, None, :]
    elif kind == "swiglu":
        out = torch.full((T, n // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
        gg, uu = acc[:, :n // 2], acc[:, n // 2:]
        epi, ref, bf = linear.swiglu(out), gg / (1.0 + torch.exp(-gg)) * uu, True
    else:
        logit = torch.randn(T, 513, device="cuda", generator=g)
        out = torch.full((T, n), float("nan"), dtype=torch.float32, device="cuda")
        epi, bf = linear.shared_scale(out, logit[:, 512:], 513), False
        ref = acc / (1.0 + torch.exp(-logit[:, 512].double()))[:, None]
    linear.linear_fp8(x, weight, epi, work)
    torch.cuda.synchronize()
    compare(torch, out, ref, bf)


def test_linear_fp8_on_a_weight_packed_by_the_reference_rule():
    """A bf16 weight matrix packed by the reference's FP8-row rule (tools/fp8row.py quantize_rows, restated in
    the oracle and pinned to the tool's own outputs: bf16 row scales, clamped round-to-nearest-even codes),
    then both routes against the fp64 product over the packed values; and the packing itself loses what
    E4M3 loses (about 3 % per element, 2.5e-2 relative L2 of the output), not more."""
    torch = _torch()
    from fngine_b200 import linear
    T, N, K = 96, 512, 1024
    wb = synth.to_bf16_bits((synth.normal(7001, N * K) * 0.02).astype(np.float32).reshape(N, K))
    wb[3] = 0  # an all-zero row: scale 0, codes 0
    codes, scales = O.quantize_fp8_rows(wb)
    weight = linear.Fp8RowWeight(torch.from_numpy(codes).cuda(),
                                 torch.from_numpy(scales.view(np.int16)).cuda().view(torch.bfloat16))
    x = bf16_tensor(torch, synth.activations(7002, T, hidden=K))
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    work = linear.linear_fp8_workspace(weight, T)
    linear.linear_fp8(x, weight, out, work)
    torch.cuda.synchronize()
    ref = exact_acc(torch, x.double(), weight)
    compare(torch, out, ref, True)
    assert float(out[:, 3].abs().max()) == 0.0
    dense = x.double() @ torch.from_numpy(synth.bf16_bits_to_f32(wb).astype(np.float64)).cuda().T
    assert float((ref - dense).norm() / dense.norm()) <= 4e-2


def test_linear_fp8_benchmark_shape():
    """bf16 [4096 x 2560] x E4M3 [9216 x 2560] with fp32 row scales -> bf16 [4096 x 9216], both routes.
    The stated bar (2e-2 relative L2 against an fp32 reference on dequantized weights and the given bf16
    activations) is asserted for the exact route, which is what Auto selects; for A8 the same figure is
    printed (mantissa-bound) and the GEMM is held to its own-quantization reference."""
    torch = _torch()
    from fngine_b200 import linear
    T, N, K = 4096, 9216, 2560
    weight = make_weight(torch, 4, N, K, False)
    wc, ws = weight.codes, weight.scales
    x = bf16_tensor(torch, synth.activations(44, T, hidden=K))
    out = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
    work = linear.linear_fp8_workspace(weight, T)
    tab = torch.from_numpy(O.e4m3_table()).cuda()
    wd = tab[wc.long()] * ws[:, None]                       # dequantized weights, fp32
    ref_u = x.float() @ wd.T                                # the given (unquantized) activations
    linear.linear_fp8(x, weight, out, work)
    torch.cuda.synchronize()
    rel_exact = float((out.float() - ref_u).norm() / ref_u.norm())
    linear.linear_fp8(x, weight, out, work, path=linear.L.FP8_PATH_A8)
    torch.cuda.synchronize()
    xq, xs = linear.fp8_quantize_tokens(x)
    ref_q = (tab[xq.long()] * xs[:, None]) @ wd.T           # same activation quantization
    got = out.float()
    rel_q = float((got - ref_q).norm() / ref_q.norm())
    rel_u = float((got - ref_u).norm() / ref_u.norm())
    print("fp8 gemm 4096x9216x2560: exact route rel L2 vs fp32 reference %.2e (bar 2e-2); A8 route %.2e vs its "
          "own-quantization reference, %.2e vs the fp32 reference" % (rel_exact, rel_q, rel_u))
    assert rel_exact <= 2e-2 and rel_exact <= 4e-3   # stated bar; bf16 output rounding alone is about 1.7e-3
    assert rel_q <= 4e-3
    assert rel_u <= 4e-2                              # A8's documented activation noise, not the stated bar


def test_linear_fp8_routes_decode_width_to_the_streaming_projection():
    """T <= 16 on the exact routes runs the decode-width projection: same bits as fb_linear_fp8_decode."""
    torch = _torch()
    from fngine_b200 import linear
    weight = make_weight(torch, 77, 1024, 512, True)
    x = bf16_tensor(torch, synth.activations(5, 9, hidden=512))
    a = torch.empty(9, 1024, dtype=torch.bfloat16, device="cuda")
    b = torch.empty_like(a)
    work = linear.linear_fp8_workspace(weight, 64)
    linear.linear_fp8(x, weight, a, work)
    linear.linear_fp8_decode(x, weight, linear.store_bf16(b), work)
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_linear_fp8_argument_errors():
    torch = _torch()
    import ctypes
    from fngine_b200 import lib as fblib
    lib = fblib.load()
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    epi = fblib.LinearEpilogue(fblib.EPI_STORE_BF16, 0, p, None, None)
    e = ctypes.byref(epi)
    assert lib.fb_linear_fp8(p, 32, p, p, 0, 100, 256, e, p, 1 << 20, None, 0) == 1   # n % 64
    assert lib.fb_linear_fp8(p, 32, p, p, 0, 128, 100, e, p, 1 << 20, None, 0) == 1   # k % 128
    assert lib.fb_linear_fp8(p, 32, p, p, 0, 128, 256, e, p, 16, None, 0) == 1        # workspace too small
    assert b"workspace" in lib.fb_last_error_string()
    assert lib.fb_linear_fp8(p, 32, p, p, 0, 128, 256, e, p, 1 << 20, None, 7) == 1   # unknown path
    sw = fblib.LinearEpilogue(fblib.EPI_SWIGLU, 0, p, None, None)
    assert lib.fb_linear_fp8(p, 32, p, p, 0, 192, 256, ctypes.byref(sw), p, 1 << 20, None, 0) == 1  # SwiGlu n % 128
    sh = fblib.LinearEpilogue(fblib.EPI_SHARED_SCALE, 513, p, None, None)
    assert lib.fb_linear_fp8(p, 32, p, p, 0, 128, 256, ctypes.byref(sh), p, 1 << 20, None, 0) == 1  # no gate logit
