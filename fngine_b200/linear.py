"""Host-side mirror of the reference's FP8-row projection (linear_fp8, src/kernels/linear/linear.h
of the reference): E4M3 weight codes with one scale per row, bf16 activations, bf16 output.
Every call goes through the C ABI; torch only owns the device buffers."""
import torch

from . import lib as L


class Fp8RowWeight:
    """Fp8RowWeight (linear.h:57-62 of the reference): codes uint8 [n][k], scales fp32 or bf16 [n]."""

    def __init__(self, codes, scales):
        assert codes.is_cuda and codes.dtype == torch.uint8 and codes.dim() == 2 and codes.is_contiguous()
        assert scales.is_cuda and scales.dtype in (torch.float32, torch.bfloat16) and scales.numel() == codes.shape[0]
        self.codes, self.scales = codes, scales.contiguous()
        self.n, self.k = codes.shape


def linear_fp8_workspace(weight, max_tokens, device="cuda"):
    n = L.load().fb_linear_fp8_workspace_bytes(weight.n, weight.k, max_tokens)
    buf = torch.empty(n + 256, dtype=torch.uint8, device=device)
    off = (-buf.data_ptr()) % 256
    return buf[off:off + n]


def linear_fp8(x, weight, out, workspace, path=L.FP8_PATH_AUTO):
    """linear_fp8 (linear.h:137-139 of the reference): x bf16 [T][k]; `out` is an epilogue (store_bf16,
    store_f32, gr_write, swiglu, shared_scale) or, as a shorthand for store_bf16, a bf16 [T][n] tensor.
    path: FP8_PATH_AUTO / FP8_PATH_A16 = exact activations (the reference's default), FP8_PATH_A8 =
    one E4M3 code per activation (faster, 1-4 % rms noise)."""
    import ctypes
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[1] == weight.k
    epi = store_bf16(out) if isinstance(out, torch.Tensor) else out
    dt = L.DT_BF16 if weight.scales.dtype == torch.bfloat16 else L.DT_F32
    L.check(L.load().fb_linear_fp8(x.data_ptr(), x.shape[0], weight.codes.data_ptr(), weight.scales.data_ptr(), dt,
                                   weight.n, weight.k, ctypes.byref(epi), workspace.data_ptr(), workspace.numel(),
                                   torch.cuda.current_stream().cuda_stream, path), "linear_fp8")


def _epilogue(kind, gate_stride, out, inj=None, gate_logit=None):
    """fb_linear_epilogue that also keeps its tensors alive: the struct holds raw device pointers."""
    e = L.LinearEpilogue(kind, gate_stride, out.data_ptr(), None if inj is None else inj.data_ptr(),
                         None if gate_logit is None else gate_logit.data_ptr())
    e._keep = (out, inj, gate_logit)
    return e


def store_bf16(out):
    """linear_store_bf16 (linear.h:88-90 of the reference): out bf16 [T][n]."""
    assert out.dtype == torch.bfloat16 and out.is_contiguous()
    return _epilogue(L.EPI_STORE_BF16, 0, out)


def store_f32(out):
    """linear_store_f32 (linear.h:91): out fp32 [T][n]."""
    assert out.dtype == torch.float32 and out.is_contiguous()
    return _epilogue(L.EPI_STORE_F32, 0, out)


def gr_write(x_streams, inj):
    """linear_gr_write (linear.h:92-94): X fp32 [T][4][n] += inj fp32 [T][4] * acc, in place."""
    assert x_streams.dtype == torch.float32 and inj.dtype == torch.float32
    assert x_streams.is_contiguous() and inj.is_contiguous()
    return _epilogue(L.EPI_GR_WRITE, 0, x_streams, inj=inj)


def swiglu(h):
    """linear_swiglu (linear.h:95): h bf16 [T][n/2] = silu(acc[j]) * acc[n/2 + j]."""
    assert h.dtype == torch.bfloat16 and h.is_contiguous()
    return _epilogue(L.EPI_SWIGLU, 0, h)


def shared_scale(y, gate_logit, gate_stride):
    """linear_shared_scale (linear.h:96-99): y fp32 [T][n] = sigmoid(gate_logit[t * gate_stride]) * acc."""
    assert y.dtype == torch.float32 and gate_logit.dtype == torch.float32 and y.is_contiguous()
    return _epilogue(L.EPI_SHARED_SCALE, gate_stride, y, gate_logit=gate_logit)


def linear_fp8_decode_workspace(weight, device="cuda"):
    n = L.load().fb_linear_fp8_decode_workspace_bytes(weight.n, weight.k)
    buf = torch.empty(n + 256, dtype=torch.uint8, device=device)
    off = (-buf.data_ptr()) % 256
    return buf[off:off + n]


def linear_fp8_decode(x, weight, epilogue, workspace):
    """linear_fp8 for T <= 16 on the exact-activation path (linear.h:137-139 with Fp8LinearPath::A16):
    x bf16 [T][k]; the output is whatever `epilogue` (store_bf16, store_f32, gr_write, swiglu,
    shared_scale) names."""
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[1] == weight.k
    dt = L.DT_BF16 if weight.scales.dtype == torch.bfloat16 else L.DT_F32
    import ctypes
    L.check(L.load().fb_linear_fp8_decode(x.data_ptr(), x.shape[0], weight.codes.data_ptr(), weight.scales.data_ptr(),
                                          dt, weight.n, weight.k, ctypes.byref(epilogue), workspace.data_ptr(),
                                          workspace.numel(), torch.cuda.current_stream().cuda_stream),
            "linear_fp8_decode")


def fp8_quantize_tokens(x):
    """Per-token E4M3 codes and fp32 scales of bf16 x [T][k]."""
    T, k = x.shape
    codes = torch.empty(T, k, dtype=torch.uint8, device=x.device)
    scales = torch.empty(T, dtype=torch.float32, device=x.device)
    L.check(L.load().fb_fp8_quantize_tokens(x.data_ptr(), T, k, codes.data_ptr(), scales.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream), "fp8_quantize_tokens")
    return codes, scales


def fp8_split_tokens(x):
    """The two E4M3 pieces and the power-of-two scale of the exact route: x == scale * (hi + lo)."""
    T, k = x.shape
    hi = torch.empty(T, k, dtype=torch.uint8, device=x.device)
    lo = torch.empty(T, k, dtype=torch.uint8, device=x.device)
    scales = torch.empty(T, dtype=torch.float32, device=x.device)
    L.check(L.load().fb_fp8_split_tokens(x.data_ptr(), T, k, hi.data_ptr(), lo.data_ptr(), scales.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream), "fp8_split_tokens")
    return hi, lo, scales
