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


def linear_fp8(x, weight, out, workspace):
    """out[t][n] = bf16((x[t] . W[n]) * scale[n]); x bf16 [T][k], out bf16 [T][n]."""
    assert x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and x.is_contiguous() and out.is_contiguous()
    dt = L.DT_BF16 if weight.scales.dtype == torch.bfloat16 else L.DT_F32
    L.check(L.load().fb_linear_fp8(x.data_ptr(), x.shape[0], weight.codes.data_ptr(), weight.scales.data_ptr(), dt,
                                   weight.n, weight.k, out.data_ptr(), workspace.data_ptr(), workspace.numel(),
                                   torch.cuda.current_stream().cuda_stream), "linear_fp8")


def fp8_quantize_tokens(x):
    """Per-token E4M3 codes and fp32 scales of bf16 x [T][k]."""
    T, k = x.shape
    codes = torch.empty(T, k, dtype=torch.uint8, device=x.device)
    scales = torch.empty(T, dtype=torch.float32, device=x.device)
    L.check(L.load().fb_fp8_quantize_tokens(x.data_ptr(), T, k, codes.data_ptr(), scales.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream), "fp8_quantize_tokens")
    return codes, scales
