"""TEST INFRASTRUCTURE ONLY: ctypes access to the CPU oracle.

Two libraries sit behind this module:
  * `port`  -- oracle/fb_oracle.c, this repository's scalar-C restatement of the reference's CPU
               expert path (always available; built by `build_port()`).
  * `ref`   -- oracle/_ref/libfngine_ref.so, the reference's own sources compiled in place by
               oracle/build_ref.py (available where that build ran and the host CPU has the
               AVX-512 subsets it needs).
Only tests/, the smoke check and the benchmark's CPU-baseline legs may import this module; the
shipped library never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
IQ4_NL, IQ3_S = 20, 21
IQ3_XXS, IQ2_S, IQ4_XS, Q2_0 = 18, 22, 23, 42  # the other expert formats of the reference (ggml type ids)
ACT_Q8_K, ACT_Q8_0 = 0, 1
BLOCK = {IQ3_S: (256, 110), IQ4_NL: (32, 18), IQ3_XXS: (256, 98), IQ2_S: (256, 82), IQ4_XS: (256, 136), Q2_0: (64, 18)}
ACT_OF = {IQ3_S: ACT_Q8_K, IQ4_NL: ACT_Q8_0, IQ3_XXS: ACT_Q8_K, IQ2_S: ACT_Q8_K, IQ4_XS: ACT_Q8_K, Q2_0: ACT_Q8_0}
ACT_BLOCK = {ACT_Q8_K: (256, 292), ACT_Q8_0: (32, 34)}

_port = None
_ref = None


def build_port(force=False):
    so = os.path.join(HERE, "_build", "libfb_oracle.so")
    src = os.path.join(HERE, "fb_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < max(
            os.path.getmtime(src), os.path.getmtime(os.path.join(HERE, "fb_oracle_codebooks.h"))):
        os.makedirs(os.path.dirname(so), exist_ok=True)
        subprocess.check_call(["gcc", "-O2", "-std=c11", "-fno-fast-math", "-ffp-contract=off", "-shared",
                               "-fPIC", src, "-o", so, "-lm", "-lpthread"])
    return so


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def port():
    global _port
    if _port is None:
        lib = C.CDLL(build_port())
        lib.fbo_fp16_to_fp32.restype = C.c_float
        lib.fbo_fp16_to_fp32.argtypes = [C.c_uint16]
        lib.fbo_fp32_to_fp16.restype = C.c_uint16
        lib.fbo_fp32_to_fp16.argtypes = [C.c_float]
        lib.fbo_dot.restype = C.c_float
        lib.fbo_dot.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        lib.fbo_e4m3_to_float.restype = C.c_float
        lib.fbo_e4m3_to_float.argtypes = [C.c_uint8]
        lib.fbo_e4m3_satfinite.restype = C.c_uint8
        lib.fbo_e4m3_satfinite.argtypes = [C.c_float]
        lib.fbo_quantize_token_e4m3.restype = C.c_float
        lib.fbo_quantize_token_e4m3.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
        lib.fbo_quantize_fp8_rows.restype = None
        lib.fbo_quantize_fp8_rows.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
        lib.fbo_split_token_e4m3x2.restype = C.c_float
        lib.fbo_split_token_e4m3x2.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
        lib.fbo_row_bytes.restype = C.c_int64
        lib.fbo_dequant_rows.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]
        lib.fbo_dequant_rows_bf16.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]
        lib.fbo_quantize_act.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
        lib.fbo_silu_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        lib.fbo_expert_ffn.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        lib.fbo_expert_ffn_bf16.argtypes = lib.fbo_expert_ffn.argtypes
        lib.fbo_down_bf16.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        lib.fbo_topk.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        lib.fbo_moe_layer.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_void_p,
                                      C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        _port = lib
    return _port


def host_cpu_flags():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def ref_available():
    so = os.path.join(HERE, "_ref", "libfngine_ref.so")
    req = os.path.join(HERE, "_ref", "REQUIRED_CPU_FLAGS")
    if not (os.path.exists(so) and os.path.exists(req)):
        return False
    need = set(open(req).read().split())
    return need <= host_cpu_flags()


def ref():
    """The reference's own CPU code, or None where it was not built / the CPU lacks AVX-512."""
    global _ref
    if _ref is None:
        if not ref_available():
            return None
        lib = C.CDLL(os.path.join(HERE, "_ref", "libfngine_ref.so"))
        lib.ref_vec_dot_iq3_s_q8_K.restype = C.c_float
        lib.ref_vec_dot_iq3_s_q8_K.argtypes = [C.c_int, C.c_void_p, C.c_void_p]
        lib.ref_vec_dot_iq4_nl_q8_0.restype = C.c_float
        lib.ref_vec_dot_iq4_nl_q8_0.argtypes = [C.c_int, C.c_void_p, C.c_void_p]
        for n in ("ref_decoded_row_bytes", "ref_packed_act_bytes", "ref_weight_row_bytes"):
            getattr(lib, n).restype = C.c_int64
            getattr(lib, n).argtypes = [C.c_int, C.c_int]
        lib.ref_dequant_iq3_s.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        lib.ref_dequant_iq4_nl.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        for n in ("ref_quantize_q8_K", "ref_quantize_q8_0", "ref_quantize_q8_K_avx", "ref_quantize_q8_0_avx",
                  "ref_quantize_q8_K_bf16", "ref_quantize_q8_0_bf16"):
            getattr(lib, n).argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        lib.ref_decode_rows.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]
        lib.ref_quantize_pack_f32.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_void_p]
        lib.ref_quantize_pack_bf16.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_void_p]
        lib.ref_gemm_decoded.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                         C.c_int64]
        lib.ref_decode_rows_bf16.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]
        lib.ref_gemm_bf16.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int64]
        lib.ref_silu_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        lib.ref_expert_ffn.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        lib.ref_moe_layer.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_void_p,
                                      C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        lib.ref_expert_ffn_bf16.argtypes = lib.ref_expert_ffn.argtypes
        if hasattr(lib, "ref_pool_decode_step"):  # built where the CUDA headers (bf16 type) were present
            lib.ref_pool_decode_step.restype = C.c_int
            lib.ref_pool_decode_step.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_longlong, C.c_int, C.c_longlong,
                                                 C.c_longlong, C.c_longlong, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                                 C.c_int, C.c_void_p, C.c_char_p, C.c_int]
        _ref = lib
    return _ref


# ------------------------------------------------------------------------- numpy-facing helpers
def row_bytes(fmt, k):
    be, bb = BLOCK[fmt]
    assert k % be == 0
    return k // be * bb


def act_row_bytes(act, k):
    be, bb = ACT_BLOCK[act]
    assert k % be == 0
    return k // be * bb


def dequant_rows(fmt, rows, nrows, k, lib=None):
    """rows: uint8 array holding nrows back-to-back rows. Returns float32 [nrows][k]."""
    rows = np.ascontiguousarray(rows, dtype=np.uint8)
    y = np.empty((nrows, k), dtype=np.float32)
    if lib is None or lib is port():
        port().fbo_dequant_rows(fmt, _ptr(rows), row_bytes(fmt, k), nrows, k, _ptr(y))
    else:
        if not lib.ref_dequant(fmt, _ptr(rows), _ptr(y), nrows * k):  # rows are contiguous blocks
            raise ValueError("the reference build does not know format %d" % fmt)
    return y


def dequant_rows_bf16(fmt, rows, nrows, k, lib=None):
    rows = np.ascontiguousarray(rows, dtype=np.uint8)
    y = np.empty((nrows, k), dtype=np.uint16)
    if lib is None or lib is port():
        port().fbo_dequant_rows_bf16(fmt, _ptr(rows), row_bytes(fmt, k), nrows, k, _ptr(y))
    else:
        lib.ref_decode_rows_bf16(fmt, _ptr(rows), row_bytes(fmt, k), nrows, k, _ptr(y))
    return y


def quantize_act(act, x, lib=None, variant="ref"):
    """x: float32 [..., k] -> uint8 [..., act_row_bytes]. variant (ref lib only): 'ref' = ggml
    reference quantizer, 'avx' = the reference's AVX-512 quantizer."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    k = x.shape[-1]
    out = np.zeros(x.shape[:-1] + (act_row_bytes(act, k),), dtype=np.uint8)
    n = x.size
    if lib is None or lib is port():
        port().fbo_quantize_act(act, _ptr(x), _ptr(out), n)
    else:
        name = "ref_quantize_q8_%s%s" % ("K" if act == ACT_Q8_K else "0", "_avx" if variant == "avx" else "")
        getattr(lib, name)(_ptr(x), _ptr(out), n)
    return out


def silu_mul(g, u, lib=None):
    g = np.ascontiguousarray(g, dtype=np.float32)
    u = np.ascontiguousarray(u, dtype=np.float32)
    h = np.empty_like(g)
    if lib is None or lib is port():
        port().fbo_silu_mul(_ptr(g), _ptr(u), _ptr(h), g.size)
    else:
        lib.ref_silu_mul(_ptr(g), _ptr(u), _ptr(h), g.size)
    return h


def expert_ffn(fmt_gu, fmt_down, hidden, inter, blob, x, lib=None):
    """blob: uint8 gate|up|down. x float32 [T][hidden]. Returns (h [T][inter], y [T][hidden]),
    unweighted, decode numerics (int8 activations)."""
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, hidden)
    T = x.shape[0]
    gb = inter * row_bytes(fmt_gu, hidden)
    h = np.empty((T, inter), dtype=np.float32)
    y = np.empty((T, hidden), dtype=np.float32)
    base = blob.ctypes.data
    fn = port().fbo_expert_ffn if (lib is None or lib is port()) else lib.ref_expert_ffn
    fn(fmt_gu, fmt_down, hidden, inter, base, base + gb, base + 2 * gb, _ptr(x), T, _ptr(h), _ptr(y))
    return h, y


def expert_ffn_bf16(fmt_gu, fmt_down, hidden, inter, blob, x_bf16, lib=None):
    """Prefill numerics (bf16 weights/activations). x_bf16: uint16 [T][hidden] raw bits.
    Returns (h uint16 [T][inter], y float32 [T][hidden])."""
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16).reshape(-1, hidden)
    T = x.shape[0]
    gb = inter * row_bytes(fmt_gu, hidden)
    h = np.empty((T, inter), dtype=np.uint16)
    y = np.empty((T, hidden), dtype=np.float32)
    base = blob.ctypes.data
    fn = port().fbo_expert_ffn_bf16 if (lib is None or lib is port()) else lib.ref_expert_ffn_bf16
    fn(fmt_gu, fmt_down, hidden, inter, base, base + gb, base + 2 * gb, _ptr(x), T, _ptr(h), _ptr(y))
    return h, y


def down_bf16(fmt_down, hidden, inter, down_bytes, h_bits):
    """Prefill-numerics down projection of given bf16 h rows (uint16 [T][inter]) -> float32 [T][hidden]."""
    down_bytes = np.ascontiguousarray(down_bytes, dtype=np.uint8)
    h = np.ascontiguousarray(h_bits, dtype=np.uint16).reshape(-1, inter)
    y = np.empty((h.shape[0], hidden), dtype=np.float32)
    port().fbo_down_bf16(fmt_down, hidden, inter, _ptr(down_bytes), _ptr(h), h.shape[0], _ptr(y))
    return y


def topk(logits, k=10):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    T, n = logits.shape
    ids = np.empty((T, k), dtype=np.int32)
    w = np.empty((T, k), dtype=np.float32)
    for t in range(T):
        port().fbo_topk(_ptr(logits[t]), n, k, _ptr(ids[t]), _ptr(w[t]))
    return ids, w


def moe_layer(fmt_gu, fmt_down, hidden, inter, blobs, blob_stride, x, ids, w, threads=1, lib=None):
    """y[t] = sum_k w[t,k] * ffn_{ids[t,k]}(x[t]), experts of a token added in ascending id."""
    blobs = np.ascontiguousarray(blobs, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, hidden)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    T, k = ids.shape
    y = np.empty((T, hidden), dtype=np.float32)
    fn = port().fbo_moe_layer if (lib is None or lib is port()) else lib.ref_moe_layer
    fn(fmt_gu, fmt_down, hidden, inter, _ptr(blobs), blob_stride, _ptr(x), T, k, _ptr(ids), _ptr(w), _ptr(y),
       threads)
    return y


def pool_available():
    """True where the reference's own cpu::ExpertPool was built into oracle/_ref and can run here."""
    return ref() is not None and hasattr(ref(), "ref_pool_decode_step")


def pool_decode_step(fmt_gu, fmt_down, blobs, blob_stride, x_bf16, ids, w, workers=4):
    """One decode step of one layer through the reference's production CPU tier, cpu::ExpertPool
    (src/cpu/expert_pool.h:76-102), driven through its host exchange as the reference's harness does
    (tests/cpu/pool_bench.h:42-140). The pool's shape is fixed: hidden 2560, intermediate 640, a Q8_0-family
    down format. blobs: experts `blob_stride` bytes apart (gate | up | down back to back); x_bf16: uint16
    [T][2560], T <= 16; ids int32 [T][10] index into blobs; w float32 [T][10]. Returns y float32 [T][2560]."""
    lib = ref()
    blobs = np.ascontiguousarray(blobs, dtype=np.uint8)
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16).reshape(-1, 2560)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    T = x.shape[0]
    assert ids.shape == (T, 10) and w.shape == (T, 10)
    gate_bytes = 640 * row_bytes(fmt_gu, 2560)
    y = np.empty((T, 2560), dtype=np.float32)
    err = C.create_string_buffer(512)
    rc = lib.ref_pool_decode_step(fmt_gu, fmt_down, _ptr(blobs), blob_stride, blobs.size // blob_stride, 0, gate_bytes,
                                  2 * gate_bytes, _ptr(x), T, _ptr(ids), _ptr(w), workers, _ptr(y), err, 512)
    if rc:
        raise RuntimeError("cpu::ExpertPool step failed: " + err.value.decode("utf-8", "replace"))
    return y


_E4M3 = None


def e4m3_table():
    global _E4M3
    if _E4M3 is None:
        _E4M3 = np.array([port().fbo_e4m3_to_float(c) for c in range(256)], dtype=np.float32)
    return _E4M3


def quantize_tokens_e4m3(x_bf16):
    """uint16 bf16 bits [T][K] -> (codes uint8 [T][K], scales float32 [T])."""
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    T, K = x.shape
    codes = np.empty((T, K), dtype=np.uint8)
    scales = np.empty(T, dtype=np.float32)
    for t in range(T):
        scales[t] = port().fbo_quantize_token_e4m3(_ptr(x[t]), K, _ptr(codes[t]))
    return codes, scales


def quantize_fp8_rows(w_bf16):
    """The FP8-row pack rule (tools/fp8row.py:21-44 of the reference): uint16 bf16 bits [n][k] ->
    (codes uint8 [n][k], scales uint16 bf16 bits [n])."""
    w = np.ascontiguousarray(w_bf16, dtype=np.uint16)
    n, k = w.shape
    codes = np.empty((n, k), dtype=np.uint8)
    scales = np.empty(n, dtype=np.uint16)
    port().fbo_quantize_fp8_rows(_ptr(w), n, k, _ptr(codes), _ptr(scales))
    return codes, scales


def split_tokens_e4m3x2(x_bf16):
    """uint16 bf16 bits [T][K] -> (hi uint8 [T][K], lo uint8 [T][K], scales float32 [T]): the two-piece
    statement of the exact route (scale a power of two, hi = rne_e4m3, lo = rne_e4m3 of the remainder)."""
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    T, K = x.shape
    hi = np.empty((T, K), dtype=np.uint8)
    lo = np.empty((T, K), dtype=np.uint8)
    scales = np.empty(T, dtype=np.float32)
    for t in range(T):
        scales[t] = port().fbo_split_token_e4m3x2(_ptr(x[t]), K, _ptr(hi[t]), _ptr(lo[t]))
    return hi, lo, scales


def linear_fp8_a16(x_bf16, codes, scales, kind="store", gate_logit=None):
    """The exact-activation FP8-row projection as the reference's own test oracle states it
    (tests/kernels/linear/test_linear.cpp:196-243): fp64 dot products of the E4M3 weight values with
    the bf16 activations, times the row scale, then the epilogue in fp64.
    x_bf16: uint16 bf16 bits [T][K]; codes uint8 [N][K]; scales float [N] (already the represented
    values: widen bf16 scales first). kind: "store" -> acc [T][N]; "swiglu" -> silu(acc[:, :N/2]) *
    acc[:, N/2:]; "shared_scale" -> sigmoid(gate_logit[t]) * acc."""
    x = (np.ascontiguousarray(x_bf16, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)
    w = e4m3_table().astype(np.float64)[np.asarray(codes, dtype=np.uint8)]
    acc = (x.astype(np.float64) @ w.T) * np.asarray(scales, dtype=np.float64)[None, :]
    if kind == "store":
        return acc
    if kind == "swiglu":
        h = acc.shape[1] // 2
        g, u = acc[:, :h], acc[:, h:]
        return g / (1.0 + np.exp(-g)) * u
    if kind == "shared_scale":
        return acc / (1.0 + np.exp(-np.asarray(gate_logit, dtype=np.float64)))[:, None]
    raise ValueError(kind)
