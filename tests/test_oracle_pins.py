"""Pins the CPU oracle (oracle/fb_oracle.c) to the reference.

Two anchors: (1) committed vectors in tests/golden/reference_vectors.npz, produced by the
reference's own code (tests/golden/make_golden.py); (2) where oracle/_ref is present and the host
CPU can run it, a direct comparison with the reference's functions on more inputs.
Bit-exact for weights, int8 activations, SwiGLU and expert outputs of the decode numerics; the
prefill (bf16) family is compared within 1e-5 relative (fp32 summation order differs).
"""
import os
import sys

import numpy as np
import pytest

from fngine_b200 import synth
from oracle import oracle as O
import patterns

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))
IQ3_S, IQ4_NL = 21, 20


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("fmt,seed,name", [(IQ3_S, 11, "iq3s"), (IQ4_NL, 12, "iq4nl")])
def test_dequant_matches_golden(fmt, seed, name):
    nb = 2 * 2560 // synth.BLOCK_ELEMS[fmt]
    rows = synth.fill_blocks(fmt, nb, 0, seed)
    assert np.array_equal(bits(O.dequant_rows(fmt, rows, 2, 2560)), bits(GOLD["dequant_" + name]))
    assert np.array_equal(O.dequant_rows_bf16(fmt, rows, 2, 2560), GOLD["dequant_bf16_" + name])


def test_other_formats_match_golden():
    """IQ3_XXS, IQ2_S, IQ4_XS and Q2_0 (the reference's other expert formats): dequantized rows against the
    vendored ggml dequantizers, single-expert outputs against the AVX-512 expert tier, bit for bit."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    import make_golden_formats as G
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors_formats.npz"))
    for fmt, seed, name in G.DEQUANT:
        rows = synth.fill_blocks(fmt, 2 * 2560 // synth.BLOCK_ELEMS[fmt], 0, seed)
        assert np.array_equal(bits(O.dequant_rows(fmt, rows, 2, 2560)), bits(gold["dequant_" + name])), name
    xs = synth.activations(32, 2)
    for fg, fd, inter, name in G.FFN:
        h, y = O.expert_ffn(fg, fd, 2560, inter, synth.expert_blob(fg, fd, inter, 43, 6), xs)
        assert np.array_equal(bits(h), bits(gold[name + "_h"])) and np.array_equal(bits(y), bits(gold[name + "_y"])), name


def test_quantizers_match_golden():
    x = patterns.all_inputs()
    assert np.array_equal(O.quantize_act(O.ACT_Q8_K, x), GOLD["q8k"])
    assert np.array_equal(O.quantize_act(O.ACT_Q8_0, x), GOLD["q80"])


def test_silu_matches_golden():
    g = (synth.normal(21, 4096) * 6).astype(np.float32)
    u = synth.normal(22, 4096).astype(np.float32)
    g[:8] = [0.0, -0.0, 100.0, -100.0, 88.0, -88.0, 1e-20, -1e-20]
    assert np.array_equal(bits(O.silu_mul(g, u)), bits(GOLD["silu"]))


@pytest.mark.parametrize("fg,fd,inter,name", [(IQ3_S, IQ3_S, 512, "ffn_iq3s_512"),
                                              (IQ4_NL, IQ4_NL, 512, "ffn_iq4nl_512"),
                                              (IQ3_S, IQ4_NL, 640, "ffn_iq3s_iq4nl_640")])
def test_expert_ffn_matches_golden(fg, fd, inter, name):
    xs = synth.activations(31, 3)
    blob = synth.expert_blob(fg, fd, inter, 41, 5)
    h, y = O.expert_ffn(fg, fd, 2560, inter, blob, xs)
    assert np.array_equal(bits(h), bits(GOLD[name + "_h"]))
    assert np.array_equal(bits(y), bits(GOLD[name + "_y"]))


def test_expert_ffn_bf16_matches_golden():
    xs = synth.activations(31, 3)
    xb = synth.to_bf16_bits(xs[:2])
    blob = synth.expert_blob(IQ3_S, IQ3_S, 512, 41, 5)
    h, y = O.expert_ffn_bf16(IQ3_S, IQ3_S, 2560, 512, blob, xb)
    gh = synth.bf16_bits_to_f32(GOLD["ffn_bf16_iq3s_512_h"])
    hh = synth.bf16_bits_to_f32(h)
    # h is a bf16 rounding of an fp32 sum taken in a different order: allow one bf16 step
    assert np.max(np.abs(hh - gh) / (np.abs(gh) + 1e-3)) < 2 ** -7
    gy = GOLD["ffn_bf16_iq3s_512_y"]
    assert np.linalg.norm(y - gy) / np.linalg.norm(gy) < 2e-3


def test_fp16_round_trip_all_codes():
    p = O.port()
    for code in range(0, 0x7C00):  # every finite positive half
        f = p.fbo_fp16_to_fp32(code)
        assert p.fbo_fp32_to_fp16(f) == code
        assert np.float32(f) == np.array([code], dtype=np.uint16).view(np.float16)[0].astype(np.float32)
        if code > 2000:
            break


def test_fp16_matches_numpy():
    p = O.port()
    xs = np.concatenate([synth.normal(3, 4000) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 300.0, 7e4)]).astype(np.float32)
    want = xs.astype(np.float16).view(np.uint16)
    got = np.array([p.fbo_fp32_to_fp16(float(v)) for v in xs], dtype=np.uint16)
    assert np.array_equal(got, want)
    codes = np.arange(65536, dtype=np.uint16)
    finite = ((codes >> 10) & 0x1F) != 31
    back = np.array([p.fbo_fp16_to_fp32(int(c)) for c in codes[finite]], dtype=np.float32)
    assert np.array_equal(back.view(np.uint32), codes[finite].view(np.float16).astype(np.float32).view(np.uint32))


def test_e4m3_tables():
    # Known values of the format (tests/common/test_util.h:105-112 of the reference): 0x7E = 448,
    # 0x38 = 1.0, 0x01 = 2^-9, 0x7F = NaN.
    t = O.e4m3_table()
    assert t[0x7E] == 448.0 and t[0x38] == 1.0 and t[0x01] == 2.0 ** -9 and np.isnan(t[0x7F])
    assert t[0xFE] == -448.0
    p = O.port()
    assert p.fbo_e4m3_satfinite(1e9) == 0x7E and p.fbo_e4m3_satfinite(-1e9) == 0xFE
    # round trip and ties-to-even on every pair of neighbours
    for c in range(0x7E):
        assert p.fbo_e4m3_satfinite(float(t[c])) == c
        mid = (float(t[c]) + float(t[c + 1])) / 2
        assert p.fbo_e4m3_satfinite(mid) == (c if c % 2 == 0 else c + 1)
    try:
        import torch
        xs = (synth.normal(5, 20000) * 40).astype(np.float32)
        want = torch.from_numpy(xs).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        got = np.array([p.fbo_e4m3_satfinite(float(v)) for v in xs], dtype=np.uint8)
        assert np.array_equal(got, want)
    except ImportError:
        pass


def test_topk_contract():
    # value descending, ties to the lower id, NaN never wins, -0 == +0
    # (tests/kernels/moe/moe_test_common.h:50-65 of the reference)
    l = np.zeros((1, 512), dtype=np.float32)
    l[0, 7] = 2.0
    l[0, 300] = 2.0
    l[0, 5] = np.nan
    l[0, 9] = -0.0
    ids, w = O.topk(l)
    assert list(ids[0][:2]) == [7, 300]
    assert 5 not in ids[0]
    assert list(ids[0][2:]) == [0, 1, 2, 3, 4, 6, 8, 9]
    assert abs(w[0].sum() - 1) < 1e-6
    e = np.exp(l[0, ids[0]].astype(np.float64) - 2.0)
    assert np.allclose(w[0], e / e.sum(), atol=1e-6)


# ------------------------------------------------------------------ direct comparison with the reference
ref_only = pytest.mark.skipif(O.ref() is None, reason="oracle/_ref not built here or CPU lacks AVX-512 VNNI/BF16")


@ref_only
@pytest.mark.parametrize("fmt", [IQ3_S, IQ4_NL])
def test_port_equals_reference_dequant_and_dot(fmt):
    ref = O.ref()
    k = 2560
    nrows = 64
    nb = nrows * k // synth.BLOCK_ELEMS[fmt]
    rows = synth.fill_blocks(fmt, nb, 123, 77)
    assert np.array_equal(bits(O.dequant_rows(fmt, rows, nrows, k)), bits(O.dequant_rows(fmt, rows, nrows, k, lib=ref)))
    x = patterns.all_inputs(k=k, trials=8)
    act = O.ACT_OF[fmt]
    aq = O.quantize_act(act, x)
    assert np.array_equal(aq, O.quantize_act(act, x, lib=ref, variant="avx"))
    # dot: port vs ggml generic (tolerance) and vs the AVX-512 tier (bit-exact through expert_ffn below)
    rb = O.row_bytes(fmt, k)
    fn = ref.ref_vec_dot_iq3_s_q8_K if fmt == IQ3_S else ref.ref_vec_dot_iq4_nl_q8_0
    for r in range(0, nrows, 7):
        for t in range(8):
            a = O.port().fbo_dot(fmt, k, rows[r * rb:].ctypes.data, aq[t].ctypes.data)
            b = fn(k, rows[r * rb:].ctypes.data, aq[t].ctypes.data)
            assert abs(a - b) <= 2e-5 * max(1.0, abs(b))


@ref_only
@pytest.mark.parametrize("fg,fd,inter", [(O.IQ3_XXS, O.IQ4_NL, 512), (O.IQ2_S, O.IQ4_NL, 640), (O.IQ4_XS, O.Q2_0, 512),
                                         (O.IQ2_S, O.Q2_0, 640), (O.IQ3_XXS, O.IQ3_XXS, 512), (O.IQ4_XS, O.IQ4_XS, 512),
                                         (O.IQ2_S, O.IQ2_S, 512)])
def test_port_equals_reference_on_the_other_formats(fg, fd, inter):
    ref = O.ref()
    for fmt in {fg, fd}:
        k = 2560
        rows = synth.fill_blocks(fmt, 16 * k // synth.BLOCK_ELEMS[fmt], 5, 78)
        assert np.array_equal(bits(O.dequant_rows(fmt, rows, 16, k)), bits(O.dequant_rows(fmt, rows, 16, k, lib=ref)))
    xs = synth.activations(89, 4)
    blob = synth.expert_blob(fg, fd, inter, 98, 11)
    h0, y0 = O.expert_ffn(fg, fd, 2560, inter, blob, xs)
    h1, y1 = O.expert_ffn(fg, fd, 2560, inter, blob, xs, lib=ref)
    assert np.array_equal(bits(h0), bits(h1)) and np.array_equal(bits(y0), bits(y1))


@ref_only
def test_port_equals_reference_quantizers_many():
    ref = O.ref()
    x = patterns.all_inputs(trials=160, seed=999)
    for act in (O.ACT_Q8_K, O.ACT_Q8_0):
        assert np.array_equal(O.quantize_act(act, x), O.quantize_act(act, x, lib=ref, variant="avx"))
        assert np.array_equal(O.quantize_act(act, x), O.quantize_act(act, x, lib=ref, variant="ref"))


@ref_only
@pytest.mark.parametrize("fg,fd,inter", [(IQ3_S, IQ3_S, 512), (IQ4_NL, IQ4_NL, 512), (IQ4_NL, IQ4_NL, 640),
                                         (IQ3_S, IQ4_NL, 640)])
def test_port_equals_reference_expert_ffn(fg, fd, inter):
    ref = O.ref()
    xs = synth.activations(88, 5)
    blob = synth.expert_blob(fg, fd, inter, 99, 17)
    h0, y0 = O.expert_ffn(fg, fd, 2560, inter, blob, xs)
    h1, y1 = O.expert_ffn(fg, fd, 2560, inter, blob, xs, lib=ref)
    assert np.array_equal(bits(h0), bits(h1))
    assert np.array_equal(bits(y0), bits(y1))
    # batch invariance of the reference tier (src/cpu/iq_cpu.h:23-27): T tokens == T single calls
    h2, y2 = O.expert_ffn(fg, fd, 2560, inter, blob, xs[3:4], lib=ref)
    assert np.array_equal(bits(y2[0]), bits(y1[3]))


@ref_only
def test_port_equals_reference_moe_layer():
    ref = O.ref()
    E, inter = 12, 512
    stride = synth.blob_bytes(IQ3_S, IQ3_S, inter)
    blobs = np.concatenate([synth.expert_blob(IQ3_S, IQ3_S, inter, 5, e) for e in range(E)])
    x = synth.activations(6, 4)
    ids = np.array([[3, 1, 7], [0, 11, 1], [7, 3, 2], [5, 6, 1]], dtype=np.int32)
    w = np.abs(synth.normal(8, 12)).astype(np.float32).reshape(4, 3)
    y0 = O.moe_layer(IQ3_S, IQ3_S, 2560, inter, blobs, stride, x, ids, w, threads=2)
    y1 = O.moe_layer(IQ3_S, IQ3_S, 2560, inter, blobs, stride, x, ids, w, threads=3, lib=ref)
    assert np.array_equal(bits(y0), bits(y1))


@pytest.mark.skipif(not O.pool_available(), reason="the reference's cpu::ExpertPool is not built here")
@pytest.mark.parametrize("fg,fd", [(IQ3_S, IQ4_NL), (IQ4_NL, IQ4_NL)])
def test_port_equals_the_reference_expert_pool(fg, fd):
    """The reference's production CPU tier itself, cpu::ExpertPool at its native shape (intermediate 640, Q8_0
    down), run through its host exchange: the restatement's MoE layer gives the same bits for the same bf16
    tokens, experts and weights. Batch sizes 1 and 9 (tokens share experts, so the pool groups pairs)."""
    inter, E = 640, 14
    stride = synth.blob_bytes(fg, fd, inter)
    blobs = np.concatenate([synth.expert_blob(fg, fd, inter, 31, e) for e in range(E)])
    rng = np.random.default_rng(5)
    for T in (1, 9):
        xb = synth.to_bf16_bits(synth.activations(60 + T, T))
        ids = np.stack([rng.permutation(E)[:10] for _ in range(T)]).astype(np.int32)
        w = rng.random((T, 10)).astype(np.float32)
        want = O.pool_decode_step(fg, fd, blobs, stride, xb, ids, w, workers=3)
        got = O.moe_layer(fg, fd, 2560, inter, blobs, stride, synth.bf16_bits_to_f32(xb), ids, w, threads=2)
        assert np.array_equal(bits(got), bits(want))


def test_fp8_row_pack_rule_matches_the_reference_tool():
    """The restatement of the FP8-row pack rule (scale = bf16_rne(max / 448), zero rows, clamped round-to-
    nearest-even codes) against outputs of the reference's own tools/fp8row.py quantize_rows, committed as
    tests/golden/fp8row_vectors.npz by tests/golden/make_fp8row_golden.py: codes and scales bit for bit."""
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fp8row_vectors.npz"))
    codes, scales = O.quantize_fp8_rows(g["weight"])
    assert np.array_equal(scales, g["scales"])
    assert np.array_equal(codes, g["codes"])
    assert scales[2] == 0 and not codes[2].any()  # the all-zero row
    # dequantized rows (code value x scale) stay within half an E4M3 step of the source
    tab = O.e4m3_table().astype(np.float64)
    w = synth.bf16_bits_to_f32(g["weight"]).astype(np.float64)
    sc = synth.bf16_bits_to_f32(scales).astype(np.float64)[:, None]
    live = sc[:, 0] > 0
    err = np.abs(tab[codes] * sc - w)[live]
    assert np.all(err <= 2.0 ** -4 * np.maximum(np.abs(w[live]), sc[live] * 2.0 ** -6) + 1e-300)


def test_split_tokens_e4m3x2_is_lossless():
    """The two-piece activation split of the exact FP8-row route (the statement the GPU kernel is checked
    against): scale * (hi + lo) returns every bf16 value of at least 2^-9 of its row's scaled range exactly."""
    x = synth.activations(3, 6) * np.array([1e-3, 0.1, 1.0, 7.0, 300.0, 1e4], dtype=np.float32)[:, None]
    xb = synth.to_bf16_bits(x)
    hi, lo, sc = O.split_tokens_e4m3x2(xb)
    tab = O.e4m3_table().astype(np.float64)
    v = synth.bf16_bits_to_f32(xb).astype(np.float64)
    s = sc.astype(np.float64)[:, None]
    back = s * (tab[hi] + tab[lo])
    big = np.abs(v) >= 0.25 * s
    assert np.array_equal(back[big], v[big]) and np.all(np.abs(back - v) <= s * 2.0 ** -10)
    mx = np.abs(v).max(axis=1)
    assert np.all((mx / sc >= 128) & (mx / sc < 256))


def test_linear_fp8_a16_known_answers():
    """The fp64 statement of the exact-activation FP8-row projection on values chosen so that every
    product is an integer: weights E4M3 {1, -2, 0.5, 448}, activations bf16 {2, 4, -8, 0.5}."""
    t = O.e4m3_table()
    code = {float(t[c]): c for c in range(256) if np.isfinite(t[c])}
    codes = np.array([[code[1.0], code[-2.0], code[0.5], code[448.0]],
                      [code[0.0], code[1.0], code[1.0], code[-1.0]]], dtype=np.uint8)
    x = np.array([[2.0, 4.0, -8.0, 0.5], [1.0, 1.0, 1.0, 1.0]], dtype=np.float32)
    xb = (x.view(np.uint32) >> 16).astype(np.uint16)  # exactly representable in bf16
    acc = O.linear_fp8_a16(xb, codes, np.array([0.5, 2.0]))
    assert np.array_equal(acc, np.array([[(2 - 8 - 4 + 224) * 0.5, (4 - 8 - 0.5) * 2.0], [447.5 * 0.5, 2.0]]))
    sw = O.linear_fp8_a16(xb, codes, np.array([0.5, 2.0]), kind="swiglu")
    g, u = acc[:, :1], acc[:, 1:]
    assert np.allclose(sw, g / (1 + np.exp(-g)) * u, rtol=1e-15)
    sh = O.linear_fp8_a16(xb, codes, np.array([0.5, 2.0]), kind="shared_scale", gate_logit=np.array([0.0, 50.0]))
    assert np.allclose(sh[0], acc[0] * 0.5, rtol=1e-15) and np.allclose(sh[1], acc[1], rtol=1e-15)
