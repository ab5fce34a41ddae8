"""Seeded synthetic inputs for the quantized-expert path (host side, numpy).

The byte streams are defined with integer arithmetic only, so the device generator
(`fb_synth_fill_blocks`) and this module produce identical expert blobs:
  word(seed, c) = splitmix64 output number c of a generator seeded with `seed`
                  (the reference's test generator, tests/common/test_util.h:58-67);
  block b of a tensor takes words [b*W, b*W + W), W = ceil(block_bytes / 8); its bytes 2.. are the
  stream's bytes 2.., and its fp16 scale (bytes 0-1) is d_table[word0 & 0xFFFF];
  d_table[i] = fp16(|N(0,1)| * scale), N(0,1) by Box-Muller over the same generator
  (tests/common/test_util.h:71-76).
"""
import numpy as np

GOLDEN = np.uint64(0x9E3779B97F4A7C15)
# ggml type ids: 21 IQ3_S, 20 IQ4_NL; the other expert formats of the reference: 18 IQ3_XXS, 22 IQ2_S, 23 IQ4_XS,
# 42 Q2_0 (a 64-element block). Every block starts with its fp16 scale.
BLOCK_BYTES = {21: 110, 20: 18, 18: 98, 22: 82, 23: 136, 42: 18}
BLOCK_ELEMS = {21: 256, 20: 32, 18: 256, 22: 256, 23: 256, 42: 64}
D_SCALE = {21: 0.02, 20: 0.05, 18: 0.004, 22: 0.004, 23: 0.002, 42: 0.05}


def splitmix_words(seed, start, count):
    """Words start..start+count-1 of the splitmix64 stream seeded with `seed` (uint64 array)."""
    with np.errstate(over="ignore"):
        c = np.arange(start + 1, start + count + 1, dtype=np.uint64)
        z = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + c * GOLDEN
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def uniform(seed, start, count):
    return (splitmix_words(seed, start, count) >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def normal(seed, count):
    """count N(0,1) variates in the order the reference's Rng::normal() yields them (float64)."""
    u = uniform(seed, 0, 2 * count)
    u1 = np.maximum(u[0::2], 1e-300)
    u2 = u[1::2]
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(6.283185307179586 * u2)


def d_table(fmt, seed=0xD7AB1E):
    """65536 fp16 scales |N(0,1)| * D_SCALE[fmt] (0.02 for IQ3_S, 0.05 for IQ4_NL), as uint16 bit patterns."""
    v = np.abs(normal(seed + fmt, 65536)) * D_SCALE[fmt]
    return v.astype(np.float16).view(np.uint16)


def fill_blocks(fmt, n_blocks, first_block, seed, table=None):
    """Host twin of fb_synth_fill_blocks: uint8 [n_blocks * block_bytes]."""
    bb = BLOCK_BYTES[fmt]
    w = (bb + 7) // 8
    table = d_table(fmt) if table is None else table
    words = splitmix_words(seed, first_block * w, n_blocks * w).reshape(n_blocks, w)
    raw = words.view(np.uint8).reshape(n_blocks, 8 * w)[:, :bb].copy()
    d = table[(words[:, 0] & np.uint64(0xFFFF)).astype(np.int64)]
    raw[:, 0] = (d & 0xFF).astype(np.uint8)
    raw[:, 1] = (d >> 8).astype(np.uint8)
    return raw.reshape(-1)


def blob_bytes(fmt_gu, fmt_down, inter, hidden=2560):
    gu = hidden // BLOCK_ELEMS[fmt_gu] * BLOCK_BYTES[fmt_gu]
    dn = inter // BLOCK_ELEMS[fmt_down] * BLOCK_BYTES[fmt_down]
    return 2 * inter * gu + hidden * dn


def expert_blob(fmt_gu, fmt_down, inter, seed, expert, hidden=2560, tables=None):
    """One expert's gate | up | down bytes. The gate/up part and the down part are separate streams
    (seed and seed ^ 0xD0), each indexed by the block's position in the whole layer."""
    tables = tables or {}
    nb_gu = 2 * inter * (hidden // BLOCK_ELEMS[fmt_gu])
    nb_dn = hidden * (inter // BLOCK_ELEMS[fmt_down])
    gu = fill_blocks(fmt_gu, nb_gu, expert * nb_gu, seed, tables.get(fmt_gu))
    dn = fill_blocks(fmt_down, nb_dn, expert * nb_dn, seed ^ 0xD0, tables.get(fmt_down))
    return np.concatenate([gu, dn])


def activations(seed, tokens, hidden=2560):
    """x ~ N(0,1) float32 [tokens][hidden]."""
    return normal(seed, tokens * hidden).astype(np.float32).reshape(tokens, hidden)


def to_bf16_bits(x):
    """float32 -> bf16 bit patterns (uint16), round to nearest even."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((b + np.uint64(0x7FFF) + ((b >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def router_weights(seed, rows=512, hidden=2560, std=0.02):
    """bf16 router [rows][hidden] ~ N(0, std) as uint16 bit patterns."""
    return to_bf16_bits((normal(seed, rows * hidden) * std).astype(np.float32)).reshape(rows, hidden)


def zipf_router_bias(seed, n_experts=512, exponent=1.1, spread=0.41):
    """Router-logit bias that makes expert popularity follow Zipf(exponent) over a seeded permutation of
    the experts: bias[perm[r]] = -exponent * spread * ln(r + 1). With unit-variance logit noise spread =
    0.41 gives a fitted log-log slope of pairs against rank of -exponent. float32 [n_experts]."""
    order = np.argsort(splitmix_words(seed, 0, n_experts), kind="stable")
    bias = np.empty(n_experts, dtype=np.float32)
    bias[order] = (-exponent * spread * np.log(np.arange(1, n_experts + 1, dtype=np.float64))).astype(np.float32)
    return bias


def fp8_row_weight(seed, n, k):
    """FP8-row weight of the dense-GEMM benchmark definition: values ~ N(0,1) clipped to +-448 and
    rounded to E4M3FN (nearest even), one fp32 scale per row ~ U(0.001, 0.01).
    Returns (codes uint8 [n][k], scales float32 [n])."""
    import torch
    v = np.clip(normal(seed, n * k), -448.0, 448.0).astype(np.float32).reshape(n, k)
    codes = torch.from_numpy(v).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    scales = (0.001 + 0.009 * uniform(seed ^ 0x5CA1E, 0, n)).astype(np.float32)
    return codes, scales
