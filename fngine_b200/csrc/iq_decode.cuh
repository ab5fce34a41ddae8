// Device routines for the GGUF expert formats: codebook tables in shared memory, exact integer
// decode of IQ3_S / IQ4_NL sub-blocks into dp4a operands, and the Q8_K / Q8_0 activation
// quantizers. The GEMV kernels and the parity probes call the same functions.
//
// Format definitions follow third_party/ggml-iq/ggml-iq.h:81-96 and the reference dequantizers
// third_party/ggml-iq/ggml-iq.c:231-288 of the reference project.
#pragma once

#include <cuda_fp16.h>

#include "common.cuh"
#include "iq_codebooks.h"

namespace fb {

// ------------------------------------------------------------------------------ tables
// IQ3_S codebook in shared memory, replicated once per lane: entry i of lane l lives at word
// i*32 + l, so a warp's 32 independent look-ups always hit 32 different banks.
constexpr int kGridRepWords = 512 * 32;
constexpr int kGridRepBytes = kGridRepWords * 4;  // 65536
// Sign masks: nibble n -> four bytes, 0xFF where bit j of n is set. 16 words, 16 banks.
constexpr int kSignTabWords = 16;

// One copy per translation unit (internal linkage), initialised at load time.
static __constant__ uint16_t c_iq3s_grid_packed[512] = {FB_IQ3S_GRID_PACKED};

__device__ __forceinline__ uint32_t iq3s_grid_entry(int i) {
  const uint32_t p = c_iq3s_grid_packed[i];
  uint32_t w = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) w |= (2u * ((p >> (3 * j)) & 7u) + 1u) << (8 * j);
  return w;
}

// Called by every thread of the block; caller synchronizes afterwards.
__device__ __forceinline__ void iq3s_tables_fill(uint32_t* gridrep, uint32_t* signtab) {
  // consecutive threads write consecutive 16-byte pieces (eight per entry): no bank conflicts
  for (int i = threadIdx.x; i < 512 * 8; i += blockDim.x) {
    const uint32_t w = iq3s_grid_entry(i >> 3);
    reinterpret_cast<uint4*>(gridrep)[i] = make_uint4(w, w, w, w);
  }
  if (threadIdx.x < 16) {
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (threadIdx.x & (1 << j)) m |= 0xFFu << (8 * j);
    signtab[threadIdx.x] = m;
  }
}

// ------------------------------------------------------------------------------ IQ3_S
// One 32-weight sub-block. Inputs: qs_lo/qs_hi = its 8 index bytes, qh = a word whose bits
// [sh, sh+8) are the 8 ninth index bits, sg = its 4 sign bytes (nibble l = signs of look-up l).
// Outputs per look-up l: g[l] = four magnitudes (bytes, element order), m[l] = 0xFF in the bytes
// whose weight is negative. grid_lane = gridrep + lane.
//
// Instruction budget matters here (the integer pipe, not HBM, bounds this kernel): the ninth
// index bits are spread to bytes with one multiply per nibble, then each 9-bit index is one
// byte-permute (low byte from qs, high byte from the spread bits) and each sign-table offset is
// one byte-permute of the pre-scaled nibbles.
// prmt.b32 in its default mode: selector nibble n picks byte (n & 7) of {a, b}; with bit 3 set the
// selected byte's sign bit is replicated over the output byte instead (0x00 for bytes < 0x80).
// (__byte_perm documents only three selector bits per byte, so the PTX form is spelled out.)
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

__device__ __forceinline__ void iq3s_decode_sub(uint32_t qs_lo, uint32_t qs_hi, uint32_t qh, int sh, uint32_t sg,
                                                const uint32_t* grid_lane, const uint32_t* signtab,
                                                uint32_t (&g)[8], uint32_t (&m)[8]) {
  // bit j of a nibble -> byte j (0 or 1): n * (1 + 2^7 + 2^14 + 2^21) has bit j at position 8j
  const uint32_t h_lo = (((qh >> sh) & 0xFu) * 0x00204081u) & 0x01010101u;
  const uint32_t h_hi = (((qh >> (sh + 4)) & 0xFu) * 0x00204081u) & 0x01010101u;
  // nibbles pre-scaled by 4 (byte offsets into the 16-word sign table)
  const uint32_t s_even = (sg << 2) & 0x3C3C3C3Cu;  // look-ups 0,2,4,6
  const uint32_t s_odd = (sg >> 2) & 0x3C3C3C3Cu;   // look-ups 1,3,5,7
  const char* signb = reinterpret_cast<const char*>(signtab);
#pragma unroll
  for (int l = 0; l < 8; ++l) {
    const int b = l & 3;
    // byte0 = qs byte b, byte1 = spread bit b, bytes 2-3 = 0 (sign-replicate of a 0/1 byte)
    const uint32_t sel = uint32_t(b) | (uint32_t(4 + b) << 4) | (uint32_t(0xC + b) << 8) | (uint32_t(0xC + b) << 12);
    const uint32_t idx = prmt(l < 4 ? qs_lo : qs_hi, l < 4 ? h_lo : h_hi, sel);
    g[l] = grid_lane[idx * 32];
    const uint32_t off = __byte_perm((l & 1) ? s_odd : s_even, 0u, 0x4440u | uint32_t(l >> 1));
    m[l] = *reinterpret_cast<const uint32_t*>(signb + off);
  }
}

// Signed int8x4 weights from (g, m): byte-wise negation where m = 0xFF; (g ^ 0xFF) + 1 never carries
// because every magnitude is odd.
__device__ __forceinline__ int iq3s_signed(uint32_t g, uint32_t m) { return int((g ^ m) + (m & 0x01010101u)); }

// sum_i s_i g_i a_i over 32 weights for one token: with x = g ^ m (negated bytes become -g-1),
// sum s g a = dp4a(x, a) - dp4a(m, a) since m's 0xFF bytes are -1.
__device__ __forceinline__ int iq3s_dot32(const uint32_t (&g)[8], const uint32_t (&m)[8], const int8_t* a) {
  const int4 a0 = *reinterpret_cast<const int4*>(a);
  const int4 a1 = *reinterpret_cast<const int4*>(a + 16);
  const int av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
  int p = 0, n = 0;
#pragma unroll
  for (int l = 0; l < 8; ++l) {
    p = __dp4a(int(g[l] ^ m[l]), av[l], p);
    n = __dp4a(int(m[l]), av[l], n);
  }
  return p - n;
}

// dp4a of 8 signed weight words with 32 int8 activations at `a` (16-byte aligned shared memory).
__device__ __forceinline__ int dot32(const int (&w)[8], const int8_t* a) {
  const int4 a0 = *reinterpret_cast<const int4*>(a);
  const int4 a1 = *reinterpret_cast<const int4*>(a + 16);
  int s = __dp4a(w[0], a0.x, 0);
  s = __dp4a(w[1], a0.y, s);
  s = __dp4a(w[2], a0.z, s);
  s = __dp4a(w[3], a0.w, s);
  s = __dp4a(w[4], a1.x, s);
  s = __dp4a(w[5], a1.y, s);
  s = __dp4a(w[6], a1.z, s);
  s = __dp4a(w[7], a1.w, s);
  return s;
}

// 4 bytes at a static byte offset (a multiple of 2) of a word-aligned unit in shared memory.
template <int OFF>
__device__ __forceinline__ uint32_t ld4(const uint32_t* u) {
  if constexpr (OFF % 4 == 0) return u[OFF / 4];
  else return __byte_perm(u[OFF / 4], u[OFF / 4 + 1], 0x5432);
}
template <int OFF>
__device__ __forceinline__ float ld_fp16(const uint32_t* u) {
  const uint32_t v = u[OFF / 4] >> (8 * (OFF % 4));
  return __half2float(__ushort_as_half(static_cast<unsigned short>(v & 0xFFFFu)));
}

// An IQ3_S block is a 2-byte scale followed by 27 words: 16 of index bytes, 2 of ninth bits, 8 of
// signs, 1 of sub-block scales. In a 220-byte unit (two blocks, word aligned) the first block's
// 27 words sit 2 bytes off word alignment, the second block's are aligned: S<MIS>(w, k) reads
// word k of the stream either way (w = the word holding the fp16 scale).
template <bool MIS>
__device__ __forceinline__ uint32_t iq3s_stream(const uint32_t* w, int k) {
  if constexpr (MIS) return __byte_perm(w[k], w[k + 1], 0x5432);
  else return w[k + 1];
}

// Integer dot of one IQ3_S block with TT activation blocks: bsum[t] = sum over its 8 sub-blocks of
// (2*s+1) * sum_i w_i * a_t,i, exact in int32 (|bsum| < 2^24, so float(bsum) is exact).
// act[t] points at the 256 int8 of the matching Q8_K block. Two runtime halves of four unrolled
// sub-blocks keep the loop body inside the instruction cache.
template <bool MIS, int TT>
__device__ __forceinline__ void iq3s_block_idot(const uint32_t* w, const uint32_t* grid_lane,
                                                const uint32_t* signtab, const int8_t* const (&act)[TT],
                                                int (&bsum)[TT]) {
  const uint32_t sc = iq3s_stream<MIS>(w, 26);
#pragma unroll
  for (int t = 0; t < TT; ++t) bsum[t] = 0;
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    const uint32_t qh = iq3s_stream<MIS>(w, 16 + half);
    const uint32_t sch = sc >> (16 * half);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int ib = 4 * half + i;
      uint32_t g[8], m[8];
      iq3s_decode_sub(iq3s_stream<MIS>(w, 2 * ib), iq3s_stream<MIS>(w, 2 * ib + 1), qh, 8 * i,
                      iq3s_stream<MIS>(w, 18 + ib), grid_lane, signtab, g, m);
      const int mult = 2 * int((sch >> (4 * i)) & 0xFu) + 1;
#pragma unroll
      for (int t = 0; t < TT; ++t) bsum[t] += iq3s_dot32(g, m, act[t] + 32 * ib) * mult;
    }
  }
}

// ------------------------------------------------------------------------------ IQ4_NL
// The 16 levels held in four registers for byte-permute look-ups.
struct Iq4nlLevels {
  uint32_t t0, t1, t2, t3;
};
__host__ __device__ constexpr uint32_t iq4nl_pack4(int q) {
  constexpr int lv[16] = {FB_IQ4NL_LEVELS};
  return uint32_t(uint8_t(lv[4 * q])) | (uint32_t(uint8_t(lv[4 * q + 1])) << 8) |
         (uint32_t(uint8_t(lv[4 * q + 2])) << 16) | (uint32_t(uint8_t(lv[4 * q + 3])) << 24);
}
__device__ __forceinline__ Iq4nlLevels iq4nl_levels() {
  constexpr uint32_t a = iq4nl_pack4(0), b = iq4nl_pack4(1), c = iq4nl_pack4(2), d = iq4nl_pack4(3);
  Iq4nlLevels L;
  L.t0 = a;
  L.t1 = b;
  L.t2 = c;
  L.t3 = d;
  return L;
}
__host__ __device__ constexpr int iq4nl_level(int i) {
  constexpr int lv[16] = {FB_IQ4NL_LEVELS};
  return lv[i];
}
// Four nibbles n0..n3 (n0 in bits 0-3 of h16) -> four int8 levels, byte i = level[n_i].
__device__ __forceinline__ uint32_t iq4nl_lookup4(const Iq4nlLevels& L, uint32_t h16) {
  const uint32_t sel = h16 & 0x7777u;
  const uint32_t lo = __byte_perm(L.t0, L.t1, sel);
  const uint32_t hi = __byte_perm(L.t2, L.t3, sel);
  return __byte_perm(lo, hi, 0x3210u | ((h16 >> 1) & 0x4444u));
}
// One 32-weight block from its 16 nibble bytes (4 words). Output word 2m+h (m = word, h = half)
// holds weights of elements {4m+2h, 4m+2h+16, 4m+2h+1, 4m+2h+17}: activations are stored in
// that interleaved order (see q8_0_interleave_index).
__device__ __forceinline__ void iq4nl_decode32(const Iq4nlLevels& L, const uint32_t (&q)[4], int (&w)[8]) {
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    w[2 * m] = int(iq4nl_lookup4(L, q[m] & 0xFFFFu));
    w[2 * m + 1] = int(iq4nl_lookup4(L, q[m] >> 16));
  }
}
// Position of element e (0..31) of a Q8_0 block in the interleaved activation order.
__host__ __device__ __forceinline__ int q8_0_interleave_index(int e) {
  return 2 * (e & 15) + (e >> 4);  // nibble byte e%16, low nibble first
}

// ------------------------------------------------------------------------------ quantizers
// Q8_K of one 256-value block by one warp; lane l holds elements 8l..8l+7 in v.
// quantize_row_q8_K_ref, third_party/ggml-iq/ggml-iq.c:313-350: max is the FIRST element of
// largest magnitude (signed), iscale = -127/max, q = min(127, rne(iscale*x)), d = 1/iscale; an
// all-zero block gives d = 0, q = 0, bsums = 0 (src/cpu/q8_cpu.h:7-8).
// Returns d; q[8] are this lane's codes; pair_sum is the sum of the 16 codes of this lane's group
// of 16 (valid in both lanes of the pair).
__device__ __forceinline__ float q8k_block_warp(const float (&v)[8], int (&q)[8], int& pair_sum) {
  const int lane = threadIdx.x & 31;
  float amax = 0.0f;
  int idx = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float a = fabsf(v[i]);
    if (a > amax) {
      amax = a;
      idx = 8 * lane + i;
    }
  }
  if (amax == 0.0f) idx = 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (oa > amax || (oa == amax && oi < idx)) {
      amax = oa;
      idx = oi;
    }
  }
  if (amax == 0.0f) {
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = 0;
    pair_sum = 0;
    return 0.0f;
  }
  float cand = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if ((idx & 7) == i) cand = v[i];
  const float mx = __shfl_sync(0xffffffffu, cand, idx >> 3);
  const float iscale = __fdiv_rn(-127.0f, mx);
  int s = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = __float2int_rn(__fmul_rn(iscale, v[i]));
    q[i] = r < 127 ? r : 127;
    s += q[i];
  }
  pair_sum = s + __shfl_xor_sync(0xffffffffu, s, 1);
  return __fdiv_rn(1.0f, iscale);
}

// Q8_0 of one 32-value block by one warp; lane l holds element l.
// quantize_row_q8_0_ref, third_party/ggml-iq/ggml-iq.c:75-98: d = amax/127 stored as fp16,
// id = 1/d computed in fp32 from the unrounded d, q = roundf(x*id).
__device__ __forceinline__ int q8_0_block_warp(float v, unsigned short& d_half) {
  float amax = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float d = __fdiv_rn(amax, 127.0f);
  const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
  d_half = __half_as_ushort(__float2half_rn(d));
  return int(roundf(__fmul_rn(v, id)));
}

// ------------------------------------------------------------------------------ routing
// Top-10 of 512 logits by one warp (lane l holds logits l + 32 i): value descending, ties to the
// lower id, NaN never wins, -0 == +0; weights = softmax over the winners in fp32, summed in rank
// order (src/kernels/moe/moe_common.cuh:33-85 of the reference states the same contract).
// Order-preserving map of a float to uint32 (larger float -> larger key); NaN maps below every
// number and -0 equals +0.
__device__ __forceinline__ uint32_t logit_key(float x) {
  if (x != x) x = -INFINITY;
  if (x == 0.0f) x = 0.0f;
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// weights = softmax over the ten winners (fp32, expf(v - top), summed in rank order).
__device__ __forceinline__ void topk_softmax(float (&vals)[FB_TOPK], float* weights) {
  float sum = 0.0f;
  const float top = vals[0];
#pragma unroll
  for (int k = 0; k < FB_TOPK; ++k) {
    vals[k] = expf(vals[k] - top);
    sum += vals[k];
  }
  const float inv = __fdiv_rn(1.0f, sum);
#pragma unroll
  for (int k = 0; k < FB_TOPK; ++k) weights[k] = vals[k] * inv;
}
__device__ __forceinline__ float key_logit(uint32_t key) {
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// Two-level top-10. Level one: a warp holds 32 consecutive experts' logits of one token, one per
// lane, and emits their ten best as (key, id) candidates, best first (lane k < 10 returns the k-th).
// The global top-10 is a subset of the union of such candidate lists, and the tie rule (lower id)
// holds inside a list because ids grow with the lane.
__device__ __forceinline__ void warp_top10_of32(float logit, int id, uint32_t& out_key, int& out_id) {
  const int lane = threadIdx.x & 31;
  uint32_t key = logit_key(logit);
  out_key = 0u;
  out_id = 0;
#pragma unroll
  for (int k = 0; k < FB_TOPK; ++k) {
    const uint32_t best = __reduce_max_sync(0xffffffffu, key);
    const int win = int(__reduce_min_sync(0xffffffffu, key == best ? uint32_t(lane) : 0xffffffffu));
    const int wid = __shfl_sync(0xffffffffu, id, win);
    if (lane == k) {
      out_key = best;
      out_id = wid;
    }
    if (lane == win) key = 0u;  // retired: below every real key
  }
}
// Level two: one warp merges n_cand (<= 160) candidates of a token; load(c, key, id) reads candidate c.
template <class LoadF>
__device__ __forceinline__ void warp_topk10_merge(LoadF load, int n_cand, int* ids, float* weights) {
  const int lane = threadIdx.x & 31;
  uint32_t key[5];
  int cid[5];
#pragma unroll
  for (int j = 0; j < 5; ++j) {
    key[j] = 0u;
    cid[j] = 0x7fffffff;
    if (lane + 32 * j < n_cand) load(lane + 32 * j, key[j], cid[j]);
  }
  float vals[FB_TOPK];
#pragma unroll
  for (int k = 0; k < FB_TOPK; ++k) {
    // lane-local best: larger key, then lower id
    uint32_t bk = key[0];
    int bi = cid[0];
#pragma unroll
    for (int j = 1; j < 5; ++j) {
      const bool up = key[j] > bk || (key[j] == bk && cid[j] < bi);
      bk = up ? key[j] : bk;
      bi = up ? cid[j] : bi;
    }
    const uint32_t best = __reduce_max_sync(0xffffffffu, bk);
    const int win = int(__reduce_min_sync(0xffffffffu, bk == best ? uint32_t(bi) : 0xffffffffu));
    ids[k] = win;
    vals[k] = key_logit(best);
#pragma unroll
    for (int j = 0; j < 5; ++j)
      if (key[j] == best && cid[j] == win) key[j] = 0u;
  }
  topk_softmax(vals, weights);
}

template <class LoadF>
__device__ __forceinline__ void warp_topk10(LoadF load_logit, int* ids, float* weights) {
  const int lane = threadIdx.x & 31;
  uint32_t key[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) key[i] = logit_key(load_logit(lane + 32 * i));
  float vals[FB_TOPK];
#pragma unroll
  for (int k = 0; k < FB_TOPK; ++k) {
    // lane-local best as a 4-level tree: a higher slot wins only when strictly greater, so equal
    // keys resolve to the lower id; the warp step is two redux operations (max key, then min id).
    uint32_t tk[16];
    int ti[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      tk[i] = key[i];
      ti[i] = i;
    }
#pragma unroll
    for (int w = 1; w < 16; w <<= 1) {
#pragma unroll
      for (int i = 0; i < 16; i += 2 * w) {
        const bool up = tk[i + w] > tk[i];
        tk[i] = up ? tk[i + w] : tk[i];
        ti[i] = up ? ti[i + w] : ti[i];
      }
    }
    const uint32_t best = __reduce_max_sync(0xffffffffu, tk[0]);
    const uint32_t cand = tk[0] == best ? uint32_t(lane + 32 * ti[0]) : 0xffffffffu;
    const int win = int(__reduce_min_sync(0xffffffffu, cand));
    ids[k] = win;
    const uint32_t u = (best & 0x80000000u) ? (best & 0x7fffffffu) : ~best;
    vals[k] = __uint_as_float(u);
    // retire the winner: key 0 is below every real key (the smallest real key is ~0xFF800000 = 0x007FFFFF)
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (win == lane + 32 * i) key[i] = 0u;
  }
  topk_softmax(vals, weights);
}

// The same selection as a short dependent chain (a decode step runs it in every CTA). The tenth largest
// of the 32 lanes' own maxima is a lower bound of the tenth largest logit (ten different logits reach it),
// so only logits at or above it can win; they are compacted into `scratch` (32 entries of this warp, shared
// memory), one per lane, every lane ranks its candidate against the others through shuffles (larger key,
// then lower id: a strict order), and ranks 0..9 are the winners. More than 32 survivors (many equal
// logits) take the general path. Same winners, same order, same weights as warp_topk10; out_ids / out_w
// (ten entries each, shared memory) are complete after the caller's next barrier.
template <class LoadF>
__device__ __forceinline__ void warp_topk10_pruned(LoadF load_logit, uint2* scratch, int* out_ids, float* out_w) {
  const int lane = threadIdx.x & 31;
  uint32_t key[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) key[i] = logit_key(load_logit(lane + 32 * i));
  uint32_t lm = key[0];
#pragma unroll
  for (int i = 1; i < 16; ++i) lm = max(lm, key[i]);
  int above = 0;  // lanes whose maximum is larger than this lane's
#pragma unroll
  for (int j = 0; j < 32; ++j) above += __shfl_sync(0xffffffffu, lm, j) > lm ? 1 : 0;
  const uint32_t thr = __reduce_min_sync(0xffffffffu, above < FB_TOPK ? lm : 0xffffffffu);
  int total = 0;
  const uint32_t below = (1u << lane) - 1u;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const bool in = key[i] >= thr;
    const uint32_t m = __ballot_sync(0xffffffffu, in);
    const int pos = total + __popc(m & below);
    if (in && pos < 32) scratch[pos] = make_uint2(key[i], uint32_t(lane + 32 * i));
    total += __popc(m);
  }
  if (total > 32) {
    int ids[FB_TOPK];
    float w[FB_TOPK];
    warp_topk10(load_logit, ids, w);
#pragma unroll
    for (int k = 0; k < FB_TOPK; ++k)
      if (lane == k) {
        out_ids[k] = ids[k];
        out_w[k] = w[k];
      }
    return;
  }
  __syncwarp();
  uint32_t ck = 0u, cid = 0xffffffffu;  // padding lanes lose to every candidate
  if (lane < total) {
    const uint2 c = scratch[lane];
    ck = c.x;
    cid = c.y;
  }
  int rank = 0;  // (only the real candidates take a turn: a lone warp pays a few cycles per instruction)
#pragma unroll 4
  for (int j = 0; j < total; ++j) {
    const uint32_t ok = __shfl_sync(0xffffffffu, ck, j), oi = __shfl_sync(0xffffffffu, cid, j);
    rank += (ok > ck || (ok == ck && oi < cid)) ? 1 : 0;
  }
  if (lane >= total) rank = 32;
  __syncwarp();  // every lane holds its candidate: the scratch entries can carry the winners' logits now
  float* vals = reinterpret_cast<float*>(scratch);
  if (rank < FB_TOPK) {
    out_ids[rank] = int(cid);
    vals[rank] = key_logit(ck);
  }
  __syncwarp();
  // softmax over the winners exactly as topk_softmax: exp(v - top), summed in rank order. Lane k computes
  // the k-th term; the ten terms then reach every lane through shuffles and are added in the same order.
  const float e = expf(vals[lane < FB_TOPK ? lane : 0] - vals[0]);
  float sum = 0.0f;
#pragma unroll
  for (int k = 0; k < FB_TOPK; ++k) sum += __shfl_sync(0xffffffffu, e, k);
  if (lane < FB_TOPK) out_w[lane] = e * __fdiv_rn(1.0f, sum);
}

}  // namespace fb
