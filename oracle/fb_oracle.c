// TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's quantized-expert path.
//
// Nothing the library ships may include, link or call this file; it exists so that the test
// suite and the benchmark's CPU-baseline leg have an independent checker. Plain scalar C, no
// intrinsics, so it runs on any host. Each function names the reference code it restates
// (paths are relative to the reference project's root).
//
// Parity status: PINNED. tests/test_oracle_pins.py checks every function below against the
// reference's own code compiled from its sources (oracle/_ref, built by oracle/build_ref.py) and
// against committed vectors in tests/golden/ that were produced by that build.
//
// Build: gcc -O2 -std=c11 -fno-fast-math -ffp-contract=off -shared -fPIC fb_oracle.c -lm -lpthread
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "fb_oracle_codebooks.h"

#define FBO_IQ3_XXS 18
#define FBO_IQ4_NL 20
#define FBO_IQ3_S 21
#define FBO_IQ2_S 22
#define FBO_IQ4_XS 23
#define FBO_Q2_0 42
#define FBO_ACT_Q8_K 0
#define FBO_ACT_Q8_0 1

// ---------------------------------------------------------------------------------- formats
// Block layouts: third_party/ggml-iq/ggml-iq.h:32-37 (q8_0), :52-57 (q8_K), :81-89 (iq3_s),
// :91-96 (iq4_nl). Byte-packed, no padding.
#pragma pack(push, 1)
typedef struct { uint16_t d; uint8_t qs[64]; uint8_t qh[8]; uint8_t signs[32]; uint8_t scales[4]; } fbo_iq3s;
typedef struct { uint16_t d; uint8_t qs[16]; } fbo_iq4nl;
typedef struct { uint16_t d; uint8_t qs[64]; uint8_t qh[8]; uint8_t scales[8]; } fbo_iq2s;   /* ggml-iq.h:59-64; qs[32..63] = signs */
typedef struct { uint16_t d; uint8_t qs[96]; } fbo_iq3xxs;                                    /* :67-70; qs[64..95] = scales and signs */
typedef struct { uint16_t d; uint16_t scales_h; uint8_t scales_l[4]; uint8_t qs[128]; } fbo_iq4xs; /* :73-78 */
typedef struct { uint16_t d; uint8_t qs[16]; } fbo_q20;                                        /* :26-29, 64 elements */
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } fbo_q8k;
typedef struct { uint16_t d; int8_t qs[32]; } fbo_q80;
#pragma pack(pop)
_Static_assert(sizeof(fbo_iq3s) == 110, "iq3_s block");
_Static_assert(sizeof(fbo_iq4nl) == 18, "iq4_nl block");
_Static_assert(sizeof(fbo_iq2s) == 82 && sizeof(fbo_iq3xxs) == 98 && sizeof(fbo_iq4xs) == 136 && sizeof(fbo_q20) == 18,
               "iq2_s / iq3_xxs / iq4_xs / q2_0 blocks");
_Static_assert(sizeof(fbo_q8k) == 292, "q8_K block");
_Static_assert(sizeof(fbo_q80) == 34, "q8_0 block");

static uint8_t g_grid[512][4];
static uint8_t g_grid3xxs[256][4];
static uint8_t g_grid2s[1024][8];
static int g_grid_ready = 0;
static void grid_init(void) {
  if (g_grid_ready) return;
  for (int i = 0; i < 512; ++i)
    for (int j = 0; j < 4; ++j) g_grid[i][j] = (uint8_t)(2 * ((kIq3sGridPacked[i] >> (3 * j)) & 7) + 1);
  for (int i = 0; i < 256; ++i)
    for (int j = 0; j < 4; ++j) {
      const int c = (kIq3xxsGridPacked[i] >> (3 * j)) & 7;
      g_grid3xxs[i][j] = (uint8_t)(c < 7 ? 4 + 8 * c : 62);
    }
  static const uint8_t lv2[4] = {8, 25, 43, 0};
  for (int i = 0; i < 1024; ++i)
    for (int j = 0; j < 8; ++j) g_grid2s[i][j] = lv2[(kIq2sGridPacked[i] >> (2 * j)) & 3];
  g_grid_ready = 1;
}
// ksigns_iq2xs (ggml-iq-tables.h): the 7-bit index with its parity as bit 7.
static uint8_t ksigns(int i) { return (uint8_t)(i | ((__builtin_popcount((unsigned)i) & 1) << 7)); }

// Row bytes: src/kernels/moe/moe_format.cpp:5-15.
int64_t fbo_row_bytes(int fmt, int k) {
  if (fmt == FBO_IQ3_S) return (int64_t)(k / 256) * 110;
  if (fmt == FBO_IQ4_NL) return (int64_t)(k / 32) * 18;
  if (fmt == FBO_IQ3_XXS) return (int64_t)(k / 256) * 98;
  if (fmt == FBO_IQ2_S) return (int64_t)(k / 256) * 82;
  if (fmt == FBO_IQ4_XS) return (int64_t)(k / 256) * 136;
  if (fmt == FBO_Q2_0) return (int64_t)(k / 64) * 18;
  return 0;
}
// Activation format a weight format pairs with: src/cpu/iq_cpu.cpp:467-478.
int fbo_act_of(int fmt) { return fmt == FBO_IQ4_NL || fmt == FBO_Q2_0 ? FBO_ACT_Q8_0 : FBO_ACT_Q8_K; }

// ---------------------------------------------------------------------------------- fp16 / bf16
// IEEE binary16 <-> binary32, round to nearest even (what GGML_FP32_TO_FP16 / _FP16_TO_FP32
// compute, third_party/ggml-iq/ggml-iq.h:113-170).
float fbo_fp16_to_fp32(uint16_t h) {
  const uint32_t s = (uint32_t)(h & 0x8000) << 16;
  const uint32_t e = (h >> 10) & 0x1F, m = h & 0x3FF;
  uint32_t w;
  if (e == 0) {
    if (m == 0) {
      w = s;
    } else {
      int sh = 0;
      uint32_t mm = m;
      while (!(mm & 0x400)) { mm <<= 1; ++sh; }
      w = s | ((uint32_t)(113 - sh) << 23) | ((mm & 0x3FF) << 13);
    }
  } else if (e == 31) {
    w = s | 0x7F800000u | (m << 13);
  } else {
    w = s | ((e + 112) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &w, 4);
  return f;
}

uint16_t fbo_fp32_to_fp16(float f) {
  uint32_t w;
  memcpy(&w, &f, 4);
  const uint16_t s = (uint16_t)((w >> 16) & 0x8000);
  const uint32_t a = w & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return (uint16_t)(s | 0x7E00);          // NaN
  if (a >= 0x477FF000u) return (uint16_t)(s | 0x7C00);         // rounds to inf (>= 65520)
  if (a < 0x33000001u) return s;                               // <= 2^-25: rounds to zero
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
  int shift;
  uint32_t base;
  if (e < -14) {  // subnormal half: value = m * 2^(e-23); unit 2^-24
    shift = 13 + (-14 - e);
    base = 0;
  } else {
    shift = 13;
    base = (uint32_t)(e + 15) << 10;
    m &= 0x7FFFFFu;
  }
  uint32_t q = m >> shift;
  const uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1))) ++q;
  return (uint16_t)(s | (base + q));  // a carry out of the mantissa bumps the exponent correctly
}

float fbo_bf16_to_fp32(uint16_t b) {
  const uint32_t w = (uint32_t)b << 16;
  float f;
  memcpy(&f, &w, 4);
  return f;
}
// RNE, NaN preserved: tests/common/test_util.h:88-100.
uint16_t fbo_fp32_to_bf16(float f) {
  uint32_t w;
  memcpy(&w, &f, 4);
  if ((w & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((w >> 16) | 0x40);
  return (uint16_t)((w + 0x7fffu + ((w >> 16) & 1u)) >> 16);
}

// ---------------------------------------------------------------------------------- dequantize
// third_party/ggml-iq/ggml-iq.c:231-270. Sub-block ib (32 weights) uses qs[8ib..8ib+7], the
// ninth index bit of entry l from qh[ib] bit l, signs[4ib..4ib+3] (bit j of signs[l'] negates
// weight j of that group of 8), and the 4-bit scale s of that sub-block: weight = d*(1+2s) * mag * sign.
void fbo_dequant_iq3_s(const void* blocks, float* y, int64_t k) {
  grid_init();
  const fbo_iq3s* x = (const fbo_iq3s*)blocks;
  for (int64_t b = 0; b < k / 256; ++b) {
    const float d = fbo_fp16_to_fp32(x[b].d);
    for (int ib = 0; ib < 8; ++ib) {
      const int s = (x[b].scales[ib / 2] >> (4 * (ib & 1))) & 0xF;
      const float db = d * (float)(1 + 2 * s);
      for (int l = 0; l < 8; ++l) {
        const int idx = x[b].qs[8 * ib + l] | (((x[b].qh[ib] >> l) & 1) << 8);
        const uint8_t sg = x[b].signs[4 * ib + l / 2];
        for (int j = 0; j < 4; ++j) {
          const int bit = 4 * (l & 1) + j;
          *y++ = db * (float)g_grid[idx][j] * (((sg >> bit) & 1) ? -1.f : 1.f);
        }
      }
    }
  }
}

// third_party/ggml-iq/ggml-iq.c:272-288: low nibbles are elements 0..15, high nibbles 16..31.
void fbo_dequant_iq4_nl(const void* blocks, float* y, int64_t k) {
  const fbo_iq4nl* x = (const fbo_iq4nl*)blocks;
  for (int64_t b = 0; b < k / 32; ++b) {
    const float d = fbo_fp16_to_fp32(x[b].d);
    for (int j = 0; j < 16; ++j) {
      y[j] = d * (float)kIq4nlLevels[x[b].qs[j] & 0xF];
      y[j + 16] = d * (float)kIq4nlLevels[x[b].qs[j] >> 4];
    }
    y += 32;
  }
}

// third_party/ggml-iq/ggml-iq.c:171-199: sub-block ib uses qs[4ib..4ib+3] with two more index bits each from
// qh[ib], signs qs[32+4ib..], and two 4-bit scales (first / second 16 weights): d*(0.5+s)*0.25.
void fbo_dequant_iq2_s(const void* blocks, float* y, int64_t k) {
  grid_init();
  const fbo_iq2s* x = (const fbo_iq2s*)blocks;
  for (int64_t b = 0; b < k / 256; ++b) {
    const float d = fbo_fp16_to_fp32(x[b].d);
    for (int ib = 0; ib < 8; ++ib) {
      float db[2];
      db[0] = d * (0.5f + (float)(x[b].scales[ib] & 0xF)) * 0.25f;
      db[1] = d * (0.5f + (float)(x[b].scales[ib] >> 4)) * 0.25f;
      for (int l = 0; l < 4; ++l) {
        const int idx = x[b].qs[4 * ib + l] | ((x[b].qh[ib] << (8 - 2 * l)) & 0x300);
        const uint8_t sg = x[b].qs[32 + 4 * ib + l];
        for (int j = 0; j < 8; ++j) *y++ = db[l / 2] * (float)g_grid2s[idx][j] * (((sg >> j) & 1) ? -1.f : 1.f);
      }
    }
  }
}

// :201-229: sub-block ib uses qs[8ib..8ib+7] (entries of four weights) and the word qs[64+4ib..]: four
// 7-bit sign indices and a 4-bit scale in the top bits: d*(0.5+s)*0.5.
void fbo_dequant_iq3_xxs(const void* blocks, float* y, int64_t k) {
  grid_init();
  const fbo_iq3xxs* x = (const fbo_iq3xxs*)blocks;
  for (int64_t b = 0; b < k / 256; ++b) {
    const float d = fbo_fp16_to_fp32(x[b].d);
    for (int ib = 0; ib < 8; ++ib) {
      uint32_t aux;
      memcpy(&aux, x[b].qs + 64 + 4 * ib, 4);
      const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
      for (int l = 0; l < 4; ++l) {
        const uint8_t sg = ksigns((aux >> (7 * l)) & 127);
        const uint8_t* g1 = g_grid3xxs[x[b].qs[8 * ib + 2 * l]];
        const uint8_t* g2 = g_grid3xxs[x[b].qs[8 * ib + 2 * l + 1]];
        for (int j = 0; j < 4; ++j) y[j] = db * (float)g1[j] * (((sg >> j) & 1) ? -1.f : 1.f);
        for (int j = 0; j < 4; ++j) y[j + 4] = db * (float)g2[j] * (((sg >> (j + 4)) & 1) ? -1.f : 1.f);
        y += 8;
      }
    }
  }
}

// :290-311: sub-block ib: 6-bit scale ls (4 bits from scales_l, 2 from scales_h), d*(ls-32); nibbles index
// the IQ4_NL levels, low nibbles first.
void fbo_dequant_iq4_xs(const void* blocks, float* y, int64_t k) {
  const fbo_iq4xs* x = (const fbo_iq4xs*)blocks;
  for (int64_t b = 0; b < k / 256; ++b) {
    const float d = fbo_fp16_to_fp32(x[b].d);
    for (int ib = 0; ib < 8; ++ib) {
      const int ls = ((x[b].scales_l[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((x[b].scales_h >> (2 * ib)) & 3) << 4);
      const float dl = d * (float)(ls - 32);
      const uint8_t* qs = x[b].qs + 16 * ib;
      for (int j = 0; j < 16; ++j) {
        y[j] = dl * (float)kIq4nlLevels[qs[j] & 0xF];
        y[j + 16] = dl * (float)kIq4nlLevels[qs[j] >> 4];
      }
      y += 32;
    }
  }
}

// :135-152: 64 two-bit codes, LSB first, value (q - 1) * d.
void fbo_dequant_q2_0(const void* blocks, float* y, int64_t k) {
  const fbo_q20* x = (const fbo_q20*)blocks;
  for (int64_t b = 0; b < k / 64; ++b) {
    const float d = fbo_fp16_to_fp32(x[b].d);
    for (int j = 0; j < 64; ++j) *y++ = (float)((int)((x[b].qs[j / 4] >> ((j % 4) * 2)) & 3) - 1) * d;
  }
}

void fbo_dequant_rows(int fmt, const void* rows, int64_t row_bytes, int nrows, int k, float* y) {
  for (int r = 0; r < nrows; ++r) {
    const uint8_t* p = (const uint8_t*)rows + (int64_t)r * row_bytes;
    float* o = y + (int64_t)r * k;
    if (fmt == FBO_IQ3_S) fbo_dequant_iq3_s(p, o, k);
    else if (fmt == FBO_IQ4_NL) fbo_dequant_iq4_nl(p, o, k);
    else if (fmt == FBO_IQ2_S) fbo_dequant_iq2_s(p, o, k);
    else if (fmt == FBO_IQ3_XXS) fbo_dequant_iq3_xxs(p, o, k);
    else if (fmt == FBO_IQ4_XS) fbo_dequant_iq4_xs(p, o, k);
    else fbo_dequant_q2_0(p, o, k);
  }
}

// Exact integer weights of one 256-block of the other Q8_K formats, the integer multiplier of each of the
// 16 lanes (elements 16j..16j+15) and the block's float factor, as the CPU tier's decoders leave them
// (src/cpu/iq_cpu.cpp:166-217 iq2_s and iq3_xxs, :238-255 iq4_xs): F_j = float(mult_j) * dprime.
static void int_weights_q8k(int fmt, const void* block, int8_t* w /*256*/, int* mult /*16*/, float* dprime) {
  grid_init();
  if (fmt == FBO_IQ2_S) {
    const fbo_iq2s* x = (const fbo_iq2s*)block;
    *dprime = fbo_fp16_to_fp32(x->d) * 0.125f;
    for (int ib = 0; ib < 8; ++ib) {
      mult[2 * ib] = 2 * (x->scales[ib] & 0xF) + 1;
      mult[2 * ib + 1] = 2 * (x->scales[ib] >> 4) + 1;
      for (int l = 0; l < 4; ++l) {
        const int idx = x->qs[4 * ib + l] | ((x->qh[ib] << (8 - 2 * l)) & 0x300);
        const uint8_t sg = x->qs[32 + 4 * ib + l];
        for (int j = 0; j < 8; ++j) {
          const int m = g_grid2s[idx][j];
          w[32 * ib + 8 * l + j] = (int8_t)(((sg >> j) & 1) ? -m : m);
        }
      }
    }
  } else if (fmt == FBO_IQ3_XXS) {
    const fbo_iq3xxs* x = (const fbo_iq3xxs*)block;
    *dprime = fbo_fp16_to_fp32(x->d) * 0.25f;
    for (int ib = 0; ib < 8; ++ib) {
      uint32_t aux;
      memcpy(&aux, x->qs + 64 + 4 * ib, 4);
      mult[2 * ib] = mult[2 * ib + 1] = 2 * (int)(aux >> 28) + 1;
      for (int l = 0; l < 4; ++l) {
        const uint8_t sg = ksigns((aux >> (7 * l)) & 127);
        for (int h = 0; h < 2; ++h)
          for (int j = 0; j < 4; ++j) {
            const int m = g_grid3xxs[x->qs[8 * ib + 2 * l + h]][j];
            w[32 * ib + 8 * l + 4 * h + j] = (int8_t)(((sg >> (4 * h + j)) & 1) ? -m : m);
          }
      }
    }
  } else {  // IQ4_XS
    const fbo_iq4xs* x = (const fbo_iq4xs*)block;
    *dprime = fbo_fp16_to_fp32(x->d);
    for (int ib = 0; ib < 8; ++ib) {
      const int ls = ((x->scales_l[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((x->scales_h >> (2 * ib)) & 3) << 4);
      mult[2 * ib] = mult[2 * ib + 1] = ls - 32;
      for (int j = 0; j < 16; ++j) {
        w[32 * ib + j] = kIq4nlLevels[x->qs[16 * ib + j] & 0xF];
        w[32 * ib + 16 + j] = kIq4nlLevels[x->qs[16 * ib + j] >> 4];
      }
    }
  }
}

// Exact integer weights of one row and the per-32 float scale: the form both CPU and GPU
// integer paths consume (src/cpu/iq_cpu.cpp:219-237, :264-277).
static void int_weights_iq3s(const fbo_iq3s* x, int8_t* w /*256*/, float* f /*8*/) {
  grid_init();
  const float d = fbo_fp16_to_fp32(x->d);
  for (int ib = 0; ib < 8; ++ib) {
    const int s = (x->scales[ib / 2] >> (4 * (ib & 1))) & 0xF;
    f[ib] = d * (float)(1 + 2 * s);
    for (int l = 0; l < 8; ++l) {
      const int idx = x->qs[8 * ib + l] | (((x->qh[ib] >> l) & 1) << 8);
      const uint8_t sg = x->signs[4 * ib + l / 2];
      for (int j = 0; j < 4; ++j) {
        const int bit = 4 * (l & 1) + j;
        const int m = g_grid[idx][j];
        w[32 * ib + 4 * l + j] = (int8_t)(((sg >> bit) & 1) ? -m : m);
      }
    }
  }
}

// ---------------------------------------------------------------------------------- quantize
// third_party/ggml-iq/ggml-iq.c:313-350 with the CPU tier's one deliberate change (an all-zero
// block also gets bsums = 0, src/cpu/q8_cpu.h:7-8). max = FIRST element of largest magnitude;
// q = min(127, rne(iscale*x)); d = 1/iscale.
void fbo_quantize_q8_K(const float* x, void* out, int64_t k) {
  fbo_q8k* y = (fbo_q8k*)out;
  for (int64_t b = 0; b < k / 256; ++b, x += 256) {
    float max = 0, amax = 0;
    for (int j = 0; j < 256; ++j) {
      const float ax = fabsf(x[j]);
      if (ax > amax) { amax = ax; max = x[j]; }
    }
    if (!amax) {
      memset(&y[b], 0, sizeof(fbo_q8k));
      continue;
    }
    const float iscale = -127.f / max;
    for (int j = 0; j < 256; ++j) {
      int v = (int)nearbyintf(iscale * x[j]);
      y[b].qs[j] = (int8_t)(v < 127 ? v : 127);
    }
    for (int j = 0; j < 16; ++j) {
      int sum = 0;
      for (int i = 0; i < 16; ++i) sum += y[b].qs[16 * j + i];
      y[b].bsums[j] = (int16_t)sum;
    }
    y[b].d = 1 / iscale;
  }
}

// third_party/ggml-iq/ggml-iq.c:75-98: d = amax/127 (stored fp16), id = 1/d in fp32, roundf.
void fbo_quantize_q8_0(const float* x, void* out, int64_t k) {
  fbo_q80* y = (fbo_q80*)out;
  for (int64_t b = 0; b < k / 32; ++b, x += 32) {
    float amax = 0.0f;
    for (int j = 0; j < 32; ++j) {
      const float a = fabsf(x[j]);
      if (a > amax) amax = a;
    }
    const float d = amax / 127;
    const float id = d ? 1.0f / d : 0.0f;
    y[b].d = fbo_fp32_to_fp16(d);
    for (int j = 0; j < 32; ++j) y[b].qs[j] = (int8_t)roundf(x[j] * id);
  }
}

void fbo_quantize_act(int act, const float* x, void* out, int64_t k) {
  if (act == FBO_ACT_Q8_K) fbo_quantize_q8_K(x, out, k);
  else fbo_quantize_q8_0(x, out, k);
}
int64_t fbo_act_row_bytes(int act, int k) {
  return act == FBO_ACT_Q8_K ? (int64_t)(k / 256) * 292 : (int64_t)(k / 32) * 34;
}

// ---------------------------------------------------------------------------------- dot
// Lane-wise sum in the order of the 16-lane horizontal add the CPU tier ends with
// (src/cpu/iq_cpu.cpp:373): halves, quarters, then the two crossed pairs.
static float hsum16(const float* a) {
  float t8[8], t4[4];
  for (int i = 0; i < 8; ++i) t8[i] = a[i + 8] + a[i];
  for (int i = 0; i < 4; ++i) t4[i] = t8[i + 4] + t8[i];
  const float p0 = t4[0] + t4[2], p1 = t4[1] + t4[3];
  return p0 + p1;
}

// One IQ3_S row against one Q8_K activation row, in the arithmetic of the CPU tier's micro-kernel
// (src/cpu/iq_cpu.cpp:332-374 over the layout of :219-237): per 256-block, lane j sums the 16
// products of elements 16j..16j+15 exactly in int32, then acc_j = fma(float(isum_j), F_j*dA, acc_j)
// with F_j = d*(1+2*s[j/2]); the 16 lanes are added at the end.
float fbo_dot_iq3_s_q8_K(int n, const void* wrow, const void* arow) {
  const fbo_iq3s* w = (const fbo_iq3s*)wrow;
  const fbo_q8k* a = (const fbo_q8k*)arow;
  float acc[16] = {0};
  int8_t iw[256];
  float f[8];
  for (int b = 0; b < n / 256; ++b) {
    int_weights_iq3s(&w[b], iw, f);
    for (int j = 0; j < 16; ++j) {
      int32_t isum = 0;
      for (int i = 0; i < 16; ++i) isum += (int32_t)iw[16 * j + i] * a[b].qs[16 * j + i];
      const float s = f[j / 2] * a[b].d;
      acc[j] = fmaf((float)isum, s, acc[j]);
    }
  }
  return hsum16(acc);
}

// One IQ4_NL row against one Q8_0 row (src/cpu/iq_cpu.cpp:264-277, :311-319): groups of two
// 32-blocks; lane j of lanes 0-7 covers elements 4j..4j+3 of the first block, lanes 8-15 the
// second; scale = fp16 weight d * fp16 activation d, both widened to fp32. An odd trailing block
// leaves lanes 8-15 with zero weights and a zero scale.
float fbo_dot_iq4_nl_q8_0(int n, const void* wrow, const void* arow) {
  const fbo_iq4nl* w = (const fbo_iq4nl*)wrow;
  const fbo_q80* a = (const fbo_q80*)arow;
  float acc[16] = {0};
  const int nb = n / 32;
  for (int b = 0; b < nb; ++b) {
    const float s = fbo_fp16_to_fp32(w[b].d) * fbo_fp16_to_fp32(a[b].d);
    int8_t iw[32];
    for (int j = 0; j < 16; ++j) {
      iw[j] = kIq4nlLevels[w[b].qs[j] & 0xF];
      iw[j + 16] = kIq4nlLevels[w[b].qs[j] >> 4];
    }
    for (int j = 0; j < 8; ++j) {
      int32_t isum = 0;
      for (int i = 0; i < 4; ++i) isum += (int32_t)iw[4 * j + i] * a[b].qs[4 * j + i];
      float* lane = &acc[8 * (b & 1) + j];
      *lane = fmaf((float)isum, s, *lane);
    }
    if ((b & 1) == 0 && b + 1 == nb)  // padded half group: fma(0, 0, acc) keeps acc (and -0 -> +0 never matters)
      for (int j = 8; j < 16; ++j) acc[j] = fmaf(0.0f, 0.0f, acc[j]);
  }
  return hsum16(acc);
}

// The other Q8_K formats in the same micro-kernel arithmetic (src/cpu/iq_cpu.cpp:332-374): per lane
// acc_j = fma(float(isum_j), F_j * dA, acc_j), F_j = float(mult_j) * dprime.
static float dot_q8k_generic(int fmt, int n, const void* wrow, const void* arow) {
  const uint8_t* w = (const uint8_t*)wrow;
  const int64_t bb = fbo_row_bytes(fmt, 256);
  const fbo_q8k* a = (const fbo_q8k*)arow;
  float acc[16] = {0};
  int8_t iw[256];
  int mult[16];
  float dp;
  for (int b = 0; b < n / 256; ++b) {
    int_weights_q8k(fmt, w + b * bb, iw, mult, &dp);
    for (int j = 0; j < 16; ++j) {
      int32_t isum = 0;
      for (int i = 0; i < 16; ++i) isum += (int32_t)iw[16 * j + i] * a[b].qs[16 * j + i];
      const float f = (float)mult[j] * dp;
      acc[j] = fmaf((float)isum, f * a[b].d, acc[j]);
    }
  }
  return hsum16(acc);
}

// Q2_0 against Q8_0 (src/cpu/iq_cpu.cpp:279-287, :311-319): a group is one 64-element weight block and two
// activation blocks; lanes 0-7 cover the first 32 elements (four each), lanes 8-15 the second; F = the block's
// d in every lane, dA = the lane's activation block scale.
static float dot_q2_0_q8_0(int n, const void* wrow, const void* arow) {
  const fbo_q20* w = (const fbo_q20*)wrow;
  const fbo_q80* a = (const fbo_q80*)arow;
  float acc[16] = {0};
  for (int g = 0; g < n / 64; ++g) {
    const float d = fbo_fp16_to_fp32(w[g].d);
    for (int j = 0; j < 16; ++j) {
      const fbo_q80* ab = &a[2 * g + j / 8];
      int32_t isum = 0;
      for (int i = 0; i < 4; ++i) {
        const int e = 4 * j + i;
        isum += ((int32_t)((w[g].qs[e / 4] >> ((e % 4) * 2)) & 3) - 1) * ab->qs[4 * (j % 8) + i];
      }
      acc[j] = fmaf((float)isum, d * fbo_fp16_to_fp32(ab->d), acc[j]);
    }
  }
  return hsum16(acc);
}

float fbo_dot(int fmt, int n, const void* wrow, const void* arow) {
  if (fmt == FBO_IQ3_S) return fbo_dot_iq3_s_q8_K(n, wrow, arow);
  if (fmt == FBO_IQ4_NL) return fbo_dot_iq4_nl_q8_0(n, wrow, arow);
  if (fmt == FBO_Q2_0) return dot_q2_0_q8_0(n, wrow, arow);
  return dot_q8k_generic(fmt, n, wrow, arow);
}

// ---------------------------------------------------------------------------------- SwiGLU
// src/cpu/iq_cpu.cpp:413-428 (Cephes expf with fused steps) and :794-803:
// h = (g / (1 + exp(-g))) * u.
static float exp_cephes(float x) {
  x = fminf(fmaxf(x, -103.0f), 88.5f);
  const float n = nearbyintf(x * 1.44269504088896341f);
  float r = fmaf(-n, 0.693359375f, x);
  r = fmaf(-n, -2.12194440e-4f, r);
  float y = 1.9875691500e-4f;
  y = fmaf(y, r, 1.3981999507e-3f);
  y = fmaf(y, r, 8.3334519073e-3f);
  y = fmaf(y, r, 4.1665795894e-2f);
  y = fmaf(y, r, 1.6666665459e-1f);
  y = fmaf(y, r, 5.0000001201e-1f);
  y = fmaf(y, r * r, r + 1.0f);
  return ldexpf(y, (int)n);
}
void fbo_silu_mul(const float* g, const float* u, float* h, int n) {
  for (int i = 0; i < n; ++i) {
    const float e = exp_cephes(0.0f - g[i]);
    const float s = g[i] / (1.0f + e);
    h[i] = s * u[i];
  }
}

// ---------------------------------------------------------------------------------- expert FFN
// One expert over T tokens in the decode numerics ("family Q"): the phase order of
// src/cpu/expert_pool.cpp:330-408 -- activations quantized once per token, gate/up dots, SwiGLU,
// h re-quantized in the activation format the down format pairs with, down dots. Outputs are
// unweighted: h [T][inter], y [T][hidden].
void fbo_expert_ffn(int fmt_gu, int fmt_down, int hidden, int inter, const uint8_t* gate,
                    const uint8_t* up, const uint8_t* down, const float* x, int T, float* h_out,
                    float* y_out) {
  const int act_gu = fbo_act_of(fmt_gu), act_dn = fbo_act_of(fmt_down);
  const int64_t rb_gu = fbo_row_bytes(fmt_gu, hidden), rb_dn = fbo_row_bytes(fmt_down, inter);
  uint8_t* xq = (uint8_t*)malloc((size_t)fbo_act_row_bytes(act_gu, hidden));
  uint8_t* hq = (uint8_t*)malloc((size_t)fbo_act_row_bytes(act_dn, inter));
  float* g = (float*)malloc(sizeof(float) * (size_t)inter * 3);
  float *u = g + inter, *h = u + inter;
  for (int t = 0; t < T; ++t) {
    fbo_quantize_act(act_gu, x + (int64_t)t * hidden, xq, hidden);
    for (int j = 0; j < inter; ++j) {
      g[j] = fbo_dot(fmt_gu, hidden, gate + j * rb_gu, xq);
      u[j] = fbo_dot(fmt_gu, hidden, up + j * rb_gu, xq);
    }
    fbo_silu_mul(g, u, h, inter);
    if (h_out) memcpy(h_out + (int64_t)t * inter, h, sizeof(float) * (size_t)inter);
    fbo_quantize_act(act_dn, h, hq, inter);
    for (int n = 0; n < hidden; ++n) y_out[(int64_t)t * hidden + n] = fbo_dot(fmt_down, inter, down + n * rb_dn, hq);
  }
  free(xq);
  free(hq);
  free(g);
}

// ---------------------------------------------------------------------------------- router
// Top-k of n logits: value descending, ties to the lower id, NaN never wins, -0 == +0; weights =
// softmax restricted to the k winners in fp32, exp(v - top), summed in rank order, multiplied by
// 1/sum (src/kernels/moe/moe_common.cuh:33-85; tests/kernels/moe/moe_test_common.h:50-65).
void fbo_topk(const float* logits, int n, int k, int32_t* ids, float* weights) {
  uint8_t* taken = (uint8_t*)calloc((size_t)n, 1);
  float vals[64];
  for (int r = 0; r < k; ++r) {
    int best = -1;
    float bv = 0;
    for (int i = 0; i < n; ++i) {
      if (taken[i]) continue;
      float v = logits[i];
      if (v != v) v = -INFINITY;
      if (best < 0 || v > bv) { best = i; bv = v; }
    }
    taken[best] = 1;
    ids[r] = best;
    vals[r] = bv;
  }
  float sum = 0.f;
  const float top = vals[0];
  for (int r = 0; r < k; ++r) { vals[r] = expf(vals[r] - top); sum += vals[r]; }
  const float inv = 1.0f / sum;
  for (int r = 0; r < k; ++r) weights[r] = vals[r] * inv;
  free(taken);
}

// ---------------------------------------------------------------------------------- MoE layer
// y[t] = sum over token t's experts in ASCENDING EXPERT ID of w * ffn_e(x_t): the deterministic
// order of the CPU tier (src/cpu/expert_pool.cpp:381-403) and of the GPU decode combine when
// slot == expert id (src/kernels/moe/moe.h:91-94). Expert e's blob is blobs + e*blob_stride with
// gate | up | down back to back (src/kernels/moe/moe_format.cpp:26-38, any `inter`).
typedef struct {
  int fmt_gu, fmt_down, hidden, inter, T, k;
  const uint8_t* blobs;
  int64_t blob_stride;
  const float* x;
  const int32_t* ids;
  const float* w;
  float* y;
  int t0, t1;
} layer_job;

static void* layer_worker(void* p) {
  layer_job* j = (layer_job*)p;
  const int64_t gate_bytes = (int64_t)j->inter * fbo_row_bytes(j->fmt_gu, j->hidden);
  float* ye = (float*)malloc(sizeof(float) * (size_t)j->hidden);
  for (int t = j->t0; t < j->t1; ++t) {
    int order[64];
    for (int r = 0; r < j->k; ++r) order[r] = r;
    for (int a = 1; a < j->k; ++a)  // insertion sort by expert id
      for (int b = a; b > 0 && j->ids[t * j->k + order[b]] < j->ids[t * j->k + order[b - 1]]; --b) {
        const int tmp = order[b]; order[b] = order[b - 1]; order[b - 1] = tmp;
      }
    float* y = j->y + (int64_t)t * j->hidden;
    for (int n = 0; n < j->hidden; ++n) y[n] = 0.0f;
    for (int r = 0; r < j->k; ++r) {
      const int e = j->ids[t * j->k + order[r]];
      const float w = j->w[t * j->k + order[r]];
      const uint8_t* blob = j->blobs + (int64_t)e * j->blob_stride;
      fbo_expert_ffn(j->fmt_gu, j->fmt_down, j->hidden, j->inter, blob, blob + gate_bytes,
                     blob + 2 * gate_bytes, j->x + (int64_t)t * j->hidden, 1, NULL, ye);
      // fused multiply-add: what GCC emits for the pool's `yb += pw * o` at the reference's
      // -O3 -march=native with its default contraction (src/cpu/expert_pool.cpp:399-403)
      for (int n = 0; n < j->hidden; ++n) y[n] = fmaf(w, ye[n], y[n]);
    }
  }
  free(ye);
  return NULL;
}

void fbo_moe_layer(int fmt_gu, int fmt_down, int hidden, int inter, const uint8_t* blobs,
                   int64_t blob_stride, const float* x, int T, int k, const int32_t* ids,
                   const float* w, float* y, int threads) {
  if (threads < 1) threads = 1;
  if (threads > T) threads = T;
  pthread_t th[64];
  layer_job jobs[64];
  if (threads > 64) threads = 64;
  for (int i = 0; i < threads; ++i) {
    layer_job j = {fmt_gu, fmt_down, hidden, inter, T, k, blobs, blob_stride, x, ids, w, y,
                   (int)((int64_t)T * i / threads), (int)((int64_t)T * (i + 1) / threads)};
    jobs[i] = j;
    pthread_create(&th[i], NULL, layer_worker, &jobs[i]);
  }
  for (int i = 0; i < threads; ++i) pthread_join(th[i], NULL);
}

// ---------------------------------------------------------------------------------- prefill numerics
// "Family B" (src/cpu/iq_cpu.cpp:712-792, src/cpu/expert_pool.cpp:341-347,364-367,390-393):
// weights = bf16_rne(exact dequant), activations bf16, fp32 accumulation, h rounded to bf16
// between the two products. Returns unweighted y [T][hidden]; x is raw bf16 bits.
void fbo_dequant_rows_bf16(int fmt, const void* rows, int64_t row_bytes, int nrows, int k, uint16_t* y) {
  float* tmp = (float*)malloc(sizeof(float) * (size_t)k);
  for (int r = 0; r < nrows; ++r) {
    fbo_dequant_rows(fmt, (const uint8_t*)rows + (int64_t)r * row_bytes, row_bytes, 1, k, tmp);
    for (int i = 0; i < k; ++i) y[(int64_t)r * k + i] = fbo_fp32_to_bf16(tmp[i]);
  }
  free(tmp);
}

static float dot_bf16(const uint16_t* w, const uint16_t* a, int k) {
  // 16 fp32 lanes, each taking pairs (2i, 2i+1) of every 32-element step, then the lane add:
  // the accumulation shape of the reference's bf16 micro-kernel (src/cpu/iq_cpu.cpp:757-770).
  float acc[16] = {0};
  for (int i = 0; i < k; i += 32)
    for (int l = 0; l < 16; ++l) {
      const float p0 = fbo_bf16_to_fp32(w[i + 2 * l]) * fbo_bf16_to_fp32(a[i + 2 * l]);
      const float p1 = fbo_bf16_to_fp32(w[i + 2 * l + 1]) * fbo_bf16_to_fp32(a[i + 2 * l + 1]);
      acc[l] = acc[l] + p0 + p1;
    }
  return hsum16(acc);
}

void fbo_expert_ffn_bf16(int fmt_gu, int fmt_down, int hidden, int inter, const uint8_t* gate,
                         const uint8_t* up, const uint8_t* down, const uint16_t* x, int T,
                         uint16_t* h_out, float* y_out) {
  const int64_t rb_gu = fbo_row_bytes(fmt_gu, hidden), rb_dn = fbo_row_bytes(fmt_down, inter);
  uint16_t* wg = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)hidden * inter * 3);
  uint16_t *wu = wg + (size_t)hidden * inter, *wd = wu + (size_t)hidden * inter;
  fbo_dequant_rows_bf16(fmt_gu, gate, rb_gu, inter, hidden, wg);
  fbo_dequant_rows_bf16(fmt_gu, up, rb_gu, inter, hidden, wu);
  fbo_dequant_rows_bf16(fmt_down, down, rb_dn, hidden, inter, wd);
  float* g = (float*)malloc(sizeof(float) * (size_t)inter * 3);
  float *u = g + inter, *h = u + inter;
  uint16_t* hb = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)inter);
  for (int t = 0; t < T; ++t) {
    const uint16_t* xt = x + (int64_t)t * hidden;
    for (int j = 0; j < inter; ++j) {
      g[j] = dot_bf16(wg + (size_t)j * hidden, xt, hidden);
      u[j] = dot_bf16(wu + (size_t)j * hidden, xt, hidden);
    }
    fbo_silu_mul(g, u, h, inter);
    for (int j = 0; j < inter; ++j) hb[j] = fbo_fp32_to_bf16(h[j]);
    if (h_out) memcpy(h_out + (int64_t)t * inter, hb, sizeof(uint16_t) * (size_t)inter);
    for (int n = 0; n < hidden; ++n) y_out[(int64_t)t * hidden + n] = dot_bf16(wd + (size_t)n * inter, hb, inter);
  }
  free(wg);
  free(g);
  free(hb);
}

// The down projection alone in the prefill numerics, from given bf16 h rows (raw bits): lets a test
// separate "h is within one bf16 step" from "the down GEMM is right for the h it was given", as the
// reference's own prefill test does (tests/kernels/moe/test_moe_experts.cpp:426-488).
void fbo_down_bf16(int fmt_down, int hidden, int inter, const uint8_t* down, const uint16_t* h, int T,
                   float* y_out) {
  const int64_t rb = fbo_row_bytes(fmt_down, inter);
  uint16_t* wd = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)hidden * inter);
  fbo_dequant_rows_bf16(fmt_down, down, rb, hidden, inter, wd);
  for (int t = 0; t < T; ++t)
    for (int n = 0; n < hidden; ++n)
      y_out[(int64_t)t * hidden + n] = dot_bf16(wd + (size_t)n * inter, h + (int64_t)t * inter, inter);
  free(wd);
}

// ---------------------------------------------------------------------------------- FP8 rows
// E4M3FN code -> float: tests/common/test_util.h:105-112 (0x7F / 0xFF are NaN).
float fbo_e4m3_to_float(uint8_t code) {
  const int sign = code >> 7, e = (code >> 3) & 0xF, m = code & 7;
  float v;
  if (e == 0xF && m == 7) return NAN;
  if (e == 0) v = ldexpf((float)m / 8.0f, -6);
  else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return sign ? -v : v;
}
// Saturating round-to-nearest-even float -> E4M3FN (tests/kernels/linear/linear_ref.h:49-70,
// the host statement of cvt.rn.satfinite.e4m3x2.f32).
uint8_t fbo_e4m3_satfinite(float v) {
  float mag = fabsf(v);
  if (!(mag <= 448.0f)) mag = 448.0f;  // also sends NaN to the maximum, as satfinite does
  int lo = 0, hi = 0x7E;               // largest code with value <= mag
  while (lo < hi) {
    const int mid = (lo + hi + 1) / 2;
    if (fbo_e4m3_to_float((uint8_t)mid) <= mag) lo = mid; else hi = mid - 1;
  }
  int code = lo;
  if (lo < 0x7E) {
    const float dl = mag - fbo_e4m3_to_float((uint8_t)lo), du = fbo_e4m3_to_float((uint8_t)(lo + 1)) - mag;
    if (du < dl || (du == dl && ((lo + 1) & 1) == 0)) code = lo + 1;
  }
  return (uint8_t)(code | (signbit(v) ? 0x80 : 0));
}
// Per-token activation quantization of the E4M3-activation path
// (src/kernels/linear/fp8/fp8_a8_quantize.cuh:14-26; tests/kernels/linear/linear_ref.h:99-107):
// scale = max|x|/448, codes = satfinite(x * (1/scale)). x: raw bf16 bits. Returns the scale.
float fbo_quantize_token_e4m3(const uint16_t* x, int64_t k, uint8_t* codes) {
  float mx = 0.0f;
  for (int64_t j = 0; j < k; ++j) mx = fmaxf(mx, fabsf(fbo_bf16_to_fp32(x[j])));
  const float scale = mx > 0.0f ? mx / 448.0f : 0.0f;
  const float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
  for (int64_t j = 0; j < k; ++j) codes[j] = fbo_e4m3_satfinite(fbo_bf16_to_fp32(x[j]) * inv);
  return scale;
}

// The exact-activation route of this repository's FP8-row GEMM above 16 tokens (no counterpart in the
// reference, whose bf16-activation GEMM widens the weights instead): a token is scaled by the power of
// two that puts its largest magnitude in [128, 256) and every value is written as hi + lo with
// hi = rne_e4m3(v), lo = rne_e4m3(v - hi). x: raw bf16 bits. Returns the scale (0 for a row of zeros or
// non-finite values: all codes 0).
float fbo_split_token_e4m3x2(const uint16_t* x, int64_t k, uint8_t* hi, uint8_t* lo) {
  float mx = 0.0f;
  for (int64_t j = 0; j < k; ++j) mx = fmaxf(mx, fabsf(fbo_bf16_to_fp32(x[j])));
  int e = 0;
  float scale = 0.0f, inv = 0.0f;
  if (mx > 0.0f && isfinite(mx)) {
    (void)frexpf(mx, &e);  // mx = f * 2^e, f in [0.5, 1): 2^(e-1) <= mx < 2^e
    e -= 1;
    if (e - 7 >= -126 && 7 - e >= -126) {
      scale = ldexpf(1.0f, e - 7);
      inv = ldexpf(1.0f, 7 - e);
    }
  }
  for (int64_t j = 0; j < k; ++j) {
    const float v = fbo_bf16_to_fp32(x[j]) * inv;
    hi[j] = fbo_e4m3_satfinite(v);
    lo[j] = fbo_e4m3_satfinite(v - fbo_e4m3_to_float(hi[j]));
  }
  return scale;
}

// FP8-row pack rule: how a bf16 weight matrix becomes E4M3FN codes + one bf16 scale per row
// (tools/fp8row.py:21-44 quantize_rows; host port tests/kernels/linear/linear_ref.h:72-97):
//   scale = bf16_rne(float(double(max|row|) / 448)), a scale that rounds to zero becomes the smallest
//   positive bf16 (word 0x0001), an all-zero row gets scale 0 and codes 0;
//   code = e4m3_rne(clamp(float(double(x) * double(float(1 / double(scale)))), -448, 448)).
// weight: raw bf16 bits [n][k]; scales: raw bf16 bits [n].
void fbo_quantize_fp8_rows(const uint16_t* weight, int64_t n, int64_t k, uint8_t* codes, uint16_t* scales) {
  for (int64_t r = 0; r < n; ++r) {
    const uint16_t* row = weight + r * k;
    uint8_t* out = codes + r * k;
    float mx = 0.0f;
    for (int64_t j = 0; j < k; ++j) mx = fmaxf(mx, fabsf(fbo_bf16_to_fp32(row[j])));
    if (mx == 0.0f) {
      memset(out, 0, (size_t)k);
      scales[r] = 0;
      continue;
    }
    const float raw = (float)((double)mx / 448.0);
    uint32_t bits;
    memcpy(&bits, &raw, 4);
    uint16_t word = (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
    if (word == 0) word = 1;
    scales[r] = word;
    const float scale = fbo_bf16_to_fp32(word);
    const float recip = (float)(1.0 / (double)scale);
    for (int64_t j = 0; j < k; ++j) {
      float v = (float)((double)fbo_bf16_to_fp32(row[j]) * (double)recip);
      v = fminf(448.0f, fmaxf(-448.0f, v));
      out[j] = fbo_e4m3_satfinite(v);
    }
  }
}

