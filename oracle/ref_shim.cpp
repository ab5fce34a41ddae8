// TEST INFRASTRUCTURE ONLY. C-linkage shim over the reference's own CPU expert path so that the
// test suite and the CPU-baseline leg of the benchmark can call it through ctypes. This file holds
// no algorithm: every function forwards to the reference sources, which the recipe in
// oracle/build_ref.py compiles in place from the reference checkout (never copied here).
//   fngine::cpu::*          src/cpu/iq_cpu.h:54-111, src/cpu/q8_cpu.h:16-21
//   ggml reference routines third_party/ggml-iq/ggml-iq.h:203-226
#include "cpu/iq_cpu.h"
#include "cpu/q8_cpu.h"

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

using namespace fngine::cpu;

extern "C" {

int ref_format_info(int fmt, int* block_elems, int* block_bytes, int* act) {
  try {
    const FormatInfo fi = format_info(WeightFormat(fmt));
    *block_elems = fi.block_elems;
    *block_bytes = fi.block_bytes;
    *act = int(fi.act);
    return 0;
  } catch (...) {
    return -1;
  }
}

// ggml reference dequantizers (ground truth for the bit-exact weight gate).
void ref_dequant_iq3_s(const void* blocks, float* y, int64_t k) {
  dequantize_row_iq3_s(static_cast<const block_iq3_s*>(blocks), y, k);
}
void ref_dequant_iq4_nl(const void* blocks, float* y, int64_t k) {
  dequantize_row_iq4_nl(static_cast<const block_iq4_nl*>(blocks), y, k);
}
// any of the six expert formats by its ggml type id; returns 0 for an id it does not know
int ref_dequant(int fmt, const void* blocks, float* y, int64_t k) {
  switch (fmt) {
    case 18: dequantize_row_iq3_xxs(static_cast<const block_iq3_xxs*>(blocks), y, k); return 1;
    case 20: dequantize_row_iq4_nl(static_cast<const block_iq4_nl*>(blocks), y, k); return 1;
    case 21: dequantize_row_iq3_s(static_cast<const block_iq3_s*>(blocks), y, k); return 1;
    case 22: dequantize_row_iq2_s(static_cast<const block_iq2_s*>(blocks), y, k); return 1;
    case 23: dequantize_row_iq4_xs(static_cast<const block_iq4_xs*>(blocks), y, k); return 1;
    case 42: dequantize_row_q2_0(static_cast<const block_q2_0*>(blocks), y, k); return 1;
    default: return 0;
  }
}

// ggml reference activation quantizers and the reference's AVX-512 versions.
void ref_quantize_q8_K(const float* x, void* y, int64_t k) {
  quantize_row_q8_K_ref(x, static_cast<block_q8_K*>(y), k);
}
void ref_quantize_q8_0(const float* x, void* y, int64_t k) {
  quantize_row_q8_0_ref(x, static_cast<block_q8_0*>(y), k);
}
void ref_quantize_q8_K_avx(const float* x, void* y, int64_t k) {
  quantize_row_q8_K_f32(x, static_cast<block_q8_K*>(y), k);
}
void ref_quantize_q8_0_avx(const float* x, void* y, int64_t k) {
  quantize_row_q8_0_f32(x, static_cast<block_q8_0*>(y), k);
}
void ref_quantize_q8_K_bf16(const uint16_t* x, void* y, int64_t k) {
  quantize_row_q8_K_bf16(x, static_cast<block_q8_K*>(y), k);
}
void ref_quantize_q8_0_bf16(const uint16_t* x, void* y, int64_t k) {
  quantize_row_q8_0_bf16(x, static_cast<block_q8_0*>(y), k);
}

// ggml generic dot products (portable C).
float ref_vec_dot_iq3_s_q8_K(int n, const void* w, const void* a) {
  float s = 0;
  ggml_vec_dot_iq3_s_q8_K_generic(n, &s, 0, w, 0, a, 0, 1);
  return s;
}
float ref_vec_dot_iq4_nl_q8_0(int n, const void* w, const void* a) {
  float s = 0;
  ggml_vec_dot_iq4_nl_q8_0_generic(n, &s, 0, w, 0, a, 0, 1);
  return s;
}

// Kernel-native layouts of the CPU expert tier.
int64_t ref_decoded_row_bytes(int fmt, int k) { return int64_t(decoded_row_bytes(WeightFormat(fmt), k)); }
int64_t ref_packed_act_bytes(int act, int k) { return int64_t(packed_act_bytes(ActFormat(act), k)); }
int64_t ref_weight_row_bytes(int fmt, int k) { return int64_t(weight_row_bytes(WeightFormat(fmt), k)); }
void ref_decode_rows(int fmt, const void* rows, int64_t row_bytes, int nrows, int k, void* dst) {
  decode_rows(WeightFormat(fmt), rows, std::size_t(row_bytes), nrows, k, dst);
}
void ref_quantize_pack_f32(int act, const float* x, int k, void* dst) {
  quantize_pack_f32(ActFormat(act), x, k, dst);
}
void ref_quantize_pack_bf16(int act, const uint16_t* x, int k, void* dst) {
  quantize_pack_bf16(ActFormat(act), x, k, dst);
}
void ref_gemm_decoded(int fmt, const void* wdec, int nrows, int k, const void* const* acts, int T,
                      float* out, int64_t ldo) {
  gemm_decoded(WeightFormat(fmt), wdec, nrows, k, acts, T, out, std::size_t(ldo));
}
void ref_decode_rows_bf16(int fmt, const void* rows, int64_t row_bytes, int nrows, int k,
                          uint16_t* dst) {
  decode_rows_bf16(WeightFormat(fmt), rows, std::size_t(row_bytes), nrows, k, dst);
}
void ref_gemm_bf16(const uint16_t* w, int nrows, int k, const void* const* acts, int T, float* out,
                   int64_t ldo) {
  gemm_bf16(w, nrows, k, acts, T, out, std::size_t(ldo));
}
void ref_silu_mul(const float* g, const float* u, float* h, int n) { silu_mul(g, u, h, n); }


// ---------------------------------------------------------------------------------------------
// Drivers over the reference primitives. The reference's ExpertPool fixes hidden 2560 / inter 640
// and a Q8_0 down projection at compile time (src/cpu/expert_pool.cpp:22-38, :525-526), so the
// benchmark shapes (inter 512, IQ3_S down) are assembled here from the same primitives in the same
// phase order (src/cpu/expert_pool.cpp:330-408): activations quantized and packed once per token,
// gate/up rows decoded four at a time and multiplied, SwiGLU, h re-quantized for the down format,
// down rows decoded and multiplied, per-token weighted sum over experts in ascending id.
namespace {

struct Aligned {
  uint8_t* p = nullptr;
  explicit Aligned(std::size_t n) { p = static_cast<uint8_t*>(std::aligned_alloc(64, (n + 63) & ~std::size_t(63))); }
  ~Aligned() { std::free(p); }
  Aligned(const Aligned&) = delete;
};

// gate/up -> SwiGLU for rows [j0, j1) of one expert over `nt` packed activation rows.
void phase_a(WeightFormat f, int hidden, const uint8_t* gate, const uint8_t* up, int j0, int j1,
             const void* const* acts, int nt, float* h /*[nt][inter]*/, int inter, uint8_t* dec,
             float* gu) {
  const std::size_t rb = weight_row_bytes(f, hidden), db = decoded_row_bytes(f, hidden);
  for (int j = j0; j < j1; j += 4) {
    const int nr = std::min(4, j1 - j);
    decode_rows(f, gate + std::size_t(j) * rb, rb, nr, hidden, dec);
    decode_rows(f, up + std::size_t(j) * rb, rb, nr, hidden, dec + std::size_t(nr) * db);
    gemm_decoded(f, dec, 2 * nr, hidden, acts, nt, gu, std::size_t(nt));
    for (int t = 0; t < nt; ++t) {
      float g[4], u[4], hv[4];
      for (int r = 0; r < nr; ++r) {
        g[r] = gu[std::size_t(r) * nt + t];
        u[r] = gu[std::size_t(nr + r) * nt + t];
      }
      silu_mul(g, u, hv, nr);
      for (int r = 0; r < nr; ++r) h[std::size_t(t) * inter + j + r] = hv[r];
    }
  }
}

}  // namespace

// One expert, T tokens, decode numerics. h [T][inter] and y [T][hidden] unweighted.
void ref_expert_ffn(int fmt_gu, int fmt_down, int hidden, int inter, const uint8_t* gate,
                    const uint8_t* up, const uint8_t* down, const float* x, int T, float* h_out,
                    float* y_out) {
  const WeightFormat fg = WeightFormat(fmt_gu), fd = WeightFormat(fmt_down);
  const ActFormat ag = format_info(fg).act, ad = format_info(fd).act;
  const std::size_t pa = packed_act_bytes(ag, hidden), ph = packed_act_bytes(ad, inter);
  Aligned xa(pa * T), ha(ph * T), dec(8 * std::max(decoded_row_bytes(fg, hidden), decoded_row_bytes(fd, inter)));
  std::vector<const void*> xp(T), hp(T);
  std::vector<float> h(std::size_t(T) * inter), gu(std::size_t(8) * T);
  for (int t = 0; t < T; ++t) {
    quantize_pack_f32(ag, x + std::size_t(t) * hidden, hidden, xa.p + pa * t);
    xp[t] = xa.p + pa * t;
  }
  phase_a(fg, hidden, gate, up, 0, inter, xp.data(), T, h.data(), inter, dec.p, gu.data());
  if (h_out) std::memcpy(h_out, h.data(), h.size() * sizeof(float));
  for (int t = 0; t < T; ++t) {
    quantize_pack_f32(ad, h.data() + std::size_t(t) * inter, inter, ha.p + ph * t);
    hp[t] = ha.p + ph * t;
  }
  const std::size_t rb = weight_row_bytes(fd, inter);
  std::vector<float> out(std::size_t(8) * T);
  for (int n = 0; n < hidden; n += 8) {
    const int nr = std::min(8, hidden - n);
    decode_rows(fd, down + std::size_t(n) * rb, rb, nr, inter, dec.p);
    gemm_decoded(fd, dec.p, nr, inter, hp.data(), T, out.data(), std::size_t(T));
    for (int r = 0; r < nr; ++r)
      for (int t = 0; t < T; ++t) y_out[std::size_t(t) * hidden + n + r] = out[std::size_t(r) * T + t];
  }
}

// One expert, T tokens, prefill numerics (bf16 weights and activations, h rounded to bf16).
void ref_expert_ffn_bf16(int fmt_gu, int fmt_down, int hidden, int inter, const uint8_t* gate,
                         const uint8_t* up, const uint8_t* down, const uint16_t* x, int T,
                         uint16_t* h_out, float* y_out) {
  const WeightFormat fg = WeightFormat(fmt_gu), fd = WeightFormat(fmt_down);
  const std::size_t rbg = weight_row_bytes(fg, hidden), rbd = weight_row_bytes(fd, inter);
  std::vector<uint16_t> w(std::size_t(8) * std::max(hidden, inter));
  std::vector<const void*> xp(T), hp(T);
  std::vector<uint16_t> hb(std::size_t(T) * inter);
  std::vector<float> gu(std::size_t(8) * T);
  for (int t = 0; t < T; ++t) xp[t] = x + std::size_t(t) * hidden;
  for (int j = 0; j < inter; j += 4) {
    decode_rows_bf16(fg, gate + std::size_t(j) * rbg, rbg, 4, hidden, w.data());
    decode_rows_bf16(fg, up + std::size_t(j) * rbg, rbg, 4, hidden, w.data() + std::size_t(4) * hidden);
    gemm_bf16(w.data(), 8, hidden, xp.data(), T, gu.data(), std::size_t(T));
    for (int t = 0; t < T; ++t) {
      float g[4], u[4], hv[4];
      for (int r = 0; r < 4; ++r) {
        g[r] = gu[std::size_t(r) * T + t];
        u[r] = gu[std::size_t(4 + r) * T + t];
      }
      silu_mul(g, u, hv, 4);
      for (int r = 0; r < 4; ++r) {
        uint32_t b;
        std::memcpy(&b, &hv[r], 4);
        // RNE to bf16, as the pool's vcvtne2ps2bf16 does (src/cpu/expert_pool.cpp:364-367).
        hb[std::size_t(t) * inter + j + r] = uint16_t((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
      }
    }
  }
  if (h_out) std::memcpy(h_out, hb.data(), hb.size() * 2);
  for (int t = 0; t < T; ++t) hp[t] = hb.data() + std::size_t(t) * inter;
  std::vector<float> out(std::size_t(8) * T);
  for (int n = 0; n < hidden; n += 8) {
    decode_rows_bf16(fd, down + std::size_t(n) * rbd, rbd, 8, inter, w.data());
    gemm_bf16(w.data(), 8, inter, hp.data(), T, out.data(), std::size_t(T));
    for (int r = 0; r < 8; ++r)
      for (int t = 0; t < T; ++t) y_out[std::size_t(t) * hidden + n + r] = out[std::size_t(r) * T + t];
  }
}

// One MoE layer step on `threads` host threads: pairs grouped by expert; phase A tasks are
// (expert group, 32 intermediate rows); phase B tasks are 32 output rows over every group in
// ascending expert id, which fixes the summation order (src/cpu/expert_pool.cpp:375-408).
void ref_moe_layer(int fmt_gu, int fmt_down, int hidden, int inter, const uint8_t* blobs,
                   int64_t blob_stride, const float* x, int T, int k, const int32_t* ids,
                   const float* w, float* y, int threads) {
  const WeightFormat fg = WeightFormat(fmt_gu), fd = WeightFormat(fmt_down);
  const ActFormat ag = format_info(fg).act, ad = format_info(fd).act;
  const std::size_t pa = packed_act_bytes(ag, hidden), ph = packed_act_bytes(ad, inter);
  const std::size_t gate_bytes = std::size_t(inter) * weight_row_bytes(fg, hidden);
  const std::size_t rbd = weight_row_bytes(fd, inter);
  struct Group { int expert, begin, end; };
  std::vector<std::pair<int, int>> pairs;  // (expert, token*k + slot)
  for (int t = 0; t < T; ++t)
    for (int r = 0; r < k; ++r) pairs.emplace_back(ids[t * k + r], t * k + r);
  std::sort(pairs.begin(), pairs.end());
  std::vector<Group> groups;
  for (int i = 0; i < int(pairs.size()); ++i) {
    if (groups.empty() || groups.back().expert != pairs[i].first) groups.push_back({pairs[i].first, i, i});
    groups.back().end = i + 1;
  }
  const int np = int(pairs.size());
  Aligned xa(pa * T), ha(ph * np);
  std::vector<float> h(std::size_t(np) * inter);
  std::vector<const void*> pair_act(np), pair_h(np);
  for (int i = 0; i < np; ++i) {
    pair_act[i] = xa.p + pa * (pairs[i].second / k);
    pair_h[i] = ha.p + ph * i;
  }
  threads = std::max(1, threads);
  auto run = [&](auto&& body) {
    std::vector<std::thread> pool;
    for (int i = 1; i < threads; ++i) pool.emplace_back(body);
    body();
    for (auto& th : pool) th.join();
  };
  std::atomic<int> next{0};
  run([&] { for (int t; (t = next.fetch_add(1)) < T;) quantize_pack_f32(ag, x + std::size_t(t) * hidden, hidden, xa.p + pa * t); });
  const int chunks = (inter + 31) / 32;
  next = 0;
  run([&] {
    Aligned dec(8 * decoded_row_bytes(fg, hidden));
    std::vector<float> gu(std::size_t(8) * 64);
    for (int task; (task = next.fetch_add(1)) < int(groups.size()) * chunks;) {
      const Group& g = groups[task / chunks];
      const int j0 = (task % chunks) * 32, j1 = std::min(inter, j0 + 32);
      const uint8_t* blob = blobs + std::size_t(g.expert) * blob_stride;
      for (int p0 = g.begin; p0 < g.end; p0 += 64) {
        const int nt = std::min(64, g.end - p0);
        phase_a(fg, hidden, blob, blob + gate_bytes, j0, j1, pair_act.data() + p0, nt,
                h.data() + std::size_t(p0) * inter, inter, dec.p, gu.data());
      }
    }
  });
  next = 0;
  run([&] { for (int p; (p = next.fetch_add(1)) < np;) quantize_pack_f32(ad, h.data() + std::size_t(p) * inter, inter, ha.p + ph * p); });
  next = 0;
  const int bchunks = hidden / 32;
  run([&] {
    Aligned dec(8 * decoded_row_bytes(fd, inter));
    std::vector<float> out, yb(std::size_t(T) * 32);
    for (int task; (task = next.fetch_add(1)) < bchunks;) {
      const int r0 = task * 32;
      std::fill(yb.begin(), yb.end(), 0.0f);
      for (const Group& g : groups) {
        const int te = g.end - g.begin;
        out.resize(std::size_t(8) * te);
        const uint8_t* down = blobs + std::size_t(g.expert) * blob_stride + 2 * gate_bytes;
        for (int tile = 0; tile < 32; tile += 8) {
          decode_rows(fd, down + std::size_t(r0 + tile) * rbd, rbd, 8, inter, dec.p);
          gemm_decoded(fd, dec.p, 8, inter, pair_h.data() + g.begin, te, out.data(), std::size_t(te));
          for (int i = 0; i < 8; ++i)
            for (int p = 0; p < te; ++p) {
              const int slot = pairs[g.begin + p].second;
              yb[std::size_t(slot / k) * 32 + tile + i] += w[slot] * out[std::size_t(i) * te + p];
            }
        }
      }
      for (int t = 0; t < T; ++t) std::memcpy(y + std::size_t(t) * hidden + r0, yb.data() + std::size_t(t) * 32, 32 * sizeof(float));
    }
  });
}

}  // extern "C"
