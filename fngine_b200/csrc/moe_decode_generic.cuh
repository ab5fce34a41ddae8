// Decode-width projections for the reference's other expert formats: IQ3_XXS, IQ2_S and IQ4_XS as
// gate/up formats (256-weight super-blocks, paired with Q8_K activations) and Q2_0 as a down format
// (64-weight blocks, paired with Q8_0), src/kernels/moe/iq_device.cuh:171-288 and
// third_party/ggml-iq/ggml-iq.h:26-78 of the reference. Included by moe_decode.cu (everything) and by
// probes.cu (the decoders and the dequantization probe only).
//
// These are plain kernels, not the streaming skeleton of the IQ3_S / IQ4_NL paths: a warp takes one
// (work item, row) unit, its lanes the row's 32-weight sub-blocks straight from global memory; every
// sub-block is decoded once into eight words of int8 weights and met with each token's codes by dp4a.
// Arithmetic per sub-block and token: d * dA * (m0 * dot(first 16) + m1 * dot(second 16)), the integer
// part exact; a warp butterfly adds the lanes. They read the device work list a selection kernel left.
// Not tuned: they are here so that a layer in any of the pack's formats runs on the GPU with the CPU
// tier's numerics (1e-3), at a fraction of the streaming kernels' rate.
// (No namespace of its own: included inside namespace fb's unnamed namespace, once per translation unit.)
#pragma once

static __constant__ uint16_t c_iq3xxs_grid_packed[256] = {FB_IQ3XXS_GRID_PACKED};
static __constant__ uint16_t c_iq2s_grid_packed[1024] = {FB_IQ2S_GRID_PACKED};

constexpr int kGenericGridWords = 2048;  // shared-memory words the largest expanded codebook takes (IQ2_S: 1024 x 8 bytes)

// Expands the format's codebook into shared memory (called by every thread; caller synchronizes).
// IQ3_XXS: 256 words of four magnitudes; IQ2_S: 1024 pairs of words of four magnitudes each.
template <int FMT>
__device__ __forceinline__ void generic_grid_fill(uint32_t* grid) {
  if constexpr (FMT == FB_FMT_IQ3_XXS) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
      const uint32_t p = c_iq3xxs_grid_packed[i];
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t c = (p >> (3 * j)) & 7u;
        w |= (4u + 8u * c + (c == 7u ? 2u : 0u)) << (8 * j);  // 4, 12, ..., 52, 62
      }
      grid[i] = w;
    }
  } else if constexpr (FMT == FB_FMT_IQ2_S) {
    for (int i = threadIdx.x; i < 2048; i += blockDim.x) {
      const uint32_t p = c_iq2s_grid_packed[i >> 1] >> (8 * (i & 1));
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t c = (p >> (2 * j)) & 3u;
        w |= (c == 0u ? 8u : c == 1u ? 25u : 43u) << (8 * j);
      }
      grid[i] = w;
    }
  }
}

__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) { return uint32_t(p[0]) | (uint32_t(p[1]) << 8); }
__device__ __forceinline__ uint32_t ld_u32_unaligned(const uint8_t* p) {  // two-byte aligned
  return ld_u16(p) | (ld_u16(p + 2) << 16);
}
__device__ __forceinline__ float fp16_bits(uint32_t h) { return __half2float(__ushort_as_half(static_cast<unsigned short>(h))); }
// bit j of an 8-bit sign pattern -> byte j = 0xFF: bits 0-3 into the first word, 4-7 into the second
__device__ __forceinline__ int sign_bytes(uint32_t s4) {
  return int(__vcmpne4((s4 * 0x00204081u) & 0x01010101u, 0u));  // bit j of the nibble at position 8j
}
__device__ __forceinline__ int apply_sign(uint32_t mag, int mask) { return int(__vsub4(mag ^ uint32_t(mask), uint32_t(mask))); }

// One 32-weight sub-block, decoded: q[0..3] = weights 0..15, q[4..7] = weights 16..31 (int8 x 4 per word),
// integer multipliers of the two halves and the float factor.
struct Sub32 {
  int q[8];
  int m0, m1;
  float d;
};

// `row` = the weight row, `sub` = index of the 32-weight sub-block inside it.
template <int FMT>
__device__ __forceinline__ void decode_sub32(const uint8_t* row, int sub, const uint32_t* grid, Sub32& s) {
  if constexpr (FMT == FB_FMT_IQ3_XXS) {
    const uint8_t* b = row + (sub >> 3) * 98;
    const int ib = sub & 7;
    const uint8_t* qs = b + 2 + 8 * ib;
    const uint32_t aux = ld_u32_unaligned(b + 2 + 64 + 4 * ib);
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const uint32_t idx7 = (aux >> (7 * l)) & 127u;
      const uint32_t sg = idx7 | ((__popc(idx7) & 1u) << 7);  // the sign pattern: index + parity bit
      s.q[2 * l] = apply_sign(grid[qs[2 * l]], sign_bytes(sg & 15u));
      s.q[2 * l + 1] = apply_sign(grid[qs[2 * l + 1]], sign_bytes(sg >> 4));
    }
    s.m0 = s.m1 = 2 * int(aux >> 28) + 1;
    s.d = fp16_bits(ld_u16(b)) * 0.25f;
  } else if constexpr (FMT == FB_FMT_IQ2_S) {
    const uint8_t* b = row + (sub >> 3) * 82;
    const int ib = sub & 7;
    const uint8_t* qs = b + 2 + 4 * ib;
    const uint8_t* sg = b + 2 + 32 + 4 * ib;
    const uint32_t qh = b[2 + 64 + ib];
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const uint32_t idx = uint32_t(qs[l]) | ((qh << (8 - 2 * l)) & 0x300u);
      s.q[2 * l] = apply_sign(grid[2 * idx], sign_bytes(uint32_t(sg[l]) & 15u));
      s.q[2 * l + 1] = apply_sign(grid[2 * idx + 1], sign_bytes(uint32_t(sg[l]) >> 4));
    }
    const uint32_t sc = b[2 + 64 + 8 + ib];
    s.m0 = 2 * int(sc & 15u) + 1;
    s.m1 = 2 * int(sc >> 4) + 1;
    s.d = fp16_bits(ld_u16(b)) * 0.125f;
  } else if constexpr (FMT == FB_FMT_IQ4_XS) {
    const uint8_t* b = row + (sub >> 3) * 136;
    const int ib = sub & 7;
    const uint8_t* qs = b + 8 + 16 * ib;  // 8-byte header: d, scales_h, scales_l[4]
    constexpr int lv[16] = {FB_IQ4NL_LEVELS};
    auto level = [&](uint32_t n) -> uint32_t {  // 16-way select on a nibble (registers only)
      int v = lv[0];
#pragma unroll
      for (int i = 1; i < 16; ++i) v = n == uint32_t(i) ? lv[i] : v;
      return uint32_t(v) & 0xFFu;
    };
#pragma unroll
    for (int wv = 0; wv < 4; ++wv) {
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t byte = qs[4 * wv + j];
        lo |= level(byte & 15u) << (8 * j);
        hi |= level(byte >> 4) << (8 * j);
      }
      s.q[wv] = int(lo);      // weights 4wv .. 4wv+3
      s.q[4 + wv] = int(hi);  // weights 16 + 4wv ..
    }
    const uint32_t sl = b[4 + (ib >> 1)], sh = ld_u16(b + 2);
    const int ls = int(((sl >> (4 * (ib & 1))) & 15u) | (((sh >> (2 * ib)) & 3u) << 4));
    s.m0 = s.m1 = ls - 32;
    s.d = fp16_bits(ld_u16(b));
  } else {  // Q2_0: the sub-block is half of a 64-weight block; weights in natural order
    const uint8_t* b = row + (sub >> 1) * 18;
    const uint8_t* qs = b + 2 + 8 * (sub & 1);
#pragma unroll
    for (int wv = 0; wv < 8; ++wv) {
      const uint32_t c = qs[wv];  // four 2-bit codes, lowest first
      const uint32_t x = (c & 3u) | ((c & 0xCu) << 6) | ((c & 0x30u) << 12) | ((c & 0xC0u) << 18);
      s.q[wv] = int(__vsub4(x, 0x01010101u));
    }
    s.m0 = s.m1 = 1;
    s.d = fp16_bits(ld_u16(b));
  }
}

// Exact fp32 values of the sub-block's 32 weights in ggml's own operation order
// (third_party/ggml-iq/ggml-iq.c:135-152, 171-229, 290-311), for the bit-exact dequantization probe.
template <int FMT>
__device__ __forceinline__ void dequant_sub32(const uint8_t* row, int sub, const uint32_t* grid, float* y) {
  Sub32 s;
  decode_sub32<FMT>(row, sub, grid, s);
  float d0, d1;
  if constexpr (FMT == FB_FMT_IQ3_XXS) {
    const float d = fp16_bits(ld_u16(row + (sub >> 3) * 98));
    d0 = d1 = d * (0.5f + float((s.m0 - 1) / 2)) * 0.5f;
  } else if constexpr (FMT == FB_FMT_IQ2_S) {
    const float d = fp16_bits(ld_u16(row + (sub >> 3) * 82));
    d0 = d * (0.5f + float((s.m0 - 1) / 2)) * 0.25f;
    d1 = d * (0.5f + float((s.m1 - 1) / 2)) * 0.25f;
  } else if constexpr (FMT == FB_FMT_IQ4_XS) {
    d0 = d1 = s.d * float(s.m0);
  } else {
    d0 = d1 = s.d;
  }
#pragma unroll
  for (int wv = 0; wv < 8; ++wv)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int v = int(int8_t(uint32_t(s.q[wv]) >> (8 * j)));
      const float dl = wv < 4 ? d0 : d1;
      float r;
      if constexpr (FMT == FB_FMT_Q2_0) r = float(v) * dl;           // (q - 1) * d
      else if constexpr (FMT == FB_FMT_IQ4_XS) r = dl * float(v);     // dl * level
      else r = dl * float(v < 0 ? -v : v) * (v < 0 ? -1.0f : 1.0f);   // dl * magnitude * sign
      y[4 * wv + j] = r;
    }
}

template <int FMT>
__global__ void __launch_bounds__(256) dequant_generic_kernel(const uint8_t* __restrict__ rows, int64_t row_bytes,
                                                              int nrows, int k, float* __restrict__ out) {
  __shared__ uint32_t s_grid[kGenericGridWords];
  generic_grid_fill<FMT>(s_grid);
  __syncthreads();
  const int subs = k / 32;
  for (int64_t u = int64_t(blockIdx.x) * 256 + threadIdx.x; u < int64_t(nrows) * subs; u += int64_t(gridDim.x) * 256) {
    const int r = int(u / subs), sub = int(u - int64_t(r) * subs);
    float y[32];
    dequant_sub32<FMT>(rows + int64_t(r) * row_bytes, sub, s_grid, y);
    float4* o = reinterpret_cast<float4*>(out + int64_t(r) * k + 32 * sub);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = make_float4(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
  }
}

#ifdef FB_MOE_DECODE_TU  // the MoE kernels below need the decode translation unit's workspace helpers
// dp4a of a decoded sub-block with 32 activation codes in natural order (Q8_K planar rows)
__device__ __forceinline__ float sub32_dot_natural(const Sub32& s, const int* a, float da) {
  int s0 = 0, s1 = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) s0 = __dp4a(s.q[j], a[j], s0);
#pragma unroll
  for (int j = 4; j < 8; ++j) s1 = __dp4a(s.q[j], a[j], s1);
  return float(s.m0 * s0 + s.m1 * s1) * (s.d * da);
}

constexpr int kGenTok = 4;  // tokens of an item handled per pass over a row

// gate/up for a Q8_K-paired format: unit = (item, intermediate row); h[pair][j] = silu(gate.x) * (up.x).
template <int FMT>
__global__ void __launch_bounds__(256) gate_up_generic_kernel(fb_moe_expert_layout L, fb_moe_decode_workspace ws) {
  __shared__ uint32_t s_grid[kGenericGridWords];
  generic_grid_fill<FMT>(s_grid);
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait_prior();
  const fb_moe_decode_work* work = ws.work;
  const int n_items = min(max(work->n_items, 0), kMaxPairs), I = L.inter;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row_bytes = int64_t(H / 256) * (FMT == FB_FMT_IQ3_XXS ? 98 : FMT == FB_FMT_IQ2_S ? 82 : 136);
  for (int u = blockIdx.x * 8 + warp; u < n_items * I; u += gridDim.x * 8) {
    const int item = u / I, j = u - item * I;
    const int pb = work->item_pair_begin[item], ntok = work->item_pair_begin[item + 1] - pb;
    const uint8_t* blob = L.slots + int64_t(work->item_slot[item]) * L.blob_stride;
    const uint8_t* grow = blob + L.gate_offset + int64_t(j) * row_bytes;
    const uint8_t* urow = blob + L.up_offset + int64_t(j) * row_bytes;
    for (int t0 = 0; t0 < ntok; t0 += kGenTok) {
      float ag[kGenTok], au[kGenTok];
      const uint8_t* xq[kGenTok];
#pragma unroll
      for (int t = 0; t < kGenTok; ++t) {
        ag[t] = au[t] = 0.0f;
        xq[t] = ws.xq + size_t(work->pair_token[pb + min(t0 + t, ntok - 1)]) * FB_XQ_STRIDE;  // Q8_K rows sit first
      }
      for (int sub = lane; sub < H / 32; sub += 32) {
        Sub32 sg, su;
        decode_sub32<FMT>(grow, sub, s_grid, sg);
        decode_sub32<FMT>(urow, sub, s_grid, su);
#pragma unroll
        for (int t = 0; t < kGenTok; ++t) {
          const int4* ap = reinterpret_cast<const int4*>(xq[t] + 32 * sub);
          const int4 a0 = ap[0], a1 = ap[1];
          const int a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
          const float da = reinterpret_cast<const float*>(xq[t] + H)[sub >> 3];
          ag[t] += sub32_dot_natural(sg, a, da);
          au[t] += sub32_dot_natural(su, a, da);
        }
      }
#pragma unroll
      for (int t = 0; t < kGenTok; ++t) {
        float g = ag[t], up = au[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          g += __shfl_xor_sync(0xffffffffu, g, o);
          up += __shfl_xor_sync(0xffffffffu, up, o);
        }
        if (lane == 0 && t0 + t < ntok) ws.h[size_t(pb + t0 + t) * I + j] = silu_mul(g, up);
      }
    }
  }
}

// h of every pair -> planar activation rows for the down projection (one warp per pair); the streaming
// gate/up kernels do this themselves, the generic one leaves it to this launch.
__global__ void __launch_bounds__(256) requant_h_kernel(fb_moe_expert_layout L, fb_moe_decode_workspace ws) {
  pdl_launch_dependents();
  pdl_wait_prior();
  const int n_pairs = min(max(ws.work->n_pairs, 0), kMaxPairs);
  const int p = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (p < n_pairs) quantize_item_h(ws, p, 1, act_of(L.down_format), L.inter);
}

// down for Q2_0 (Q8_0 activations, stored per 32-block in the order position p <- element (p % 2) * 16 + p / 2):
// unit = (item, pair of output rows): lanes 0-15 take the 16 sub-blocks of row 2n (inter 512; 20 of 640 wrap),
// lanes 16-31 those of row 2n + 1. partial[pair][n] = w_pair * (down_n . q8(h[pair])).
__global__ void __launch_bounds__(256) down_q2_0_kernel(fb_moe_expert_layout L, fb_moe_decode_workspace ws) {
  pdl_launch_dependents();
  pdl_wait_prior();
  const fb_moe_decode_work* work = ws.work;
  const int n_items = min(max(work->n_items, 0), kMaxPairs), I = L.inter;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, half = lane >> 4, hl = lane & 15;
  const int64_t row_bytes = int64_t(I / 64) * 18;
  for (int u = blockIdx.x * 8 + warp; u < n_items * (H / 2); u += gridDim.x * 8) {
    const int item = u / (H / 2), n = 2 * (u - item * (H / 2)) + half;
    const int pb = work->item_pair_begin[item], ntok = work->item_pair_begin[item + 1] - pb;
    const uint8_t* row = L.slots + int64_t(work->item_slot[item]) * L.blob_stride + L.down_offset + int64_t(n) * row_bytes;
    for (int t0 = 0; t0 < ntok; t0 += kGenTok) {
      float acc[kGenTok];
#pragma unroll
      for (int t = 0; t < kGenTok; ++t) acc[t] = 0.0f;
      for (int sub = hl; sub < I / 32; sub += 16) {
        Sub32 s;
        decode_sub32<FB_FMT_Q2_0>(row, sub, nullptr, s);
        // weights into the activation rows' order: word w <- weights (2w, 2w + 16, 2w + 1, 2w + 17)
        int wq[8];
#pragma unroll
        for (int wv = 0; wv < 8; ++wv) {
          const uint32_t lo = uint32_t(s.q[wv >> 1]), hi = uint32_t(s.q[4 + (wv >> 1)]);
          wq[wv] = int(__byte_perm(lo, hi, (wv & 1) ? 0x7362 : 0x5140));
        }
#pragma unroll
        for (int t = 0; t < kGenTok; ++t) {
          const uint8_t* hq = ws.hq + size_t(pb + min(t0 + t, ntok - 1)) * FB_HQ_STRIDE;
          const int4* ap = reinterpret_cast<const int4*>(hq + 32 * sub);
          const int4 a0 = ap[0], a1 = ap[1];
          const int a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
          int sum = 0;
#pragma unroll
          for (int wv = 0; wv < 8; ++wv) sum = __dp4a(wq[wv], a[wv], sum);
          acc[t] = fmaf(float(sum), s.d * reinterpret_cast<const float*>(hq + I)[sub], acc[t]);
        }
      }
#pragma unroll
      for (int t = 0; t < kGenTok; ++t) {
        float v = acc[t];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (hl == 0 && t0 + t < ntok) ws.partial[size_t(pb + t0 + t) * H + n] = work->pair_weight[pb + t0 + t] * v;
      }
    }
  }
}

#endif  // FB_MOE_DECODE_TU
