// Parity probes and the seeded expert-byte generator. The probes run the same device routines the
// GEMV kernels use (iq_decode.cuh) and write results in the reference's own layouts, so dequantized
// weights and int8 activations can be compared bit for bit with the CPU reference.
#include "iq_decode.cuh"

#include <cuda_bf16.h>

namespace fb {
namespace {

#include "moe_decode_generic.cuh"

// One warp per row; lane l walks the row's sub-blocks l, l+32, ... through the shared-memory
// codebook path. Output value = (d * (1 + 2s)) * float(signed magnitude), the reference's
// rounding (third_party/ggml-iq/ggml-iq.c:242-250).
__global__ void __launch_bounds__(256) dequant_iq3s_kernel(const uint8_t* __restrict__ rows, int64_t row_bytes,
                                                           int nrows, int k, float* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t smem[];
  uint32_t* gridrep = reinterpret_cast<uint32_t*>(smem);
  uint32_t* signtab = reinterpret_cast<uint32_t*>(smem + kGridRepBytes);
  iq3s_tables_fill(gridrep, signtab);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const uint32_t* grid_lane = gridrep + lane;
  for (int r = blockIdx.x * 8 + (threadIdx.x >> 5); r < nrows; r += gridDim.x * 8) {
    const uint8_t* row = rows + int64_t(r) * row_bytes;
    for (int sb = lane; sb < k / 32; sb += 32) {
      const uint8_t* blk = row + (sb >> 3) * 110;
      const int ib = sb & 7;
      auto rd16 = [&](int off) { return uint32_t(blk[off]) | (uint32_t(blk[off + 1]) << 8); };
      auto rd32 = [&](int off) { return rd16(off) | (rd16(off + 2) << 16); };
      const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(rd16(0))));
      uint32_t g[8], m[8];
      iq3s_decode_sub(rd32(2 + 8 * ib), rd32(6 + 8 * ib), blk[66 + ib], 0, rd32(74 + 4 * ib), grid_lane, signtab, g, m);
      int w[8];
#pragma unroll
      for (int l = 0; l < 8; ++l) w[l] = iq3s_signed(g[l], m[l]);
      const int s = (blk[106 + ib / 2] >> (4 * (ib & 1))) & 0xF;
      const float db = __fmul_rn(d, float(1 + 2 * s));
      float* o = out + int64_t(r) * k + 32 * sb;
#pragma unroll
      for (int l = 0; l < 8; ++l)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[4 * l + j] = __fmul_rn(db, float(int8_t(uint32_t(w[l]) >> (8 * j))));
    }
  }
}

__global__ void __launch_bounds__(256) dequant_iq4nl_kernel(const uint8_t* __restrict__ rows, int64_t row_bytes,
                                                            int nrows, int k, float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const Iq4nlLevels lv = iq4nl_levels();
  for (int r = blockIdx.x * 8 + (threadIdx.x >> 5); r < nrows; r += gridDim.x * 8) {
    const uint8_t* row = rows + int64_t(r) * row_bytes;
    for (int b = lane; b < k / 32; b += 32) {
      const uint8_t* blk = row + b * 18;
      auto rd16 = [&](int off) { return uint32_t(blk[off]) | (uint32_t(blk[off + 1]) << 8); };
      const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(rd16(0))));
      uint32_t q[4];
#pragma unroll
      for (int m = 0; m < 4; ++m) q[m] = rd16(2 + 4 * m) | (rd16(4 + 4 * m) << 16);
      int w[8];
      iq4nl_decode32(lv, q, w);
      float* o = out + int64_t(r) * k + 32 * b;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int pos = q8_0_interleave_index(e);
        o[e] = __fmul_rn(d, float(int8_t(uint32_t(w[pos >> 2]) >> (8 * (pos & 3)))));
      }
    }
  }
}

// ggml block_q8_K: float d | int8 qs[256] | int16 bsums[16] (292 bytes); one warp per block.
template <bool XBF16>
__global__ void __launch_bounds__(256) quantize_q8k_kernel(const void* __restrict__ xv, int64_t n_blocks,
                                                           uint8_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  for (int64_t b = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5); b < n_blocks; b += int64_t(gridDim.x) * 8) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int64_t idx = b * 256 + 8 * lane + i;
      if constexpr (XBF16) v[i] = __bfloat162float(static_cast<const __nv_bfloat16*>(xv)[idx]);
      else v[i] = static_cast<const float*>(xv)[idx];
    }
    int q[8], ps;
    const float d = q8k_block_warp(v, q, ps);
    uint8_t* blk = out + b * 292;
#pragma unroll
    for (int i = 0; i < 8; ++i) blk[4 + 8 * lane + i] = uint8_t(int8_t(q[i]));
    if ((lane & 1) == 0) {
      const uint16_t s = uint16_t(int16_t(ps));
      blk[260 + lane] = uint8_t(s & 0xFF);  // bsums[lane / 2]
      blk[261 + lane] = uint8_t(s >> 8);
    }
    if (lane == 0) {
      const uint32_t u = __float_as_uint(d);
      blk[0] = uint8_t(u);
      blk[1] = uint8_t(u >> 8);
      blk[2] = uint8_t(u >> 16);
      blk[3] = uint8_t(u >> 24);
    }
  }
}

// ggml block_q8_0: fp16 d | int8 qs[32] (34 bytes); one warp per block, natural element order.
template <bool XBF16>
__global__ void __launch_bounds__(256) quantize_q8_0_kernel(const void* __restrict__ xv, int64_t n_blocks,
                                                            uint8_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  for (int64_t b = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5); b < n_blocks; b += int64_t(gridDim.x) * 8) {
    const int64_t idx = b * 32 + lane;
    float v;
    if constexpr (XBF16) v = __bfloat162float(static_cast<const __nv_bfloat16*>(xv)[idx]);
    else v = static_cast<const float*>(xv)[idx];
    unsigned short dh;
    const int q = q8_0_block_warp(v, dh);
    uint8_t* blk = out + b * 34;
    blk[2 + lane] = uint8_t(int8_t(q));
    if (lane == 0) {
      blk[0] = uint8_t(dh & 0xFF);
      blk[1] = uint8_t(dh >> 8);
    }
  }
}

// splitmix64 finalizer over (seed + (counter + 1) * golden): word `counter` of the stream a
// sequential splitmix64 generator seeded with `seed` would produce.
__host__ __device__ __forceinline__ uint64_t splitmix_at(uint64_t seed, uint64_t counter) {
  uint64_t z = seed + (counter + 1) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// Block b takes ceil(block_bytes/8) stream words starting at b * words; bytes 2.. of the block are
// the stream bytes 2.., bytes 0-1 are d_table[word0 & 0xFFFF]. The blocks are written in chunks of
// `chunk_blocks` consecutive blocks, chunk c starting at dst + c * chunk_stride (one chunk per
// expert when a whole slot array is filled by one launch).
template <int BLOCK_BYTES>
__global__ void __launch_bounds__(256) synth_fill_kernel(uint8_t* __restrict__ dst, int64_t n_blocks,
                                                         int64_t first_block, uint64_t seed,
                                                         const uint16_t* __restrict__ d_table, int64_t chunk_blocks,
                                                         int64_t chunk_stride) {
  constexpr int kWords = (BLOCK_BYTES + 7) / 8;
  for (int64_t b = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; b < n_blocks; b += int64_t(gridDim.x) * blockDim.x) {
    const uint64_t g = uint64_t(first_block + b);
    const int64_t chunk = b / chunk_blocks;
    uint8_t* blk = dst + chunk * chunk_stride + (b - chunk * chunk_blocks) * BLOCK_BYTES;
    uint64_t w0 = 0;
#pragma unroll
    for (int i = 0; i < kWords; ++i) {
      const uint64_t w = splitmix_at(seed, g * kWords + i);
      if (i == 0) w0 = w;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int off = 8 * i + j;
        if (off >= 2 && off < BLOCK_BYTES) blk[off] = uint8_t(w >> (8 * j));
      }
    }
    const uint16_t d = d_table[w0 & 0xFFFF];
    blk[0] = uint8_t(d & 0xFF);
    blk[1] = uint8_t(d >> 8);
  }
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" {

int32_t fb_dequant_rows(int32_t format, const uint8_t* rows, int64_t row_bytes, int32_t nrows, int32_t k, float* out,
                        void* stream) {
  if (!rows || !out || nrows <= 0 || !fb_moe_row_bytes(format, k) || row_bytes < fb_moe_row_bytes(format, k))
    return invalid("dequant_rows: bad arguments");
  const int grid = (nrows + 7) / 8 < 1184 ? (nrows + 7) / 8 : 1184;
  if (format == FB_FMT_IQ3_S) {
    const size_t smem = kGridRepBytes + 64;
    static PerDeviceOnce once;
    const cudaError_t attr = per_device_once(once, [] { return opt_in_smem(dequant_iq3s_kernel, kGridRepBytes + 64); });
    if (attr != cudaSuccess) {
      set_error("dequant_rows: shared-memory opt-in: %s", cudaGetErrorString(attr));
      return int32_t(attr);
    }
    dequant_iq3s_kernel<<<grid, 256, smem, as_stream(stream)>>>(rows, row_bytes, nrows, k, out);
  } else if (format == FB_FMT_IQ4_NL) {
    dequant_iq4nl_kernel<<<grid, 256, 0, as_stream(stream)>>>(rows, row_bytes, nrows, k, out);
  } else {
    const int64_t units = int64_t(nrows) * (k / 32);
    const int g2 = int((units + 255) / 256 < 2368 ? (units + 255) / 256 : 2368);
    if (format == FB_FMT_IQ3_XXS) dequant_generic_kernel<FB_FMT_IQ3_XXS><<<g2, 256, 0, as_stream(stream)>>>(rows, row_bytes, nrows, k, out);
    else if (format == FB_FMT_IQ2_S) dequant_generic_kernel<FB_FMT_IQ2_S><<<g2, 256, 0, as_stream(stream)>>>(rows, row_bytes, nrows, k, out);
    else if (format == FB_FMT_IQ4_XS) dequant_generic_kernel<FB_FMT_IQ4_XS><<<g2, 256, 0, as_stream(stream)>>>(rows, row_bytes, nrows, k, out);
    else dequant_generic_kernel<FB_FMT_Q2_0><<<g2, 256, 0, as_stream(stream)>>>(rows, row_bytes, nrows, k, out);
  }
  return check_launch("dequant_rows");
}

int32_t fb_quantize_act(int32_t act_format, const void* x, int32_t x_dtype, int32_t rows, int32_t k, uint8_t* out,
                        void* stream) {
  if (!x || !out || rows <= 0 || !fb_act_row_bytes(act_format, k)) return invalid("quantize_act: bad arguments");
  const bool bf = x_dtype == FB_DT_BF16;
  if (act_format == FB_ACT_Q8_K) {
    const int64_t nb = int64_t(rows) * (k / 256);
    const int grid = int((nb + 7) / 8 < 1184 ? (nb + 7) / 8 : 1184);
    if (bf) quantize_q8k_kernel<true><<<grid, 256, 0, as_stream(stream)>>>(x, nb, out);
    else quantize_q8k_kernel<false><<<grid, 256, 0, as_stream(stream)>>>(x, nb, out);
  } else {
    const int64_t nb = int64_t(rows) * (k / 32);
    const int grid = int((nb + 7) / 8 < 1184 ? (nb + 7) / 8 : 1184);
    if (bf) quantize_q8_0_kernel<true><<<grid, 256, 0, as_stream(stream)>>>(x, nb, out);
    else quantize_q8_0_kernel<false><<<grid, 256, 0, as_stream(stream)>>>(x, nb, out);
  }
  return check_launch("quantize_act");
}

static int32_t synth_fill(int32_t format, uint8_t* dst, int64_t n_blocks, int64_t first_block, uint64_t seed,
                          const uint16_t* d_table, int64_t chunk_blocks, int64_t chunk_stride, void* stream) {
  const int grid = int((n_blocks + 255) / 256 < 4736 ? (n_blocks + 255) / 256 : 4736);
  if (format == FB_FMT_IQ3_S)
    synth_fill_kernel<110><<<grid, 256, 0, as_stream(stream)>>>(dst, n_blocks, first_block, seed, d_table, chunk_blocks,
                                                                chunk_stride);
  else if (format == FB_FMT_IQ4_NL || format == FB_FMT_Q2_0)
    synth_fill_kernel<18><<<grid, 256, 0, as_stream(stream)>>>(dst, n_blocks, first_block, seed, d_table, chunk_blocks,
                                                               chunk_stride);
  else if (format == FB_FMT_IQ3_XXS)
    synth_fill_kernel<98><<<grid, 256, 0, as_stream(stream)>>>(dst, n_blocks, first_block, seed, d_table, chunk_blocks,
                                                               chunk_stride);
  else if (format == FB_FMT_IQ2_S)
    synth_fill_kernel<82><<<grid, 256, 0, as_stream(stream)>>>(dst, n_blocks, first_block, seed, d_table, chunk_blocks,
                                                               chunk_stride);
  else if (format == FB_FMT_IQ4_XS)
    synth_fill_kernel<136><<<grid, 256, 0, as_stream(stream)>>>(dst, n_blocks, first_block, seed, d_table, chunk_blocks,
                                                                chunk_stride);
  else
    return invalid("synth_fill: unsupported format");
  return check_launch("synth_fill");
}

int32_t fb_synth_fill_blocks(int32_t format, uint8_t* dst, int64_t n_blocks, int64_t first_block, uint64_t seed,
                             const uint16_t* d_table, void* stream) {
  if (!dst || !d_table || n_blocks <= 0) return invalid("synth_fill_blocks: bad arguments");
  return synth_fill(format, dst, n_blocks, first_block, seed, d_table, n_blocks, 0, stream);
}

int32_t fb_synth_fill_experts(int32_t format, uint8_t* dst, int64_t expert_stride, int32_t n_experts,
                              int32_t first_expert, int64_t blocks_per_expert, uint64_t seed, const uint16_t* d_table,
                              void* stream) {
  if (!dst || !d_table || n_experts <= 0 || first_expert < 0 || blocks_per_expert <= 0 || expert_stride <= 0)
    return invalid("synth_fill_experts: bad arguments");
  return synth_fill(format, dst, int64_t(n_experts) * blocks_per_expert, int64_t(first_expert) * blocks_per_expert, seed,
                    d_table, blocks_per_expert, expert_stride, stream);
}

}  // extern "C"
