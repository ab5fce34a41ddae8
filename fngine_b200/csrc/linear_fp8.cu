// FP8-row dense projection for sm_100a: out = epilogue( (sum_k a[t][k] * w8[n][k]) * sa[t] * sw[n] )
//
//   w8, sw : E4M3 weight codes [n][k] with one scale per row (src/kernels/linear/linear.h:57-62 of the
//            reference project);
//   a, sa  : the bf16 activations, two routes as in the reference (linear.h:27-37):
//            exact (Auto / A16): each token is scaled by a power of two and written as the SUM OF TWO
//              E4M3 numbers, hi = rne(x) and lo = x - hi, which represents a bf16 value without loss
//              (eight significant bits = 4 + 4); the GEMM adds both products into one accumulator,
//              so the result is that of the reference's bf16-activation path while the weight codes
//              still go from HBM to the tensor core untouched;
//            A8: one E4M3 code per activation with scale = max|x| / 448
//              (src/kernels/linear/fp8/fp8_a8_quantize.cuh:14-26, fp8_a8.cu:22-69): half the tensor
//              work, 1-4 % rms output noise, only on request.
//
// The GEMM is a persistent tcgen05 kernel (kind::f8f6f4, E4M3 x E4M3 -> fp32 in tensor memory). One
// thread issues TMA tile loads (128-byte swizzle, no multicast) into a shared-memory ring, one
// thread issues the MMAs into one of two 256-column TMEM accumulators, four warps drain the other
// accumulator (tcgen05.ld), apply the two scales and run the epilogue (StoreBf16, StoreF32, GrWrite,
// SwiGlu, SharedScale of linear.h:64-103). All hand-offs are mbarriers; every wait is bounded and
// reports through a status word. Two variants:
//   * CTA pairs (tokens >= 256): the two-SM MMA (cta_group::2), 256 x 256 tiles per cluster of two
//     CTAs, each CTA staging its 128 token rows (one or two pieces) and its 128 weight rows per K
//     step (32 / 48 KB, six / four stages);
//   * single CTA: 128 x 256 tiles, 48 / 64 KB per K step, four / three stages.
// What the measurements said (B200, 4096 x 9216 x 2560, one piece): operand traffic is not the limit
// (a run that skips every load after the first ring fill takes the same time); the per-K-step work of
// the MMA-issuing thread is. A tcgen05 fence after each full-barrier wait and a shared-memory flag load
// in front of it cost 17 % of the kernel; with both gone the pair kernel runs at 2.4 PFLOP/s, within
// 8 % of issuing the MMAs back to back with no barriers at all (2.65 PFLOP/s), while a library FP8
// GEMM of the same shape on the same GPU reaches 2.7 - 2.9 PFLOP/s.
//
// A second operation lives here: the same weights at decode width (T <= 16) with the bf16 activations
// kept exactly and the same epilogues, a stream over the weight codes that reaches 0.9 of the HBM copy
// rate; see "decode-width projection" below. fb_linear_fp8 routes T <= 16 there.
#include "common.cuh"

#include <cuda.h>

#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace fb {
namespace {

constexpr int BM = 128, BN = 256, BK = 128, kStages = 4;      // kStages: the most stages the single-CTA ring has
constexpr int kRingBytes = kStages * (BM * BK + BN * BK);      // 196608 (1 byte per element)
constexpr int kGemmSmem = kRingBytes + 256 + 1024;             // + barriers + alignment slack
constexpr int kThreads = 192;                                  // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr uint32_t kTmemCols = 512;                            // two 256-column fp32 accumulators

// ------------------------------------------------------------------------------ PTX
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem desc] * B[smem desc], E4M3 operands, fp32 accumulate.
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 32 lanes x 32 columns of fp32: thread i of the warp receives lane (base lane + i), 32 columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzled,
// 8-row groups 1024 bytes apart (the layout the TMA box below writes): start address, leading
// offset 1 (unused for this layout), stride offset 1024 B, descriptor version 1, SWIZZLE_128B.
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_addr) {
  return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) |
         (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// Instruction descriptor: D fp32, A and B E4M3, both K-major, N = 256, M = 128.
constexpr uint32_t kIdescF8 = (1u << 4) | (0u << 7) | (0u << 10) | (uint32_t(BN >> 3) << 17) | (uint32_t(BM >> 4) << 24);

struct GemmBars {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort;
};

// Bounded wait. The barrier is tried first: the abort flag (set by a role whose own wait ran out)
// is looked at only every 32nd failed try, so the common path is one instruction.
__device__ __forceinline__ bool gemm_wait(GemmBars* b, uint64_t* bar, uint32_t parity, uint32_t* status) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 31u) == 31u && *reinterpret_cast<volatile int*>(&b->abort)) return false;
  }
  *reinterpret_cast<volatile int*>(&b->abort) = 1;
  atomicMax(status, uint32_t(FB_STATUS_PIPELINE_TIMEOUT));
  return false;
}

// ------------------------------------------------------------------------------ activation quantization
// A8 (one piece): one block per token, scale = max|x| / 448, codes = satfinite_rne_e4m3(x * (1 / scale)).
// Exact (two pieces, codes_lo given): the scale is the power of two that puts the row maximum in
// [128, 256), hi = rne_e4m3(x / scale) and lo = rne_e4m3(x / scale - hi). A bf16 value has eight
// significant bits; hi keeps four of them and the remainder is a multiple of the value's last bit of at
// most four significant bits, so lo is exact whenever that last bit is at least 2^-9 of the scaled
// range (|x| >= 2^-9..2^-10 of the row maximum); smaller elements lose bits below 2^-17 of the row
// maximum. scale * (hi + lo) therefore IS the bf16 activation: the two-piece GEMM has the numerics of
// the reference's bf16-activation path (src/kernels/linear/linear.h:27-31) on the FP8 tensor cores.
// Each thread keeps up to kQPer 16-byte pieces of the row in registers between the two phases (rows up
// to 256 * 8 * kQPer elements are read from memory once); longer rows re-read the remainder.
constexpr int kQPer = 2;

__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t pair) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(pair), __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

__global__ void __launch_bounds__(256) fp8_quantize_tokens_kernel(const __nv_bfloat16* __restrict__ x, int K,
                                                                  uint8_t* __restrict__ codes,
                                                                  uint8_t* __restrict__ codes_lo,
                                                                  float* __restrict__ scales) {
  const int t = blockIdx.x;
  const __nv_bfloat16* row = x + size_t(t) * K;
  __shared__ float s_red[8];
  uint4 held[kQPer];
  float m = 0.0f;
  auto absmax = [&](const uint4& v) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      m = fmaxf(m, fabsf(__uint_as_float(u[j] << 16)));
      m = fmaxf(m, fabsf(__uint_as_float(u[j] & 0xFFFF0000u)));
    }
  };
#pragma unroll
  for (int p = 0; p < kQPer; ++p) {
    const int i = (p * 256 + threadIdx.x) * 8;
    held[p] = i < K ? *reinterpret_cast<const uint4*>(row + i) : make_uint4(0, 0, 0, 0);
    absmax(held[p]);
  }
  for (int i = (kQPer * 256 + threadIdx.x) * 8; i < K; i += 256 * 8) absmax(*reinterpret_cast<const uint4*>(row + i));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = s_red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) m = fmaxf(m, s_red[i]);
  const bool two = codes_lo != nullptr;
  float scale, inv;
  if (two) {
    // 2^(e - 7) with 2^e <= m < 2^(e+1); rows of zeros, infinities or NaN get scale 0 (all-zero codes)
    const int e = int((__float_as_uint(m) >> 23) & 0xFFu) - 127;
    const bool ok = m > 0.0f && e < 128 && e - 7 >= -126 && 7 - e >= -126;
    scale = ok ? __uint_as_float(uint32_t(e - 7 + 127) << 23) : 0.0f;
    inv = ok ? __uint_as_float(uint32_t(7 - e + 127) << 23) : 0.0f;
  } else {
    scale = m > 0.0f ? __fdiv_rn(m, 448.0f) : 0.0f;
    inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
  }
  if (threadIdx.x == 0) scales[t] = scale;
  auto encode = [&](const uint4& v, int i) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[2] = {0, 0}, ol[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = make_float2(__fmul_rn(__uint_as_float(u[j] << 16), inv),
                                   __fmul_rn(__uint_as_float(u[j] & 0xFFFF0000u), inv));
      const uint32_t pair = __nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
      o[j >> 1] |= pair << (16 * (j & 1));
      if (two) {
        const float2 hi = e4m3x2_to_float2(pair);
        const float2 r = make_float2(__fsub_rn(f.x, hi.x), __fsub_rn(f.y, hi.y));
        ol[j >> 1] |= uint32_t(__nv_cvt_float2_to_fp8x2(r, __NV_SATFINITE, __NV_E4M3)) << (16 * (j & 1));
      }
    }
    *reinterpret_cast<uint2*>(codes + size_t(t) * K + i) = make_uint2(o[0], o[1]);
    if (two) *reinterpret_cast<uint2*>(codes_lo + size_t(t) * K + i) = make_uint2(ol[0], ol[1]);
  };
#pragma unroll
  for (int p = 0; p < kQPer; ++p) {
    const int i = (p * 256 + threadIdx.x) * 8;
    if (i < K) encode(held[p], i);
  }
  for (int i = (kQPer * 256 + threadIdx.x) * 8; i < K; i += 256 * 8) encode(*reinterpret_cast<const uint4*>(row + i), i);
}

// ------------------------------------------------------------------------------ GEMM: tiles and epilogues
// What both GEMM kernels need besides the tensor maps. An output tile is 128 (256 for a CTA pair)
// tokens x 256 weight rows, staged as two boxes of 128 weight rows: rows n0 .. n0+127 and n0+128 ..
// n0+255 of the weight, or, for SwiGlu, 128 gate rows j0 .. j0+127 and the matching up rows
// N/2 + j0 .., so that accumulator column c (gate) and column 128 + c (up) meet in one thread.
struct GemmArgs {
  const float* act_scale;   // [M] token scales
  const void* w_scale;      // [N] fp32 or bf16 row scales
  void* out;
  const float* inj;         // GrWrite: fp32 [M][4]
  const float* gate_logit;  // SharedScale
  uint32_t* status;
  int scale_bf16, kind, gate_stride;
  int M, N, K;
  int lo_row0;              // two pieces: first row of the second piece inside the activation map
};

__device__ __forceinline__ int gemm_n_tiles(const GemmArgs& a) {
  return a.kind == FB_EPI_SWIGLU ? ((a.N >> 1) + 127) / 128 : (a.N + BN - 1) / BN;
}
// First weight row of box `half` (0 / 1) of column tile n_blk.
__device__ __forceinline__ int gemm_box_row(const GemmArgs& a, int n_blk, int half) {
  return a.kind == FB_EPI_SWIGLU ? half * (a.N >> 1) + n_blk * 128 : n_blk * BN + half * 128;
}
// 32 consecutive row scales starting at row n (n % 32 == 0).
__device__ __forceinline__ void gemm_scales32(const GemmArgs& a, int n, float (&s)[32]) {
  if (a.scale_bf16) {
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.w_scale) + n);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 v = p[q];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        s[8 * q + 2 * j] = __uint_as_float(u[j] << 16);
        s[8 * q + 2 * j + 1] = __uint_as_float(u[j] & 0xFFFF0000u);
      }
    }
  } else {
    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(a.w_scale) + n);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 v = p[q];
      s[4 * q] = v.x;
      s[4 * q + 1] = v.y;
      s[4 * q + 2] = v.z;
      s[4 * q + 3] = v.w;
    }
  }
}
__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const float (&v)[32]) {
  uint32_t packed[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    packed[j] = *reinterpret_cast<const uint32_t*>(&b);
  }
  uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int j = 0; j < 4; ++j) d[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
}

// The epilogue of one token row of one tile, by the thread that owns the row's tensor-memory lane:
// `taddr` = the accumulator's address at this warp's lane quarter, column 0 of the tile; sa = the
// token scale (0 for rows past M, which are not stored).
__device__ __forceinline__ void gemm_epilogue_row(const GemmArgs& a, uint32_t taddr, int row, int n_blk, float sa) {
  const bool live = row < a.M;
  if (a.kind == FB_EPI_SWIGLU) {
    const int half_n = a.N >> 1;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t rg[32], ru[32];
      tmem_ld32(taddr + uint32_t(c * 32), rg);
      tmem_ld32(taddr + uint32_t(128 + c * 32), ru);
      const int j0 = n_blk * 128 + c * 32;
      if (live && j0 < half_n) {
        float sg[32], su[32], h[32];
        gemm_scales32(a, j0, sg);
        gemm_scales32(a, half_n + j0, su);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float g = __uint_as_float(rg[i]) * sa * sg[i], u = __uint_as_float(ru[i]) * sa * su[i];
          h[i] = g / (1.0f + expf(-g)) * u;
        }
        store_bf16x32(static_cast<__nv_bfloat16*>(a.out) + size_t(row) * half_n + j0, h);
      }
    }
    return;
  }
  if (a.kind == FB_EPI_SHARED_SCALE && live) sa /= 1.0f + expf(-a.gate_logit[size_t(row) * a.gate_stride]);
  float4 inj4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  if (a.kind == FB_EPI_GR_WRITE && live) inj4 = *reinterpret_cast<const float4*>(a.inj + size_t(row) * 4);
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr + uint32_t(c * 32), r);
    const int n0 = n_blk * BN + c * 32;
    if (!live || n0 >= a.N) continue;
    float s[32], v[32];
    gemm_scales32(a, n0, s);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * sa * s[i];
    if (a.kind == FB_EPI_STORE_BF16) {
      store_bf16x32(static_cast<__nv_bfloat16*>(a.out) + size_t(row) * a.N + n0, v);
    } else if (a.kind == FB_EPI_GR_WRITE) {
      const float inj[4] = {inj4.x, inj4.y, inj4.z, inj4.w};
#pragma unroll
      for (int s4 = 0; s4 < 4; ++s4) {
        float4* X = reinterpret_cast<float4*>(static_cast<float*>(a.out) + (size_t(row) * 4 + s4) * a.N + n0);
        float4 xv[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) xv[q] = X[q];  // all loads of a stream before its first store
#pragma unroll
        for (int q = 0; q < 8; ++q)
          X[q] = make_float4(fmaf(inj[s4], v[4 * q], xv[q].x), fmaf(inj[s4], v[4 * q + 1], xv[q].y),
                             fmaf(inj[s4], v[4 * q + 2], xv[q].z), fmaf(inj[s4], v[4 * q + 3], xv[q].w));
      }
    } else {  // StoreF32, SharedScale
      float4* d = reinterpret_cast<float4*>(static_cast<float*>(a.out) + size_t(row) * a.N + n0);
#pragma unroll
      for (int q = 0; q < 8; ++q) d[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    }
  }
}

// ------------------------------------------------------------------------------ GEMM, one CTA per tile
// PIECES activation tiles (128 tokens x 128 bytes each) and the two weight boxes per K step; the
// MMA thread adds PIECES products per K step into the same accumulator.
template <int PIECES>
struct Gemm1 {
  static constexpr int kStageA = PIECES * BM * BK, kStageB = BN * BK, kStage = kStageA + kStageB;
  static constexpr int kStages = kRingBytes / kStage;  // 4 (one piece) / 3 (two pieces)
};

template <int PIECES>
__global__ void __launch_bounds__(kThreads, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const GemmArgs a) {
  using G = Gemm1<PIECES>;
  constexpr int S = G::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmBars* bars = reinterpret_cast<GemmBars*>(smem + kRingBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (a.M + BM - 1) / BM, n_tiles = gemm_n_tiles(a), k_blocks = a.K / BK;
  const int n_work = m_tiles * n_tiles;
  uint32_t* status = a.status;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], 4);
    }
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&bars->tmem_base, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == 0) {
    // ---------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < n_work; tile += gridDim.x) {
        const int m_blk = tile % m_tiles, n_blk = tile / m_tiles;
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % S;
          if (!gemm_wait(bars, &bars->empty[s], ((it / S) & 1) ^ 1, status)) { ok = false; break; }
          uint8_t* st = smem + s * G::kStage;
          mbar_expect_tx(&bars->full[s], G::kStage);
#pragma unroll
          for (int p = 0; p < PIECES; ++p)
            tma_load_2d(st + p * BM * BK, &map_a, kb * BK, p * a.lo_row0 + m_blk * BM, &bars->full[s]);
          tma_load_2d(st + G::kStageA, &map_b, kb * BK, gemm_box_row(a, n_blk, 0), &bars->full[s]);
          tma_load_2d(st + G::kStageA + 128 * BK, &map_b, kb * BK, gemm_box_row(a, n_blk, 1), &bars->full[s]);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tl = 0;
      for (int tile = blockIdx.x; tile < n_work; tile += gridDim.x, ++tl) {
        const int ab = tl & 1;
        if (!gemm_wait(bars, &bars->tmem_empty[ab], ((tl >> 1) & 1) ^ 1, status)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(ab * BN);
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % S;
          // (no tcgen05 fence here: the operands were written through the async proxy and the
          // barrier wait orders them; a fence per K step costs a fifth of the kernel)
          if (!gemm_wait(bars, &bars->full[s], (it / S) & 1, status)) { ok = false; break; }
          const uint32_t st = smem_u32(smem + s * G::kStage);
          const uint64_t db = umma_desc_k128(st + G::kStageA);
#pragma unroll
          for (int p = 0; p < PIECES; ++p) {
            const uint64_t da = umma_desc_k128(st + p * BM * BK);
#pragma unroll
            for (int k4 = 0; k4 < BK / 32; ++k4)  // 32 bytes of K per instruction: +2 in 16-byte units
              umma_f8(d_tmem, da + uint64_t(2 * k4), db + uint64_t(2 * k4), kIdescF8, (kb | k4 | p) ? 1u : 0u);
          }
          umma_commit(&bars->empty[s]);  // stage reusable once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(&bars->tmem_full[ab]);  // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue warps 2..5: TMEM lane quarter = warp % 4
    const int q = warp & 3;
    uint32_t tl = 0;
    for (int tile = blockIdx.x; tile < n_work; tile += gridDim.x, ++tl) {
      const int m_blk = tile % m_tiles, n_blk = tile / m_tiles;
      const int ab = tl & 1;
      if (!gemm_wait(bars, &bars->tmem_full[ab], (tl >> 1) & 1, status)) break;
      tc_fence_after();
      const int row = m_blk * BM + q * 32 + lane;
      const float sa = row < a.M ? a.act_scale[row] : 0.0f;
      gemm_epilogue_row(a, tmem_base + (uint32_t(q * 32) << 16) + uint32_t(ab * BN), row, n_blk, sa);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[ab]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------ GEMM on CTA pairs
// The same GEMM with the two-SM MMA (cta_group::2): a cluster of two CTAs computes a 256 x 256 output
// tile, CTA r of the pair holding A rows [128 r, 128 r + 128) and B rows (output columns)
// [128 r, 128 r + 128) of every K step, so each SM stages 32 KB per K step instead of 48 KB and the
// tensor cores of the pair share the B halves. Each CTA keeps its 128 x 256 half of the accumulator
// in its own tensor memory. Barrier protocol (one pipeline, CTA 0 is the leader):
//   full[s]   lives in the leader: its producer arms it with the bytes of BOTH CTAs, both CTAs' TMA
//             loads complete on it (barrier address with the peer bit cleared);
//   empty[s]  in each CTA, freed for both by one multicast commit of the leader's MMA thread;
//   tmem_full[a] in each CTA, same multicast commit; tmem_empty[a] in the leader, eight arrivals
//             (four epilogue warps per CTA, CTA 1's through the cluster window).
// No TMA load is multicast: each CTA loads only its own operand halves.
constexpr int BM2 = 256, kStages2 = 6;                               // kStages2: the most stages the pair ring has
constexpr int kRingBytes2 = kStages2 * (128 * BK + 128 * BK);         // 196608 per CTA
constexpr int kGemmSmem2 = kRingBytes2 + 256 + 1024;
constexpr uint32_t kIdescF8Pair = (1u << 4) | (uint32_t(BN >> 3) << 17) | (uint32_t(BM2 >> 4) << 24);
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;  // clears the bit that separates the two CTAs of a pair

struct GemmBars2 {
  uint64_t full[kStages2];
  uint64_t empty[kStages2];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint64_t* leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(leader_bar) & kPeerBitMask)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(static_cast<unsigned short>(3))
      : "memory");
}
// Arrive on the leader CTA's copy of `bar`.
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\tmapa.shared::cluster.u32 ra, %0, 0;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}"
      ::"r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ bool gemm_wait2(GemmBars2* b, uint64_t* bar, uint32_t parity, uint32_t* status) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 31u) == 31u && *reinterpret_cast<volatile int*>(&b->abort)) return false;  // a peer role gave up
  }
  *reinterpret_cast<volatile int*>(&b->abort) = 1;
  atomicMax(status, uint32_t(FB_STATUS_PIPELINE_TIMEOUT));
  return false;
}

template <int PIECES>
struct Gemm2 {
  static constexpr int kStageA = PIECES * 128 * BK, kStageB = 128 * BK, kStage = kStageA + kStageB;  // per CTA
  static constexpr int kStages = kRingBytes2 / kStage;  // 6 (one piece) / 4 (two pieces)
};

template <int PIECES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
fp8_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const GemmArgs a) {
  using G = Gemm2<PIECES>;
  constexpr int S = G::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmBars2* bars = reinterpret_cast<GemmBars2*>(smem + kRingBytes2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = int(cluster_ctarank());
  const int m_tiles = (a.M + BM2 - 1) / BM2, n_tiles = gemm_n_tiles(a), k_blocks = a.K / BK;
  const int n_work = m_tiles * n_tiles, pair = int(blockIdx.x) >> 1, n_pairs = int(gridDim.x) >> 1;
  uint32_t* status = a.status;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], 8);
    }
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc_pair(&bars->tmem_base, kTmemCols);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs): own token rows and own weight box, completion on the leader's barrier
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = pair; tile < n_work; tile += n_pairs) {
        const int m_blk = tile % m_tiles, n_blk = tile / m_tiles;
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % S;
          if (!gemm_wait2(bars, &bars->empty[s], ((it / S) & 1) ^ 1, status)) { ok = false; break; }
          uint8_t* st = smem + s * G::kStage;
          if (rank == 0) mbar_expect_tx(&bars->full[s], 2 * G::kStage);
#pragma unroll
          for (int p = 0; p < PIECES; ++p)
            tma_load_2d_pair(st + p * 128 * BK, &map_a, kb * BK, p * a.lo_row0 + m_blk * BM2 + rank * 128, &bars->full[s]);
          tma_load_2d_pair(st + G::kStageA, &map_b, kb * BK, gemm_box_row(a, n_blk, rank), &bars->full[s]);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      uint32_t it = 0, tl = 0;
      for (int tile = pair; tile < n_work; tile += n_pairs, ++tl) {
        const int ab = tl & 1;
        if (!gemm_wait2(bars, &bars->tmem_empty[ab], ((tl >> 1) & 1) ^ 1, status)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(ab * BN);
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % S;
          if (!gemm_wait2(bars, &bars->full[s], (it / S) & 1, status)) { ok = false; break; }
          const uint32_t st = smem_u32(smem + s * G::kStage);
          const uint64_t db = umma_desc_k128(st + G::kStageA);
#pragma unroll
          for (int p = 0; p < PIECES; ++p) {
            const uint64_t da = umma_desc_k128(st + p * 128 * BK);
#pragma unroll
            for (int k4 = 0; k4 < BK / 32; ++k4)
              umma_f8_pair(d_tmem, da + uint64_t(2 * k4), db + uint64_t(2 * k4), kIdescF8Pair, (kb | k4 | p) ? 1u : 0u);
          }
          umma_commit_pair(&bars->empty[s]);
        }
        if (!ok) break;
        umma_commit_pair(&bars->tmem_full[ab]);
      }
    }
  } else {
    // ---------------- epilogue warps 2..5 of each CTA: its 128 token rows of the pair's tile
    const int q = warp & 3;
    uint32_t tl = 0;
    for (int tile = pair; tile < n_work; tile += n_pairs, ++tl) {
      const int m_blk = tile % m_tiles, n_blk = tile / m_tiles;
      const int ab = tl & 1;
      if (!gemm_wait2(bars, &bars->tmem_full[ab], (tl >> 1) & 1, status)) break;
      tc_fence_after();
      const int row = m_blk * BM2 + rank * 128 + q * 32 + lane;
      const float sa = row < a.M ? a.act_scale[row] : 0.0f;
      gemm_epilogue_row(a, tmem_base + (uint32_t(q * 32) << 16) + uint32_t(ab * BN), row, n_blk, sa);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&bars->tmem_empty[ab]);
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody leaves (or frees tensor memory) while the peer may still signal or read
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------ decode-width projection
// T <= 16 tokens with the activations kept exactly (the reference's "A16" numerics: exact E4M3
// weights x the represented bf16 activation, fp32 accumulation, one multiplication by the row
// scale; src/kernels/linear/linear.h:27-31, fp8/fp8_gemv.cuh:8-12). The operation is a stream over
// the weight codes, so nothing may stand between HBM and the tensor core: the codes go from the
// TMA box straight into tcgen05.mma as the E4M3 A operand, with no widening pass. The bf16
// activations become the B operand without loss by writing each one as a sum of three E5M2
// numbers: after a per-token power-of-two scale that puts the row maximum in [2^14, 2^15), round to
// nearest E5M2 (three significant bits), subtract, and repeat twice; the second remainder has one
// significant bit and the third piece is exact (values below 2^-16 of the scaled range, 2^-30 of the
// row maximum, are dropped). The three pieces of the sixteen token slots are 48 B-operand rows, so
// one MMA of N = 48 per 32 bytes of K produces three partial columns per token, which the epilogue
// adds (smallest first) before the token and row scales.
//
// Work is cut stream-K fashion: the (row tile, K block) sequence is divided evenly over the
// resident CTAs, so every shape - 1940 row tiles of the vocabulary projection or 10 of the
// shared expert - keeps all SMs streaming. A CTA whose range covers a whole row tile finishes it
// from tensor memory; partial ranges leave fp32 partial sums in the workspace and the last CTA to
// arrive at a tile (a ticket) adds them in CTA order, which is fixed for a shape: results are
// deterministic.
constexpr int kDecTok = 16;                              // token slots per piece
constexpr int kDecN = 3 * kDecTok;                       // B-operand rows
constexpr int kDecStages = 8;
constexpr int kDecStageA = 128 * BK;                     // 16 KB of weight codes
constexpr int kDecStageB = kDecN * BK;                   // 6 KB of activation pieces
constexpr int kDecStage = kDecStageA + kDecStageB;       // 22 KB, a multiple of the 1024-byte swizzle atom
constexpr int kDecXchFloats = 128 * 17;
constexpr int kDecSmem = kDecStages * kDecStage + kDecXchFloats * 4 + 256 + 1024;
constexpr uint32_t kDecTmemCols = 128;                   // two accumulators of 64 columns (48 used)
constexpr int kDecPartialFloats = 128 * kDecTok;         // one partial tile
// D fp32, A = E4M3 (format 0), B = E5M2 (format 1), both K-major, N = 48, M = 128.
constexpr uint32_t kIdescDec = (1u << 4) | (0u << 7) | (1u << 10) | (uint32_t(kDecN >> 3) << 17) | (uint32_t(128 >> 4) << 24);
static_assert(kDecStage % 1024 == 0 && kDecStageA % 1024 == 0, "operand tiles start on swizzle atoms");

struct DecArgs {
  const float* tok_scale;   // [16] power-of-two scale of each token's pieces
  const void* w_scale;      // [n] fp32 or bf16
  int scale_bf16;
  int kind;                 // FB_EPI_*
  void* out;
  const float* inj;         // GrWrite: [T][4]
  const float* gate_logit;  // SharedScale: logit of token t at gate_logit[t * gate_stride]
  int gate_stride;
  int T, n, k;
  float* partial;           // [2 * grid][16][128] fp32
  int32_t* tickets;         // [row tiles], zero at kernel start
  uint32_t* status;
};

struct DecBars {
  uint64_t full[kDecStages];
  uint64_t empty[kDecStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort;
  int last;
};
static_assert(sizeof(DecBars) <= 256, "barrier block");

__device__ __forceinline__ bool dec_wait(DecBars* b, uint64_t* bar, uint32_t parity, uint32_t* status) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 31u) == 31u && *reinterpret_cast<volatile int*>(&b->abort)) return false;
  }
  *reinterpret_cast<volatile int*>(&b->abort) = 1;
  atomicMax(status, uint32_t(FB_STATUS_PIPELINE_TIMEOUT));
  return false;
}
// Adds to the pending byte count of a barrier without arriving on it.
__device__ __forceinline__ void mbar_expect_tx_only(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// All `threads` threads of named barrier `id` learn whether every one of them passed `ok`.
__device__ __forceinline__ bool named_bar_all(int id, int threads, bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %3, 0;\n\t"
      "barrier.cta.red.and.pred p, %1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(id), "r"(threads), "r"(uint32_t(ok))
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ float e5m2_to_float(uint32_t code) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(code << 8)));  // E5M2 = the top byte of binary16
}
__device__ __forceinline__ uint32_t float_to_e5m2(float v) {
  return uint32_t(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2));  // round to nearest even
}

constexpr int kSplitPer = 5;  // 16-byte pieces of a row a thread keeps in registers (rows up to 10240 values)

// One block per token slot. pieces[(p * 16 + t) * K + j], p = 0..2; slots >= T are zero rows. Block 0
// also clears the tickets and the status word of the projection that follows.
__global__ void __launch_bounds__(256) fp8_split_tokens_kernel(const __nv_bfloat16* __restrict__ x, int T, int K,
                                                               uint8_t* __restrict__ pieces,
                                                               float* __restrict__ tok_scale,
                                                               int32_t* __restrict__ tickets, int n_tickets,
                                                               uint32_t* __restrict__ status) {
  pdl_launch_dependents();
  const int t = blockIdx.x, tid = threadIdx.x;
  if (t == 0) {
    for (int i = tid; i < n_tickets; i += 256) tickets[i] = 0;
    if (tid == 0) *status = 0;
  }
  uint8_t* piece[3] = {pieces + size_t(t) * K, pieces + size_t(kDecTok + t) * K, pieces + size_t(2 * kDecTok + t) * K};
  if (t >= T) {
    for (int i = tid; i < K / 8; i += 256)
#pragma unroll
      for (int p = 0; p < 3; ++p) reinterpret_cast<uint2*>(piece[p])[i] = make_uint2(0u, 0u);
    if (tid == 0) tok_scale[t] = 0.0f;
    return;
  }
  const uint4* row = reinterpret_cast<const uint4*>(x + size_t(t) * K);
  // the row stays in registers between the two phases (up to 256 * 8 * kSplitPer values; longer rows
  // re-read the remainder)
  uint4 keep[kSplitPer];
  float m = 0.0f;
#pragma unroll
  for (int j = 0; j < kSplitPer; ++j) {
    const int i = tid + j * 256;
    keep[j] = i < K / 8 ? row[i] : make_uint4(0u, 0u, 0u, 0u);
    const uint32_t w[4] = {keep[j].x, keep[j].y, keep[j].z, keep[j].w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      m = fmaxf(m, fabsf(__uint_as_float(w[q] << 16)));
      m = fmaxf(m, fabsf(__uint_as_float(w[q] & 0xFFFF0000u)));
    }
  }
  for (int i = tid + kSplitPer * 256; i < K / 8; i += 256) {
    const uint4 v = row[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      m = fmaxf(m, fabsf(__uint_as_float(w[q] << 16)));
      m = fmaxf(m, fabsf(__uint_as_float(w[q] & 0xFFFF0000u)));
    }
  }
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  if ((tid & 31) == 0) red[tid >> 5] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
  // scale = 2^(exponent(max) - 14): the scaled maximum lies in [2^14, 2^15), so rounding up stays finite
  uint32_t e = (__float_as_uint(m) >> 23) & 0xFFu;
  e = e < 15u ? 15u : (e > 253u ? 253u : e);
  const float scale = __uint_as_float((e - 14u) << 23), inv = __uint_as_float((268u - e) << 23);
  auto split8 = [&](const uint4 v, int i) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t out[3][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t bits = (j & 1) ? (w[j >> 1] & 0xFFFF0000u) : (w[j >> 1] << 16);
      float r = __uint_as_float(bits) * inv;
#pragma unroll
      for (int p = 0; p < 3; ++p) {
        const uint32_t c = float_to_e5m2(r);
        r -= e5m2_to_float(c);
        out[p][j >> 2] |= c << (8 * (j & 3));
      }
    }
#pragma unroll
    for (int p = 0; p < 3; ++p) reinterpret_cast<uint2*>(piece[p])[i] = make_uint2(out[p][0], out[p][1]);
  };
#pragma unroll
  for (int j = 0; j < kSplitPer; ++j) {
    const int i = tid + j * 256;
    if (i < K / 8) split8(keep[j], i);
  }
  for (int i = tid + kSplitPer * 256; i < K / 8; i += 256) split8(row[i], i);
  if (tid == 0) tok_scale[t] = scale;
}

// First K-block position of CTA c when `total` positions are divided over G CTAs.
__device__ __forceinline__ long long dec_begin(int c, int G, long long total) { return (total * c) / G; }
// The CTA whose range holds position p.
__device__ __forceinline__ int dec_owner(long long p, int G, long long total) {
  int c = int((p * G) / total);
  while (c + 1 < G && dec_begin(c + 1, G, total) <= p) ++c;
  while (c > 0 && dec_begin(c, G, total) > p) --c;
  return c;
}

__device__ __forceinline__ float dec_row_scale(const DecArgs& a, int row) {
  return a.scale_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.w_scale)[row])
                      : static_cast<const float*>(a.w_scale)[row];
}

// Finishes row tile m: v[t] is the K-complete sum of tile row `rl` for token slot t, before scales.
// Called by all 128 epilogue threads (et = 0..127; rl is the thread's tensor-memory lane).
// Row scale of tile row rl of tile m (0 outside the matrix). SwiGlu tiles hold 64 gate rows, then the 64
// matching up rows.
__device__ __forceinline__ float dec_tile_row_scale(const DecArgs& a, int m, int rl) {
  if (a.kind == FB_EPI_SWIGLU) {
    const int half_n = a.n >> 1, j = m * 64 + (rl & 63);
    return j < half_n ? dec_row_scale(a, rl < 64 ? j : half_n + j) : 0.0f;
  }
  const int row = m * 128 + rl;
  return row < a.n ? dec_row_scale(a, row) : 0.0f;
}

// ts[t] = token scale (times sigmoid(gate logit) for SharedScale), ws = the row scale of this thread's
// tile row (dec_tile_row_scale): both are fetched by the caller before it waits for the tile, so no
// memory round trip stands between the accumulator and the stores.
__device__ __forceinline__ void dec_emit(const DecArgs& a, int m, int rl, int et, const float (&v)[kDecTok],
                                         const float (&ts)[kDecTok], float ws, float* xch) {
  if (a.kind == FB_EPI_SWIGLU) {
    // tile rows 0..63 are gate rows m*64.., rows 64..127 the matching up rows
    const int half_n = a.n >> 1;
#pragma unroll
    for (int t = 0; t < kDecTok; ++t) xch[rl * 17 + t] = v[t] * ts[t] * ws;
    named_bar_sync(2, 128);
    const int r = et & 63, t0 = (et >> 6) * 8, jo = m * 64 + r;
    if (jo < half_n) {
      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(a.out);
#pragma unroll
      for (int t = t0; t < t0 + 8; ++t)
        if (t < a.T) {
          const float g = xch[r * 17 + t], u = xch[(r + 64) * 17 + t];
          out[size_t(t) * half_n + jo] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
        }
    }
    named_bar_sync(2, 128);
    return;
  }
  const int row = m * 128 + rl;
  if (row >= a.n) return;
  if (a.kind == FB_EPI_GR_WRITE) {
    // X[t][s][row] += inj[t][s] * val. All loads first: interleaved with the stores they would be
    // issued one memory round trip at a time.
    float* xs = static_cast<float*>(a.out) + row;
    const size_t n = size_t(a.n);
#pragma unroll
    for (int h = 0; h < kDecTok; h += 8) {  // eight tokens at a time: 32 values in registers
      if (h >= a.T) break;
      float x4[8][4];
#pragma unroll
      for (int t = 0; t < 8; ++t)
        if (h + t < a.T) {
#pragma unroll
          for (int st = 0; st < 4; ++st) x4[t][st] = __ldcg(xs + (size_t(h + t) * 4 + st) * n);
        }
#pragma unroll
      for (int t = 0; t < 8; ++t)
        if (h + t < a.T) {
          const float val = v[h + t] * ts[h + t] * ws;
          const float4 g = __ldg(reinterpret_cast<const float4*>(a.inj + size_t(h + t) * 4));
          xs[(size_t(h + t) * 4 + 0) * n] = fmaf(g.x, val, x4[t][0]);
          xs[(size_t(h + t) * 4 + 1) * n] = fmaf(g.y, val, x4[t][1]);
          xs[(size_t(h + t) * 4 + 2) * n] = fmaf(g.z, val, x4[t][2]);
          xs[(size_t(h + t) * 4 + 3) * n] = fmaf(g.w, val, x4[t][3]);
        }
    }
    return;
  }
#pragma unroll
  for (int t = 0; t < kDecTok; ++t) {
    if (t >= a.T) break;
    const float val = v[t] * ts[t] * ws;
    if (a.kind == FB_EPI_STORE_BF16)
      static_cast<__nv_bfloat16*>(a.out)[size_t(t) * a.n + row] = __float2bfloat16_rn(val);
    else
      static_cast<float*>(a.out)[size_t(t) * a.n + row] = val;  // StoreF32, SharedScale
  }
}

// v[t] (t < TT) = sum over the CTAs c_first..c_last that hold a part of row tile m, in CTA order: fixed, so
// results do not depend on the order of arrival. Two contributors' loads are in flight at a time, six with at
// most four tokens (usually the whole list in one round trip).
template <int TT>
__device__ __forceinline__ void dec_sum_partials(const DecArgs& a, int m, int rl, int c_first, int c_last, int G,
                                                 long long total, int kbt, float (&v)[kDecTok]) {
  constexpr int kPer = TT == 16 ? 2 : 6;
  for (int c0 = c_first; c0 <= c_last; c0 += kPer) {
    float part[kPer][TT];
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int cc = c0 + i;
      if (cc <= c_last) {
        // a contributor's range meets the tile; it is the CTA's first segment iff the range starts inside it
        // (floor(total * cc / G) >= m * kbt without the division)
        const bool first_seg = total * cc >= (long long)m * kbt * G;
        const float* theirs = a.partial + size_t(2 * cc + (first_seg ? 0 : 1)) * kDecPartialFloats;
#pragma unroll
        for (int t = 0; t < TT; ++t) part[i][t] = __ldcg(theirs + t * 128 + rl);
      }
    }
#pragma unroll
    for (int i = 0; i < kPer; ++i)
      if (c0 + i <= c_last) {
#pragma unroll
        for (int t = 0; t < TT; ++t) v[t] += part[i][t];
      }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
fp8_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_p,
                  const __grid_constant__ DecArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  float* xch = reinterpret_cast<float*>(smem + kDecStages * kDecStage);
  DecBars* bars = reinterpret_cast<DecBars*>(smem + kDecStages * kDecStage + kDecXchFloats * 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool swiglu = a.kind == FB_EPI_SWIGLU;
  const int kbt = a.k / BK;
  const int m_tiles = swiglu ? ((a.n >> 1) + 63) / 64 : (a.n + 127) / 128;
  const int G = int(gridDim.x);
  const long long total = (long long)m_tiles * kbt;
  const long long begin = dec_begin(int(blockIdx.x), G, total), end = dec_begin(int(blockIdx.x) + 1, G, total);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kDecStages; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], 4);
    }
    bars->abort = 0;
    bars->last = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&bars->tmem_base, kDecTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == 0) {
    // ---------------- TMA producer: 128 weight rows (two 64-row boxes) + the 48 piece rows per K block
    if (lane == 0) {
      // The weight codes do not depend on the kernel launched just before (the activation split), so
      // the first ring's worth of them is requested before waiting for it: under programmatic
      // dependent launch this kernel is resident while the split still runs.
      const int pre = end - begin < kDecStages ? int(end - begin) : kDecStages;
      for (int i = 0; i < pre; ++i) {
        const long long pos = begin + i;
        const int m = int(pos / kbt), kb = int(pos - (long long)m * kbt);
        const int r0 = swiglu ? m * 64 : m * 128, r1 = swiglu ? (a.n >> 1) + m * 64 : m * 128 + 64;
        uint8_t* st = ring + i * kDecStage;
        mbar_expect_tx_only(&bars->full[i], kDecStageA);
        tma_load_2d(st, &map_w, kb * BK, r0, &bars->full[i]);
        tma_load_2d(st + 64 * BK, &map_w, kb * BK, r1, &bars->full[i]);
      }
      pdl_wait_prior();  // the pieces are written by the kernel launched just before
      uint32_t it = 0;
      bool ok = true;
      for (long long pos = begin; pos < end && ok;) {
        const int m = int(pos / kbt), kb0 = int(pos - (long long)m * kbt);
        const int kb1 = int(end - pos) < kbt - kb0 ? kb0 + int(end - pos) : kbt;
        const int r0 = swiglu ? m * 64 : m * 128, r1 = swiglu ? (a.n >> 1) + m * 64 : m * 128 + 64;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kDecStages;
          uint8_t* st = ring + s * kDecStage;
          if (it < uint32_t(pre)) {  // codes already requested: add the pieces and the arrival
            mbar_expect_tx(&bars->full[s], kDecStageB);
            tma_load_2d(st + kDecStageA, &map_p, kb * BK, 0, &bars->full[s]);
            continue;
          }
          if (!dec_wait(bars, &bars->empty[s], ((it / kDecStages) & 1) ^ 1, a.status)) { ok = false; break; }
          mbar_expect_tx(&bars->full[s], kDecStage);
          tma_load_2d(st, &map_w, kb * BK, r0, &bars->full[s]);
          tma_load_2d(st + 64 * BK, &map_w, kb * BK, r1, &bars->full[s]);
          tma_load_2d(st + kDecStageA, &map_p, kb * BK, 0, &bars->full[s]);
        }
        pos += kb1 - kb0;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (lane == 0) {
      uint32_t it = 0, seg = 0;
      bool ok = true;
      for (long long pos = begin; pos < end && ok; ++seg) {
        const int m = int(pos / kbt), kb0 = int(pos - (long long)m * kbt);
        const int kb1 = int(end - pos) < kbt - kb0 ? kb0 + int(end - pos) : kbt;
        const int ab = seg & 1;
        if (!dec_wait(bars, &bars->tmem_empty[ab], ((seg >> 1) & 1) ^ 1, a.status)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(ab * 64);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kDecStages;
          if (!dec_wait(bars, &bars->full[s], (it / kDecStages) & 1, a.status)) { ok = false; break; }
          uint8_t* st = ring + s * kDecStage;
          const uint64_t da = umma_desc_k128(smem_u32(st)), db = umma_desc_k128(smem_u32(st + kDecStageA));
#pragma unroll
          for (int k4 = 0; k4 < BK / 32; ++k4)
            umma_f8(d_tmem, da + uint64_t(2 * k4), db + uint64_t(2 * k4), kIdescDec, (kb > kb0 || k4) ? 1u : 0u);
          umma_commit(&bars->empty[s]);
        }
        if (!ok) break;
        umma_commit(&bars->tmem_full[ab]);
        pos += kb1 - kb0;
      }
    }
  } else {
    // ---------------- epilogue warps 2..5: tensor-memory lane quarter = warp % 4
    const int q = warp & 3, rl = q * 32 + lane, et = (warp - 2) * 32 + lane;
    pdl_wait_prior();  // token scales and cleared tickets come from the kernel launched just before
    float ts[kDecTok];
#pragma unroll
    for (int t4 = 0; t4 < kDecTok / 4; ++t4) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(a.tok_scale) + t4);
      ts[4 * t4] = f.x, ts[4 * t4 + 1] = f.y, ts[4 * t4 + 2] = f.z, ts[4 * t4 + 3] = f.w;
    }
    if (a.kind == FB_EPI_SHARED_SCALE) {  // sigmoid(gate logit) folded into the token scale
      float gl[kDecTok];
#pragma unroll
      for (int t = 0; t < kDecTok; ++t)  // all loads first: the division below branches, and loads do not move across it
        gl[t] = __ldg(a.gate_logit + size_t(t < a.T ? t : 0) * a.gate_stride);
#pragma unroll
      for (int t = 0; t < kDecTok; ++t) ts[t] /= 1.0f + expf(-gl[t]);
    }
    uint32_t seg = 0;
    for (long long pos = begin; pos < end; ++seg) {
      const int m = int(pos / kbt), kb0 = int(pos - (long long)m * kbt);
      const int kb1 = int(end - pos) < kbt - kb0 ? kb0 + int(end - pos) : kbt;
      const int ab = seg & 1;
      const float ws = dec_tile_row_scale(a, m, rl);
      const bool got = dec_wait(bars, &bars->tmem_full[ab], (seg >> 1) & 1, a.status);
      if (!named_bar_all(1, 128, got)) break;  // the four warps leave together
      tc_fence_after();
      uint32_t c[kDecN];
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(ab * 64);
      tmem_ld16_nowait(taddr, c);
      tmem_ld16_nowait(taddr + 16, c + 16);
      tmem_ld16_nowait(taddr + 32, c + 32);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      float v[kDecTok];
#pragma unroll
      for (int t = 0; t < kDecTok; ++t)
        v[t] = (__uint_as_float(c[32 + t]) + __uint_as_float(c[16 + t])) + __uint_as_float(c[t]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[ab]);
      if (kb0 == 0 && kb1 == kbt) {
        dec_emit(a, m, rl, et, v, ts, ws, xch);
      } else {
        // a partial range: leave the sums in this CTA's slot (first segment: slot 0, a later one: 1)
        float* mine = a.partial + size_t(2 * blockIdx.x + (pos == begin ? 0 : 1)) * kDecPartialFloats;
#pragma unroll
        for (int t = 0; t < kDecTok; ++t) __stcg(mine + t * 128 + rl, v[t]);
        __threadfence();
        named_bar_sync(1, 128);
        const int c_first = dec_owner((long long)m * kbt, G, total);
        const int c_last = dec_owner((long long)(m + 1) * kbt - 1, G, total);
        if (et == 0) bars->last = atomicAdd(&a.tickets[m], 1) == c_last - c_first ? 1 : 0;
        named_bar_sync(1, 128);
        if (*reinterpret_cast<volatile int*>(&bars->last)) {
          __threadfence();
#pragma unroll
          for (int t = 0; t < kDecTok; ++t) v[t] = 0.0f;
          if (a.T <= 4) dec_sum_partials<4>(a, m, rl, c_first, c_last, G, total, kbt, v);
          else dec_sum_partials<16>(a, m, rl, c_first, c_last, G, total, kbt, v);
          dec_emit(a, m, rl, et, v, ts, ws, xch);
        }
      }
      pos += kb1 - kb0;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kDecTmemCols);
  }
}

// ------------------------------------------------------------------------------ host
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// uint8 [rows][k] row-major, boxes of 128 bytes x box_rows, 128-byte swizzle, zero fill outside.
bool make_map_u8(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(k)};
  const cuuint32_t box[2] = {cuuint32_t(BK), cuuint32_t(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

// CTA pairs of the two-SM kernel that can be resident at once (asked of the occupancy calculator once per device).
int pair_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return sm_count() / 2;
  if (!cached[dev]) {
    opt_in_smem(fp8_gemm_pair_kernel<1>, kGemmSmem2);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(sm_count()) & ~1u);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kGemmSmem2;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, fp8_gemm_pair_kernel<1>, &cfg) != cudaSuccess || clusters < 1) {
      cudaGetLastError();
      clusters = sm_count() / 2;
    }
    cached[dev] = clusters;
  }
  return cached[dev];
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" {

size_t fb_linear_fp8_workspace_bytes(int32_t n, int32_t k, int32_t max_tokens) {
  if (n <= 0 || k <= 0 || max_tokens <= 0) return 0;
  // two activation pieces [2][T][k] | token scales | status; at T <= 16 the decode-width projection's scratch
  const size_t gemm = align256(size_t(2) * size_t(max_tokens) * size_t(k)) + align256(size_t(max_tokens) * 4) + 256;
  const size_t dec = fb_linear_fp8_decode_workspace_bytes(n, k);
  return gemm > dec ? gemm : dec;
}

int32_t fb_fp8_quantize_tokens(const void* x_bf16, int32_t tokens, int32_t k, uint8_t* codes, float* scales,
                               void* stream) {
  if (!x_bf16 || !codes || !scales || tokens <= 0 || k <= 0 || k % 8)
    return invalid("fp8_quantize_tokens: bad arguments (k must be a multiple of 8)");
  fp8_quantize_tokens_kernel<<<tokens, 256, 0, as_stream(stream)>>>(static_cast<const __nv_bfloat16*>(x_bf16), k, codes,
                                                                    nullptr, scales);
  return check_launch("fp8_quantize_tokens");
}

int32_t fb_fp8_split_tokens(const void* x_bf16, int32_t tokens, int32_t k, uint8_t* codes_hi, uint8_t* codes_lo,
                            float* scales, void* stream) {
  if (!x_bf16 || !codes_hi || !codes_lo || !scales || tokens <= 0 || k <= 0 || k % 8)
    return invalid("fp8_split_tokens: bad arguments (k must be a multiple of 8)");
  fp8_quantize_tokens_kernel<<<tokens, 256, 0, as_stream(stream)>>>(static_cast<const __nv_bfloat16*>(x_bf16), k, codes_hi,
                                                                    codes_lo, scales);
  return check_launch("fp8_split_tokens");
}

int32_t fb_linear_fp8(const void* x_bf16, int32_t tokens, const uint8_t* w_codes, const void* w_scales,
                      int32_t w_scales_dtype, int32_t n, int32_t k, const fb_linear_epilogue* epilogue, void* workspace,
                      size_t workspace_bytes, void* stream, int32_t path) {
  if (!x_bf16 || !w_codes || !w_scales || !epilogue || !epilogue->out || tokens <= 0)
    return invalid("linear_fp8: null argument or no tokens");
  if (path != FB_FP8_PATH_AUTO && path != FB_FP8_PATH_A16 && path != FB_FP8_PATH_A8)
    return invalid("linear_fp8: unknown path");
  // decode width on the exact routes: the streaming projection (same numerics, tuned for T <= 16)
  if (tokens <= kDecTok && path != FB_FP8_PATH_A8)
    return fb_linear_fp8_decode(x_bf16, tokens, w_codes, w_scales, w_scales_dtype, n, k, epilogue, workspace,
                                workspace_bytes, stream);
  const int kind = epilogue->kind;
  if (kind < FB_EPI_STORE_BF16 || kind > FB_EPI_SHARED_SCALE) return invalid("linear_fp8: unknown epilogue");
  if (n <= 0 || k <= 0 || n % 64 || k % BK)
    return invalid("linear_fp8: unsupported shape (n must be a multiple of 64, k of 128)");
  if (kind == FB_EPI_SWIGLU && n % 128) return invalid("linear_fp8: SwiGlu needs n %% 128 == 0");
  if (kind == FB_EPI_GR_WRITE && (!epilogue->inj || (reinterpret_cast<uintptr_t>(epilogue->inj) & 15)))
    return invalid("linear_fp8: GrWrite needs inj fp32 [tokens][4], 16-byte aligned");
  if (kind == FB_EPI_SHARED_SCALE && !epilogue->gate_logit) return invalid("linear_fp8: SharedScale needs gate_logit");
  if ((reinterpret_cast<uintptr_t>(w_codes) | reinterpret_cast<uintptr_t>(x_bf16) |
       reinterpret_cast<uintptr_t>(epilogue->out) | reinterpret_cast<uintptr_t>(w_scales)) & 15)
    return invalid("linear_fp8: x, weight codes, row scales and out must be 16-byte aligned");
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
      workspace_bytes < fb_linear_fp8_workspace_bytes(n, k, tokens))
    return invalid("linear_fp8: workspace missing, misaligned (256 B) or smaller than fb_linear_fp8_workspace_bytes");
  const int pieces = path == FB_FP8_PATH_A8 ? 1 : 2;
  uint8_t* a_codes = static_cast<uint8_t*>(workspace);
  uint8_t* a_lo = pieces == 2 ? a_codes + size_t(tokens) * size_t(k) : nullptr;  // directly behind: one tensor map
  float* a_scales = reinterpret_cast<float*>(a_codes + align256(size_t(2) * size_t(tokens) * size_t(k)));
  uint32_t* status = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(a_scales) + align256(size_t(tokens) * 4));
  fp8_quantize_tokens_kernel<<<tokens, 256, 0, as_stream(stream)>>>(static_cast<const __nv_bfloat16*>(x_bf16), k, a_codes,
                                                                    a_lo, a_scales);
  int32_t st = check_launch("linear_fp8: activation pieces");
  if (st) return st;
  static PerDeviceOnce once;
  const cudaError_t attr = per_device_once(once, [] {
    cudaError_t a = opt_in_smem(fp8_gemm_kernel<1>, kGemmSmem);
    if (a == cudaSuccess) a = opt_in_smem(fp8_gemm_kernel<2>, kGemmSmem);
    if (a == cudaSuccess) a = opt_in_smem(fp8_gemm_pair_kernel<1>, kGemmSmem2);
    if (a == cudaSuccess) a = opt_in_smem(fp8_gemm_pair_kernel<2>, kGemmSmem2);
    return a;
  });
  if (attr != cudaSuccess) {
    set_error("linear_fp8: shared-memory opt-in: %s", cudaGetErrorString(attr));
    return int32_t(attr);
  }
  cudaError_t e = cudaMemsetAsync(status, 0, 4, as_stream(stream));
  if (e != cudaSuccess) return check_launch("linear_fp8: status clear");
  // Two-SM tiles (256 x 256 per CTA pair) once there are enough rows to fill them; the single-CTA
  // kernel (128 x 256) below that and when FB_FP8_SINGLE_CTA is set (for comparisons).
  static const bool force_single = getenv("FB_FP8_SINGLE_CTA") != nullptr;
  const bool pair = tokens >= BM2 && !force_single;
  CUtensorMap map_a, map_b;
  if (!make_map_u8(&map_a, a_codes, int64_t(pieces) * tokens, k, 128) || !make_map_u8(&map_b, w_codes, n, k, 128)) {
    set_error("linear_fp8: cuTensorMapEncodeTiled failed");
    return int32_t(cudaErrorInvalidValue);
  }
  GemmArgs ga;
  ga.act_scale = a_scales;
  ga.w_scale = w_scales;
  ga.out = epilogue->out;
  ga.inj = epilogue->inj;
  ga.gate_logit = epilogue->gate_logit;
  ga.status = status;
  ga.scale_bf16 = w_scales_dtype == FB_DT_BF16;
  ga.kind = kind;
  ga.gate_stride = epilogue->gate_stride;
  ga.M = tokens;
  ga.N = n;
  ga.K = k;
  ga.lo_row0 = tokens;
  const int n_tiles = kind == FB_EPI_SWIGLU ? ((n >> 1) + 127) / 128 : (n + BN - 1) / BN;
  if (pair) {
    const int work = ((tokens + BM2 - 1) / BM2) * n_tiles;
    const int pairs = work < pair_count() ? work : pair_count();
    if (pieces == 2)
      fp8_gemm_pair_kernel<2><<<2 * pairs, kThreads, kGemmSmem2, as_stream(stream)>>>(map_a, map_b, ga);
    else
      fp8_gemm_pair_kernel<1><<<2 * pairs, kThreads, kGemmSmem2, as_stream(stream)>>>(map_a, map_b, ga);
    return check_launch("linear_fp8");
  }
  const int m_tiles = (tokens + BM - 1) / BM;
  const int grid = m_tiles * n_tiles < sm_count() ? m_tiles * n_tiles : sm_count();
  if (pieces == 2)
    fp8_gemm_kernel<2><<<grid, kThreads, kGemmSmem, as_stream(stream)>>>(map_a, map_b, ga);
  else
    fp8_gemm_kernel<1><<<grid, kThreads, kGemmSmem, as_stream(stream)>>>(map_a, map_b, ga);
  return check_launch("linear_fp8");
}

size_t fb_linear_fp8_decode_workspace_bytes(int32_t n, int32_t k) {
  if (n <= 0 || k <= 0) return 0;
  // pieces [48][k] | token scales | status | tickets (one per 64 output rows) | partial tiles (two per CTA,
  // sized for 256 multiprocessors so that the figure does not depend on the device)
  return align256(size_t(kDecN) * size_t(k)) + 256 + 256 + align256(size_t((n + 63) / 64) * 4) +
         size_t(2 * 256) * kDecPartialFloats * 4;
}

int32_t fb_linear_fp8_decode(const void* x_bf16, int32_t tokens, const uint8_t* w_codes, const void* w_scales,
                             int32_t w_scales_dtype, int32_t n, int32_t k, const fb_linear_epilogue* epilogue,
                             void* workspace, size_t workspace_bytes, void* stream) {
  if (!x_bf16 || !w_codes || !w_scales || !epilogue || !epilogue->out)
    return invalid("linear_fp8_decode: null argument");
  if (tokens <= 0 || tokens > kDecTok) return invalid("linear_fp8_decode: tokens must be 1..16");
  if (n <= 0 || k <= 0 || k % BK || n % 8) return invalid("linear_fp8_decode: unsupported shape (n %% 8, k %% 128)");
  const int kind = epilogue->kind;
  if (kind < FB_EPI_STORE_BF16 || kind > FB_EPI_SHARED_SCALE) return invalid("linear_fp8_decode: unknown epilogue");
  if (kind == FB_EPI_GR_WRITE && (!epilogue->inj || (reinterpret_cast<uintptr_t>(epilogue->inj) & 15)))
    return invalid("linear_fp8_decode: GrWrite needs inj fp32 [tokens][4], 16-byte aligned");
  if (kind == FB_EPI_SHARED_SCALE && !epilogue->gate_logit)
    return invalid("linear_fp8_decode: SharedScale needs gate_logit");
  if (kind == FB_EPI_SWIGLU && n % 16) return invalid("linear_fp8_decode: SwiGlu needs n %% 16 == 0");
  if ((reinterpret_cast<uintptr_t>(w_codes) | reinterpret_cast<uintptr_t>(x_bf16)) & 15)
    return invalid("linear_fp8_decode: x and weight codes must be 16-byte aligned");
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
      workspace_bytes < fb_linear_fp8_decode_workspace_bytes(n, k))
    return invalid("linear_fp8_decode: workspace missing, misaligned (256 B) or smaller than "
                   "fb_linear_fp8_decode_workspace_bytes");
  if (sm_count() > 256) return invalid("linear_fp8_decode: more than 256 multiprocessors");
  uint8_t* pieces = static_cast<uint8_t*>(workspace);
  float* tok_scale = reinterpret_cast<float*>(pieces + align256(size_t(kDecN) * size_t(k)));
  uint32_t* status = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(tok_scale) + 256);
  int32_t* tickets = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(status) + 256);
  const int n_tickets = (n + 63) / 64;
  float* partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(tickets) + align256(size_t(n_tickets) * 4));
  static PerDeviceOnce once;
  const cudaError_t attr = per_device_once(once, [] { return opt_in_smem(fp8_decode_kernel, kDecSmem); });
  if (attr != cudaSuccess) {
    set_error("linear_fp8_decode: shared-memory opt-in: %s", cudaGetErrorString(attr));
    return int32_t(attr);
  }
  cudaStream_t s = as_stream(stream);
  fp8_split_tokens_kernel<<<kDecTok, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x_bf16), tokens, k, pieces,
                                                   tok_scale, tickets, n_tickets, status);
  int32_t st = check_launch("linear_fp8_decode: split");
  if (st) return st;
  CUtensorMap map_w, map_p;
  if (!make_map_u8(&map_w, w_codes, n, k, 64) || !make_map_u8(&map_p, pieces, kDecN, k, kDecN)) {
    set_error("linear_fp8_decode: cuTensorMapEncodeTiled failed");
    return int32_t(cudaErrorInvalidValue);
  }
  DecArgs a;
  a.tok_scale = tok_scale;
  a.w_scale = w_scales;
  a.scale_bf16 = w_scales_dtype == FB_DT_BF16;
  a.kind = kind;
  a.out = epilogue->out;
  a.inj = epilogue->inj;
  a.gate_logit = epilogue->gate_logit;
  a.gate_stride = epilogue->gate_stride;
  a.T = tokens;
  a.n = n;
  a.k = k;
  a.partial = partial;
  a.tickets = tickets;
  a.status = status;
  const int m_tiles = kind == FB_EPI_SWIGLU ? ((n >> 1) + 63) / 64 : (n + 127) / 128;
  const long long total = (long long)m_tiles * (k / BK);
  // Row tiles that nearly fill the GPU get one CTA each (whole tiles: no partial sums, whose ticketed
  // reduction costs more than the idle multiprocessors). Otherwise the K blocks are divided evenly,
  // with at least two per CTA: below that the partial-sum traffic outweighs the extra parallelism.
  const int sms = sm_count();
  const long long want = total / 2 > 0 ? total / 2 : 1;
  int grid = want < sms ? int(want) : sms;
  if (m_tiles <= sms && 4 * m_tiles >= 3 * sms) grid = m_tiles;
  const cudaError_t e = launch_pdl(fp8_decode_kernel, dim3(grid), dim3(kThreads), size_t(kDecSmem), s, map_w, map_p, a);
  const int32_t launched = check_launch("linear_fp8_decode");
  return launched ? launched : int32_t(e);
}

}  // extern "C"
