// Prefill-width routed experts: route -> grouped gate/up -> grouped down -> combine.
//
// Numerics are the reference's prefill family (src/kernels/moe/moe.h:32-35 and the CPU pool's
// prefill mode, src/cpu/iq_cpu.h:93-99): weights dequantized exactly and rounded to bf16, bf16
// activations, fp32 accumulation, h stored as bf16.
//
// Both grouped GEMMs run on tcgen05 (kind::f16, bf16 x bf16 -> fp32 in tensor memory) with the
// WEIGHT rows on the 128 TMEM lanes and the expert's TOKENS on the N axis (a multiple of 16, up to
// 256), so ragged per-expert token counts waste at most 15 columns:
//   D[128 weight rows][tokens] += W_bf16[128][64] * X[tokens][64]^T        per 64-wide K step.
// The A operand never exists in global memory: dequant warps (16 for gate/up, 8 for down; a warp =
// 16 weight rows, a lane = half of a row's K step = one IQ3_S sub-block or one IQ4_NL block) decode
// straight into the 128-byte-swizzled shared-memory tile the MMA reads. The raw block bytes reach
// them through a coalesced, register-prefetched staging copy in shared memory. The B operand is
// gathered token rows (cp.async, gate/up) or the expert-sorted h rows (TMA, down). One thread
// issues the MMAs; four warps drain tensor memory. All hand-offs are mbarriers with bounded waits.
#include "iq_decode.cuh"

#include <cuda.h>
#include <cuda_bf16.h>

#include <type_traits>
#include <utility>

namespace fb {
namespace {

constexpr int H = FB_HIDDEN;
constexpr int kExperts = FB_EXPERTS;
constexpr int kTopK = FB_TOPK;
constexpr int kBK = 64;          // K elements per pipeline stage = one 128-byte swizzled row
constexpr int kTileM = 128;      // weight rows per unit (TMEM lanes)
constexpr int kTileN = 256;      // tokens per unit (TMEM columns per accumulator)
constexpr int kStagesGU = 3, kStagesDN = 4;
constexpr int kTileA = kTileM * 128;  // 16 KB
constexpr int kTileB = kTileN * 128;  // 32 KB

// ------------------------------------------------------------------------------ PTX (tcgen05 / TMA / cp.async)
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
// D[tmem] (+)= A * B, bf16 operands in shared memory. The operand descriptors are given by their low words (the
// high word is the same for every tile of these kernels, see umma_desc_lo_k128): the issuing lane steps through a
// stage's tiles and K slices with 32-bit adds.
constexpr uint32_t kDescHiK128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ void umma_bf16_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiK128)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
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
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// One arrival on `bar` (already counted in its expected arrivals) once every cp.async this thread has issued so far
// is complete.
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Shared-memory operand descriptor of a K-major bf16 tile, rows of 128 bytes, 128-byte swizzle, 8-row groups 1024
// bytes apart: low word = address / 16 | leading offset 1 << 16, high word (kDescHiK128) = stride 1024 / 16 |
// descriptor version 1 << 14 | swizzle mode 2 << 29.
__device__ __forceinline__ uint32_t umma_desc_lo_k128(uint32_t smem_addr) {
  return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
}
static_assert((uint64_t(kDescHiK128) << 32) == ((uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61)),
              "descriptor high word");
// D fp32, A and B bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t idesc_bf16(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(kTileM >> 4) << 24);
}
// Byte offset of 16-byte chunk c of row r inside a 128-byte-swizzled tile.
__device__ __forceinline__ int swz(int r, int c) { return r * 128 + ((c ^ (r & 7)) << 4); }

struct Abort {
  volatile int* flag;
  uint32_t* status;
  __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity) const {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((i & 31u) == 31u && *flag) return false;  // another role gave up: fall through every later wait
    }
    *flag = 1;
    atomicMax(status, uint32_t(FB_STATUS_PIPELINE_TIMEOUT));
    return false;
  }
};

// ------------------------------------------------------------------------------ weights -> bf16 tile rows
// A dequant thread owns half of a weight row per K step: 32 weights (one IQ3_S sub-block or one
// IQ4_NL block) = four 16-byte chunks of the swizzled tile. Values are bf16_rne(fp32 dequantized
// weight), the reference's rounding (cpu::decode_rows_bf16, src/cpu/iq_cpu.cpp:712-753).
//
// Integer -> float without the conversion pipe: PRMT drops the byte b into the mantissa of 2^23
// (0x4B0000bb = 8388608 + b, exact), and one FMA with the exact constant -db * 2^23 gives
// rn(db * b), bit-identical to fmul_rn(db, float(b)).
__device__ __forceinline__ uint32_t lds16(const uint8_t* p) { return *reinterpret_cast<const unsigned short*>(p); }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// Shared-memory accesses by 32-bit window address with a compile-time offset: one instruction
// each, no 64-bit pointer arithmetic.
template <int OFF>
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF) : "memory");
  return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
  uint32_t v;
  asm volatile("{\n\t.reg .b16 t;\n\tld.shared.u16 t, [%1+%2];\n\tcvt.u32.u16 %0, t;\n\t}" : "=r"(v) : "r"(a), "n"(OFF) : "memory");
  return v;
}
template <int OFF>
__device__ __forceinline__ uint2 lds_v2(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(a), "n"(OFF) : "memory");
  return v;
}
__device__ __forceinline__ void sts_v4(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
template <int OFF>
__device__ __forceinline__ void sts_u32(uint32_t a, uint32_t v) {
  asm volatile("st.shared.u32 [%0+%1], %2;" ::"r"(a), "n"(OFF), "r"(v) : "memory");
}

template <int STRIDE, int PP = 0>
__device__ __forceinline__ void sts_rows(uint32_t a, const uint32_t (&v)[16]) {  // v[pp] -> a + pp * STRIDE
  sts_u32<PP * STRIDE>(a, v[PP]);
  if constexpr (PP + 1 < 16) sts_rows<STRIDE, PP + 1>(a, v);
}

template <int K>
__device__ __forceinline__ float byte_as_magic(uint32_t w) {  // 2^23 + byte K of w
  return __uint_as_float(prmt(w, 0x4B000000u, 0x7440u | uint32_t(K)));
}

// IQ3_S, one sub-block (32 weights) per call. A weight is db * g * sign with g one of the 8 odd
// magnitudes 1..15, so the 8 possible bf16 values of the sub-block are computed once
// (db * (2k+1) is exact in fp32, then rounded like the reference rounds) and kept as two byte
// planes in four registers; the codebook table holds, per 9-bit index, the four 3-bit magnitude
// numbers as PRMT selector nibbles, so one PRMT per plane picks four weights, one XOR flips their
// signs (bit 7 of the high bytes; rounding is sign-symmetric) and two PRMTs interleave the planes
// into bf16 pairs. The integer ALU does ~2.7 operations per weight, none on the conversion pipe.
//
// `slot` = the row's staged block, 8-byte aligned + 4, block byte 0 at slot + 2: that puts qs
// (8 bytes per sub-block), qh and the sign words on their natural alignment.
struct Iq3sColumn {  // per-thread constants of a column (4 K steps of one block)
  float d;
  uint32_t qh_lo, qh_hi;  // qh bytes, shifted so that step q's byte is byte 2*(q&1) of word q>>1
  uint32_t sc;            // scale nibbles, shifted so that step q's nibble is bits 8q..8q+3
};
__device__ __forceinline__ Iq3sColumn iq3s_column(uint32_t slot, int half) {
  Iq3sColumn c;
  c.d = __half2float(__ushort_as_half(static_cast<unsigned short>(lds_u16<2>(slot))));
  const uint2 qh = lds_v2<68>(slot);
  c.qh_lo = qh.x >> (8 * half);
  c.qh_hi = qh.y >> (8 * half);
  c.sc = lds_u32<108>(slot) >> (4 * half);
  return c;
}
// seltab[idx] (16-bit entries) = k0 | k1 << 4 | k2 << 8 | k3 << 12 with grid magnitude j = 2 k_j + 1.
// `slot_h` = slot + 8 * half (window address); `tile_row` = window address of the tile row.
template <int Q>
__device__ __forceinline__ void dequant_sub_iq3s(uint32_t slot_h, uint32_t slot_hh, const Iq3sColumn& col,
                                                 const uint16_t* seltab, uint32_t (&out)[16]) {
  const uint2 qs = lds_v2<4 + 16 * Q>(slot_h);      // slot + 4 + 16 Q + 8 half
  const uint32_t sg = lds_u32<76 + 8 * Q>(slot_hh);  // slot + 76 + 8 Q + 4 half
  const uint32_t B = (((Q >> 1) ? col.qh_hi : col.qh_lo) >> (16 * (Q & 1))) & 0xFFu;  // this sub-block's qh
  const float db = __fmul_rn(col.d, float(int(1u + 2u * ((col.sc >> (8 * Q)) & 0xFu))));
  const float db2 = db + db;
  float pv[8];
  pv[0] = db;
#pragma unroll
  for (int k = 1; k < 8; ++k) pv[k] = pv[k - 1] + db2;  // exact: (2k+1) * db has at most 20 significant bits
  const uint32_t t01 = pack_bf16(pv[0], pv[1]), t23 = pack_bf16(pv[2], pv[3]);
  const uint32_t t45 = pack_bf16(pv[4], pv[5]), t67 = pack_bf16(pv[6], pv[7]);
  const uint32_t lo_a = prmt(t01, t23, 0x6420u), hi_a = prmt(t01, t23, 0x7531u);
  const uint32_t lo_b = prmt(t45, t67, 0x6420u), hi_b = prmt(t45, t67, 0x7531u);
  // Table byte offsets (2 * index) of two look-ups per word: qs byte << 1 in bits 1..8 (17..24), the
  // ninth index bit, taken from qh by a multiply that lands it on bit 9 (25).
  constexpr uint32_t kM = 0x01FE01FEu, kM2 = 0x02000200u;
  uint32_t a[4];
  a[0] = ((qs.x << 1) & kM) | ((B * 0x00800200u) & kM2);  // look-ups 0, 2
  a[1] = ((qs.x >> 7) & kM) | ((B * 0x00400100u) & kM2);  // look-ups 1, 3
  a[2] = ((qs.y << 1) & kM) | ((B * 0x00080020u) & kM2);  // look-ups 4, 6
  a[3] = ((qs.y >> 7) & kM) | ((B * 0x00040010u) & kM2);  // look-ups 5, 7
#pragma unroll
  for (int c = 0; c < 4; ++c) {  // two look-ups = 8 weights = one 16-byte chunk (out[4c .. 4c+3])
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int l = 2 * c + h;
      const uint32_t aw = a[2 * (l >> 2) + (l & 1)];
      const uint32_t off = (l & 2) ? (aw >> 16) : (aw & 0xFFFFu);
      const uint32_t sel = *reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(seltab) + off);
      const uint32_t sx = ((sg >> (4 * l)) & 0xFu) * 0x10204080u;  // sign bit j -> bit 7 of byte j
      const uint32_t lo4 = prmt(lo_a, lo_b, sel);
      const uint32_t hi4 = prmt(hi_a, hi_b, sel) ^ (sx & 0x80808080u);
      out[4 * c + 2 * h] = prmt(lo4, hi4, 0x5140u);
      out[4 * c + 2 * h + 1] = prmt(lo4, hi4, 0x7362u);
    }
  }
}

// IQ4_NL: `blk` = one staged 18-byte block (32 weights; low nibbles are elements 0..15). Levels
// are signed bytes: biased by 128 they go through the same mantissa trick, un-biased by an exact
// subtraction before the multiply.
template <int OFF>
__device__ __forceinline__ void dequant_sub_iq4nl(uint32_t blk, uint32_t (&out)[16]) {
  const Iq4nlLevels lv = iq4nl_levels();
  const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(lds_u16<OFF>(blk))));
  uint32_t qw[4];
  qw[0] = lds_u16<OFF + 2>(blk) | (lds_u16<OFF + 4>(blk) << 16);
  qw[1] = lds_u16<OFF + 6>(blk) | (lds_u16<OFF + 8>(blk) << 16);
  qw[2] = lds_u16<OFF + 10>(blk) | (lds_u16<OFF + 12>(blk) << 16);
  qw[3] = lds_u16<OFF + 14>(blk) | (lds_u16<OFF + 16>(blk) << 16);
  int w[8];  // word e/2 holds levels of elements {e, e+16, e+1, e+17} (e even)
  iq4nl_decode32(lv, qw, w);
#pragma unroll
  for (int hi = 0; hi < 2; ++hi) {    // elements 16*hi .. 16*hi+15
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2) {  // 8 elements per 16-byte chunk (out[4c .. 4c+3], c = 2 hi + c2)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t ww = uint32_t(w[4 * c2 + e]) ^ 0x80808080u;
        const float m0 = hi ? byte_as_magic<1>(ww) : byte_as_magic<0>(ww);
        const float m1 = hi ? byte_as_magic<3>(ww) : byte_as_magic<2>(ww);
        out[4 * (2 * hi + c2) + e] = pack_bf16(__fmul_rn(d, m0 - 8388736.0f), __fmul_rn(d, m1 - 8388736.0f));
      }
    }
  }
}

// How the raw expert bytes reach the dequant threads. Per "column" (kColSteps consecutive K steps)
// a thread needs one contiguous piece of its row. Reading pieces straight from global memory costs
// one cache line per lane, so each warp copies the pieces of its 16 rows with coalesced word loads
// (lane = word of the piece, one piece per instruction) into a padded shared-memory array, one
// column ahead in registers. Row sizes and matrix offsets are multiples of 4, so a piece starts 0
// or 2 bytes into its first word (the same for all rows of a column) and never needs a word that
// starts beyond the end of its matrix. IQ3_S pieces are stored with byte 0 at slot + 2: columns
// whose pieces start on a word boundary are shifted by two bytes on the way (one shuffle and one
// funnel shift per word).
template <int FMT>
struct RawCfg;
template <>
struct RawCfg<FB_FMT_IQ3_S> {
  static constexpr int kColSteps = 4, kPiece = 110, kWords = 28, kStride = 120;
};
template <>
struct RawCfg<FB_FMT_IQ4_NL> {
  static constexpr int kColSteps = 2, kPiece = 72, kWords = 18, kStride = 76;
};
constexpr int kRawBase = 4;       // slots start 8-byte aligned + 4
constexpr int kRawStrideMax = 120;

template <int FMT>
__device__ __forceinline__ void raw_prefetch(const uint8_t* warp_rows, int row_bytes, int col, int lane,
                                             uint32_t (&pre)[16]) {
  using R = RawCfg<FMT>;
  const uint8_t* src = warp_rows + col * R::kPiece;
  const uint8_t* w = src - (reinterpret_cast<uintptr_t>(src) & 3) + 4 * lane;
#pragma unroll
  for (int pp = 0; pp < 16; ++pp)
    pre[pp] = lane < R::kWords ? __ldg(reinterpret_cast<const uint32_t*>(w + size_t(pp) * row_bytes)) : 0u;
}

// One unit's weight rows -> bf16 tiles, K step by K step, by warps of 16 rows x 2 halves.
// `warp_rows` = the first of this warp's 16 rows, `slot0` = their index in the staging array,
// `tile_off` = byte offset of the A tile inside a ring stage, `row` = this thread's tile row and
// `half` its half of the K step. `s`/`ph` = ring stage and phase, carried across units. After a
// failed wait the remaining waits fall through at once (the abort flag is set), so the loop just
// drains. `pre` holds the warp's raw words of this unit's first column on entry (raw_prefetch) and
// those of `next_rows`' first column on return (next_rows = the warp's rows in its next unit, or
// nullptr): the load is issued behind the last column's staging, so that a unit does not start with
// a round trip to memory.
template <int FMT, int STAGES>
__device__ __forceinline__ void dequant_unit(const uint8_t* warp_rows, const uint8_t* next_rows, uint32_t (&pre)[16],
                                             int row_bytes, int k_steps, uint8_t* raw,
                                             int slot0, uint8_t* ring, int stage_bytes, int tile_off, int row,
                                             int half, uint64_t* full, uint64_t* empty, int& s, uint32_t& ph,
                                             const Abort& ab, const uint16_t* seltab) {
  using R = RawCfg<FMT>;
  const int lane = threadIdx.x & 31;
  const int n_cols = k_steps / R::kColSteps;
  int coff[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) coff[c] = ((4 * half + c) ^ (row & 7)) << 4;
  const uint32_t tile_row0 = smem_u32(ring) + tile_off + row * 128;
  const uint32_t wslots = smem_u32(raw) + kRawBase + slot0 * R::kStride + 4 * lane;  // this lane's word of row 0
  const uint32_t slot = smem_u32(raw) + kRawBase + (slot0 + (lane >> 1)) * R::kStride;
  const uint32_t slot_h = slot + (FMT == FB_FMT_IQ3_S ? 8 : 18) * half, slot_hh = slot + 4 * half;
  const int shift0 = int(reinterpret_cast<uintptr_t>(warp_rows) & 3);
  int pending = -1;  // stage whose tile rows are stored but not yet fenced and announced
  auto publish_pending = [&]() {
    if (pending >= 0) {
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[pending]);
      pending = -1;
    }
  };
  for (int col = 0; col < n_cols; ++col) {
    const int shift = (shift0 + col * R::kPiece) & 3;
    if (FMT == FB_FMT_IQ3_S && shift == 0) {
#pragma unroll
      for (int pp = 0; pp < 16; ++pp) pre[pp] = __funnelshift_r(__shfl_up_sync(0xFFFFFFFFu, pre[pp], 1), pre[pp], 16);
    }
    if (lane < R::kWords) {
      sts_rows<R::kStride>(wslots, pre);
    }
    __syncwarp();  // a warp stages and consumes only its own 16 rows
    if (col + 1 < n_cols) raw_prefetch<FMT>(warp_rows, row_bytes, col + 1, lane, pre);
    else if (next_rows) raw_prefetch<FMT>(next_rows, row_bytes, 0, lane, pre);
    Iq3sColumn cc{};
    if constexpr (FMT == FB_FMT_IQ3_S) cc = iq3s_column(slot, half);
    // One K step. Reading a barrier costs a few hundred cycles even when its phase is long complete, and so do
    // the tile stores followed by the proxy fence; neither may sit on the decode's path, the longest chain of the
    // kernel. So the stage's `empty` barrier is probed without blocking BEFORE the step is decoded (the answer is
    // looked at after the decode; only a stage that was really still in use falls into the bounded wait), and a
    // step's fence + arrival are issued after the NEXT step's decode, when its stores have long landed.
    // (Decoding two steps per round of probe, fence and arrivals was measured and is slower: with three or four
    // stages the later publication of the first step costs more than the saved synchronization.)
    auto step = [&](auto qc) {
      constexpr int Q = decltype(qc)::value;
      const uint32_t free_now = mbar_test_wait(&empty[s], ph ^ 1);
      uint32_t out[16];
      if constexpr (FMT == FB_FMT_IQ3_S) dequant_sub_iq3s<Q>(slot_h, slot_hh, cc, seltab, out);
      else dequant_sub_iq4nl<36 * Q>(slot_h, out);
      publish_pending();
      if (!free_now) ab.wait(&empty[s], ph ^ 1);
      const uint32_t tile_row = tile_row0 + s * stage_bytes;
#pragma unroll
      for (int c = 0; c < 4; ++c) sts_v4(tile_row + coff[c], out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]);
      pending = s;
      if (++s == STAGES) { s = 0; ph ^= 1; }
    };
    step(std::integral_constant<int, 0>{});
    step(std::integral_constant<int, 1>{});
    if constexpr (R::kColSteps == 4) {
      step(std::integral_constant<int, 2>{});
      step(std::integral_constant<int, 3>{});
    }
    __syncwarp();  // the warp is done with this column's pieces
  }
  publish_pending();  // a unit's last step does not wait for the next unit's first decode
}

// Fills the 512-entry selector table of dequant_sub_iq3s from the packed codebook (3 bits per
// magnitude number).
__device__ __forceinline__ void iq3s_selector_table_fill(uint16_t* seltab, int tid, int n_threads) {
  for (int i = tid; i < 512; i += n_threads) {
    const uint32_t p = c_iq3s_grid_packed[i];
    seltab[i] = uint16_t((p & 7u) | (((p >> 3) & 7u) << 4) | (((p >> 6) & 7u) << 8) | (((p >> 9) & 7u) << 12));
  }
}

// ------------------------------------------------------------------------------ route
// Top-10 per token (one warp each), per-expert pair counts.
__global__ void __launch_bounds__(256) pf_topk_kernel(const float* __restrict__ logits, int stride, int T,
                                                      int32_t* __restrict__ topk_e, float* __restrict__ topk_w,
                                                      int32_t* __restrict__ count) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  int ids[kTopK];
  float w[kTopK];
  warp_topk10([&](int e) { return logits[size_t(t) * stride + e]; }, ids, w);
  if (lane < kTopK) {
    int id = 0;
    float wt = 0.0f;
#pragma unroll
    for (int k = 0; k < kTopK; ++k)
      if (lane == k) {
        id = ids[k];
        wt = w[k];
      }
    topk_e[t * kTopK + lane] = id;
    topk_w[t * kTopK + lane] = wt;
    if (count) atomicAdd(&count[id], 1);
  }
}

// Expert-parallel routing: the (expert, weight) lists arrive with the dispatched rows; entries of
// experts other ranks own ([lo, hi) is this rank's range) become -1 and take no part. With a share
// table (placement with copies) the rule is per expert instead: share[e] < 0 = not held here, else
// (n << 8) | i = this rank holds copy i of n and takes the rows r with r % n == i.
__global__ void __launch_bounds__(256) pf_import_kernel(const int32_t* __restrict__ in_e, const float* __restrict__ in_w,
                                                        int lo, int hi, const int32_t* __restrict__ share, int n,
                                                        int32_t* __restrict__ topk_e, float* __restrict__ topk_w,
                                                        int32_t* __restrict__ count) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const int e = in_e[i];
  bool local = e >= lo && e < hi;
  if (share) {
    const int sh = e >= 0 && e < kExperts ? share[e] : -1;
    local = sh >= 0 && (i / kTopK) % max(sh >> 8, 1) == (sh & 255);
  }
  topk_e[i] = local ? e : -1;
  topk_w[i] = in_w[i];
  if (local) atomicAdd(&count[e], 1);
}

// Exclusive scan of the counts and the unit lists of both grouped GEMMs (one block of 512).
// unit = {expert, first row of the 128-row weight tile, first pair, tokens in this unit}.
__global__ void __launch_bounds__(512) pf_scan_kernel(const int32_t* __restrict__ count, int32_t* __restrict__ offset,
                                                      int32_t* __restrict__ cursor, int4* __restrict__ units_gu,
                                                      int4* __restrict__ units_dn, int32_t* __restrict__ meta,
                                                      int inter, int max_units_gu, int max_units_dn) {
  __shared__ int s_scan[16];
  __shared__ int s_tiles[16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = count[tid];
  const int tiles = (c + kTileN - 1) / kTileN;
  int ic = c, it = tiles;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, ic, o), b = __shfl_up_sync(0xffffffffu, it, o);
    if (lane >= o) {
      ic += a;
      it += b;
    }
  }
  if (lane == 31) {
    s_scan[warp] = ic;
    s_tiles[warp] = it;
  }
  __syncthreads();
  int bc = 0, bt = 0, tot_c = 0, tot_t = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (i < warp) {
      bc += s_scan[i];
      bt += s_tiles[i];
    }
    tot_c += s_scan[i];
    tot_t += s_tiles[i];
  }
  const int off = bc + ic - c, tile0 = bt + it - tiles;
  offset[tid] = off;
  cursor[tid] = 0;
  if (tid == 0) {
    offset[kExperts] = tot_c;
    meta[0] = min(tot_t * (inter / kTileM), max_units_gu);
    meta[1] = min(tot_t * (H / kTileM), max_units_dn);
    meta[2] = tot_c;
  }
  const int mg = inter / kTileM, md = H / kTileM;
  for (int t = 0; t < tiles; ++t) {
    const int p0 = off + t * kTileN, nt = min(kTileN, c - t * kTileN);
    for (int m = 0; m < mg; ++m) {
      const int u = (tile0 + t) * mg + m;
      if (u < max_units_gu) units_gu[u] = make_int4(tid, m * kTileM, p0, nt);
    }
    for (int m = 0; m < md; ++m) {
      const int u = (tile0 + t) * md + m;
      if (u < max_units_dn) units_dn[u] = make_int4(tid, m * kTileM, p0, nt);
    }
  }
}

// Pairs grouped by expert. The order inside an expert depends on the atomics, the results do not:
// every pair's h and y rows depend only on (token, expert) and the combine adds a token's ten rows
// in ascending-expert order.
__global__ void __launch_bounds__(256) pf_scatter_kernel(const int32_t* __restrict__ topk_e,
                                                         const float* __restrict__ topk_w,
                                                         const int32_t* __restrict__ offset, int32_t* __restrict__ cursor,
                                                         int32_t* __restrict__ pair_token, float* __restrict__ pair_weight,
                                                         int32_t* __restrict__ token_pair, int T) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= T * kTopK) return;
  const int e = topk_e[i];
  if (e < 0) {  // an expert of another rank
    token_pair[i] = -1;
    return;
  }
  const int pos = offset[e] + atomicAdd(&cursor[e], 1);
  pair_token[pos] = i / kTopK;
  pair_weight[pos] = topk_w[i];
  token_pair[i] = pos;
}

// Owner-side sum of an expert-parallel step: y[t] = sum over source ranks d, in rank order, of the
// partial row that rank d returned for token t (row_of[t][d] = its row in `recv`, -1 if rank d held
// none of the token's experts).
__global__ void __launch_bounds__(256) ep_scatter_sum_kernel(const float* __restrict__ recv,
                                                             const int32_t* __restrict__ row_of, int n_ranks,
                                                             float* __restrict__ y) {
  const int t = blockIdx.y, n = blockIdx.x * 256 + threadIdx.x;
  float acc = 0.0f;
  for (int d = 0; d < n_ranks; ++d) {
    const int r = row_of[t * n_ranks + d];
    if (r >= 0) acc += recv[size_t(r) * H + n];
  }
  y[size_t(t) * H + n] = acc;
}

// ------------------------------------------------------------------------------ grouped gate/up
struct GuBars {
  uint64_t full[kStagesGU];
  uint64_t empty[kStagesGU];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort;
};
constexpr int kGuStage = 2 * kTileA + kTileB;                       // 64 KB
constexpr int kGuRaw = 256 * kRawStrideMax + 16;  // staged raw pieces of the 256 weight rows
constexpr int kGuSmem = kStagesGU * kGuStage + kGuRaw + sizeof(GuBars) + 1024;
#ifndef GU_EPI
#define GU_EPI 8
#endif
// warp 0 MMA, four gather warps, 16 dequant warps, the epilogue warps (a multiple of four: one or two per
// tensor-memory lane quarter)
constexpr int kGuGatherWarps = 4, kGuEpilogueWarps = GU_EPI;
constexpr int kGuFirstDequant = 1 + kGuGatherWarps, kGuFirstEpilogue = kGuFirstDequant + 16;
constexpr int kGuThreads = (kGuFirstEpilogue + kGuEpilogueWarps) * 32;
constexpr int kGuRowsPerGather = kTileN / (4 * kGuGatherWarps);  // token rows a gather thread copies per K step

template <int FMT>
__global__ void __launch_bounds__(kGuThreads, 1)
grouped_gate_up_kernel(fb_moe_expert_layout L, const uint8_t* const* __restrict__ expert_blob,
                       const __nv_bfloat16* __restrict__ x, const int4* __restrict__ units,
                       const int32_t* __restrict__ meta, const int32_t* __restrict__ pair_token,
                       __nv_bfloat16* __restrict__ h, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* raw = smem + kStagesGU * kGuStage;
  __shared__ uint16_t seltab[512];  // static: its address folds into the look-up instruction
  GuBars* bars = reinterpret_cast<GuBars*>(raw + kGuRaw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int I = L.inter;
  const int n_units = meta[0];
  const int row_bytes = FMT == FB_FMT_IQ3_S ? 1100 : 1440;
  const Abort ab{&bars->abort, status};

  iq3s_selector_table_fill(seltab, tid, kGuThreads);
  if (tid == 0) {
    for (int i = 0; i < kStagesGU; ++i) {
      mbar_init(&bars->full[i], 32 * kGuGatherWarps + 16);  // gather threads (arrival tied to their copies) + dequant warps
      mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], kGuEpilogueWarps);
    }
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&bars->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  constexpr int kSteps = H / kBK;  // 40

  if (warp == 0) {
    // ---------------- MMA issuer. Tensor memory holds two accumulator buffers of 256 columns. A
    // unit of at most 128 tokens takes one buffer (gate in its first 128 columns, up in the
    // second), so its epilogue overlaps the next unit's K loop; a wider unit takes both (gate in
    // columns [0,256), up in [256,512)). The epilogue warps walk the same sequence.
    if (lane == 0) {
      const uint32_t ring_lo = umma_desc_lo_k128(smem_u32(ring));
      uint32_t it = 0, use0 = 0, use1 = 0, nb = 0;
      for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
        const int4 un = units[u];
        const int n = (un.w + 15) & ~15;
        const bool wide = n > 128;
        const uint32_t idesc = idesc_bf16(n);
        bool ok = true;
        if (wide || nb == 0) ok = ab.wait(&bars->tmem_empty[0], (use0 & 1) ^ 1);
        if (ok && (wide || nb == 1)) ok = ab.wait(&bars->tmem_empty[1], (use1 & 1) ^ 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t gcol = tmem_base + (wide ? 0u : nb * 256u), ucol = gcol + (wide ? 256u : 128u);
        for (int kb = 0; kb < kSteps; ++kb, ++it) {
          const int s = it % kStagesGU;
          if (!ab.wait(&bars->full[s], (it / kStagesGU) & 1)) { ok = false; break; }
          fence_proxy_async();  // the token rows were written by cp.async (generic proxy), the MMA reads them through the async proxy
          // low descriptor words of the stage's gate tile; the up tile and the token tile sit kTileA and 2 kTileA
          // bytes on (descriptor addresses count 16 bytes)
          const uint32_t lg = ring_lo + uint32_t(s) * (kGuStage >> 4);
          constexpr uint32_t kUp = kTileA >> 4, kTok = (2 * kTileA) >> 4;
          const uint32_t first = kb ? 1u : 0u;
          umma_bf16_lo(gcol, lg, lg + kTok, idesc, first);
          umma_bf16_lo(ucol, lg + kUp, lg + kTok, idesc, first);
#pragma unroll
          for (int k4 = 1; k4 < 4; ++k4) {  // 16 bf16 = 32 bytes of K per instruction
            umma_bf16_lo(gcol, lg + 2 * k4, lg + kTok + 2 * k4, idesc, 1u);
            umma_bf16_lo(ucol, lg + kUp + 2 * k4, lg + kTok + 2 * k4, idesc, 1u);
          }
          umma_commit(&bars->empty[s]);
        }
        if (!ok) break;
        if (wide || nb == 0) { umma_commit(&bars->tmem_full[0]); ++use0; }
        if (wide || nb == 1) { umma_commit(&bars->tmem_full[1]); ++use1; }
        if (!wide) nb ^= 1u;
      }
    }
  } else if (warp < kGuFirstDequant) {
    // ---------------- token-row gather: 256 rows x 128 bytes per K step, 16-byte cp.async each. Thread tg
    // copies chunk (tg & 7) of rows (tg >> 3) + 16 i; it keeps those token ids in registers for the whole
    // unit. A thread's arrival on the stage's barrier is tied to the completion of its copies, so it goes on to
    // the next stage at once, as many stages ahead as the ring is free. (Measured alternatives: a TMA gather of
    // four rows per instruction is correct and slower, 1.46 ms against 0.91 ms per layer - 64 small copies per
    // K step; rows pre-gathered into pair order by an extra kernel and loaded as one TMA box per K step come to
    // the same time as this and cost 420 MB of workspace.)
    const int tg = tid - 32;
    const int c = tg & 7, nbase = tg >> 3;
    constexpr int kRowStep = 4 * kGuGatherWarps;
    uint32_t it = 0;
    for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
      const int4 un = units[u];
      int tok[kGuRowsPerGather];
#pragma unroll
      for (int i = 0; i < kGuRowsPerGather; ++i) {
        const int n = kRowStep * i + nbase;
        tok[i] = n < un.w ? pair_token[un.z + n] : -1;
      }
      bool ok = true;
      for (int kb = 0; kb < kSteps; ++kb, ++it) {
        const int s = it % kStagesGU;
        if (!ab.wait(&bars->empty[s], ((it / kStagesGU) & 1) ^ 1)) { ok = false; break; }
        uint8_t* tb = ring + s * kGuStage + 2 * kTileA;
#pragma unroll
        for (int i = 0; i < kGuRowsPerGather; ++i) {
          const int n = kRowStep * i + nbase;
          if (tok[i] >= 0) cp_async16(tb + swz(n, c), x + size_t(tok[i]) * H + kb * kBK + c * 8);
        }
        cp_async_arrive_noinc(&bars->full[s]);
      }
      if (!ok) break;
    }
    cp_async_wait_all();
  } else if (warp < kGuFirstEpilogue) {
    // ---------------- dequant: warp = (matrix, 16 rows), lane = (row, half of the K step)
    const int wd = warp - kGuFirstDequant, mat = wd >> 3, row0 = (wd & 7) * 16;
    int s = 0;
    uint32_t ph = 0;
    auto rows_of = [&](int u) -> const uint8_t* {  // the warp's 16 rows in unit u (nullptr behind the last unit)
      if (u >= n_units) return nullptr;
      const int4 un = units[u];
      const uint8_t* blob = expert_blob ? expert_blob[un.x] : L.slots + int64_t(un.x) * L.blob_stride;
      return blob + (mat ? L.up_offset : L.gate_offset) + size_t(un.y + row0) * row_bytes;
    };
    uint32_t pre[16];
    const uint8_t* warp_rows = rows_of(blockIdx.x);
    if (warp_rows) raw_prefetch<FMT>(warp_rows, row_bytes, 0, lane, pre);
    for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
      const uint8_t* next_rows = rows_of(u + gridDim.x);  // (read well before its use behind the unit's last column)
      dequant_unit<FMT, kStagesGU>(warp_rows, next_rows, pre, row_bytes, kSteps, raw, wd * 16, ring, kGuStage,
                                          mat * kTileA, row0 + (lane >> 1), lane & 1, bars->full, bars->empty, s, ph, ab,
                                          seltab);
      warp_rows = next_rows;
    }
  } else {
    // ---------------- epilogue: lane quarter = warp % 4 (two warps per quarter, which take alternate chunks of 16
    // tokens); thread = intermediate row j
    const int q = warp & 3, chunk0 = 16 * ((warp - kGuFirstEpilogue) >> 2);
    uint32_t use0 = 0, use1 = 0, nb = 0;
    for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
      const int4 un = units[u];
      const bool wide = ((un.w + 15) & ~15) > 128;
      bool ok = true;
      if (wide || nb == 0) ok = ab.wait(&bars->tmem_full[0], use0 & 1);
      if (ok && (wide || nb == 1)) ok = ab.wait(&bars->tmem_full[1], use1 & 1);
      if (!ok) break;
      tc_fence_after();
      const uint32_t gcol = tmem_base + (uint32_t(q * 32) << 16) + (wide ? 0u : nb * 256u);
      const uint32_t ucol = gcol + (wide ? 256u : 128u);
      const int j = un.y + q * 32 + lane;
      for (int c0 = chunk0; c0 < un.w; c0 += 4 * kGuEpilogueWarps) {
        uint32_t g[16], up[16];
        tmem_ld16(gcol + uint32_t(c0), g);
        tmem_ld16(ucol + uint32_t(c0), up);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if (c0 + i < un.w) {
            // silu(g) * u; fast exp and divide: their error (a few fp32 ulp) is far below the bf16 step of h
            const float gv = __uint_as_float(g[i]), uv = __uint_as_float(up[i]);
            const float hv = __fdividef(gv, 1.0f + __expf(-gv)) * uv;
            h[size_t(un.z + c0 + i) * I + j] = __float2bfloat16_rn(hv);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (wide || nb == 0) { if (lane == 0) mbar_arrive(&bars->tmem_empty[0]); ++use0; }
      if (wide || nb == 1) { if (lane == 0) mbar_arrive(&bars->tmem_empty[1]); ++use1; }
      if (!wide) nb ^= 1u;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------ grouped down
struct DnBars {
  uint64_t full[kStagesDN];
  uint64_t empty[kStagesDN];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort;
};
constexpr int kDnStage = kTileA + kTileB;  // 48 KB
constexpr int kDnRaw = 128 * kRawStrideMax + 16;
constexpr int kDnSmem = kStagesDN * kDnStage + kDnRaw + sizeof(DnBars) + 1024;
#ifndef PREFILL_FIXED_DEFAULT
#define PREFILL_FIXED_DEFAULT 0
#endif
#ifndef DN_EPI
#define DN_EPI 8
#endif
constexpr int kDnEpilogueWarps = DN_EPI;               // a multiple of four: every lane quarter gets as many
constexpr int kDnThreads = (10 + kDnEpilogueWarps) * 32;  // warp 0 MMA, warp 1 TMA, 2-9 dequant, the rest epilogue

// yp[pair][n] = w_pair * (down_n . h[pair])
template <int FMT>
__global__ void __launch_bounds__(kDnThreads, 1)
grouped_down_kernel(fb_moe_expert_layout L, const uint8_t* const* __restrict__ expert_blob,
                    const __grid_constant__ CUtensorMap map_h, const int4* __restrict__ units,
                    const int32_t* __restrict__ meta, const float* __restrict__ pair_weight, float* __restrict__ yp,
                    const int32_t* __restrict__ pair_token, unsigned long long* __restrict__ y_fixed, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* raw = smem + kStagesDN * kDnStage;
  __shared__ uint16_t seltab[512];  // static: its address folds into the look-up instruction
  DnBars* bars = reinterpret_cast<DnBars*>(raw + kDnRaw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int I = L.inter;
  const int n_units = meta[1];
  const int row_bytes = FMT == FB_FMT_IQ3_S ? I / 256 * 110 : I / 32 * 18;
  const int k_steps = I / kBK;
  const Abort ab{&bars->abort, status};

  iq3s_selector_table_fill(seltab, tid, kDnThreads);
  if (tid == 0) {
    for (int i = 0; i < kStagesDN; ++i) {
      mbar_init(&bars->full[i], 9);  // TMA thread (with its byte count) + 8 dequant warps
      mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], kDnEpilogueWarps);
    }
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&bars->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t ring_lo = umma_desc_lo_k128(smem_u32(ring));
      uint32_t it = 0, ul = 0;
      for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++ul) {
        const int4 un = units[u];
        const uint32_t idesc = idesc_bf16((un.w + 15) & ~15);
        const int acc = ul & 1;
        if (!ab.wait(&bars->tmem_empty[acc], ((ul >> 1) & 1) ^ 1)) break;
        tc_fence_after();
        bool ok = true;
        for (int kb = 0; kb < k_steps; ++kb, ++it) {
          const int s = it % kStagesDN;
          if (!ab.wait(&bars->full[s], (it / kStagesDN) & 1)) { ok = false; break; }
          const uint32_t la = ring_lo + uint32_t(s) * (kDnStage >> 4);  // low descriptor word of the stage's weight tile
          constexpr uint32_t kTok = kTileA >> 4;
          const uint32_t dcol = tmem_base + uint32_t(acc * 256);
          umma_bf16_lo(dcol, la, la + kTok, idesc, kb ? 1u : 0u);
#pragma unroll
          for (int k4 = 1; k4 < 4; ++k4) umma_bf16_lo(dcol, la + 2 * k4, la + kTok + 2 * k4, idesc, 1u);
          umma_commit(&bars->empty[s]);
        }
        if (!ok) break;
        umma_commit(&bars->tmem_full[acc]);
      }
    }
  } else if (warp == 1) {
    // ---------------- h rows of the unit's pairs: expert-sorted, so one TMA box per K step
    if (lane == 0) {
      uint32_t it = 0;
      int4 un_next = blockIdx.x < n_units ? units[blockIdx.x] : make_int4(0, 0, 0, 0);
      for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
        const int4 un = un_next;
        if (u + gridDim.x < n_units) un_next = units[u + gridDim.x];  // one unit ahead: off the copy path
        bool ok = true;
        for (int kb = 0; kb < k_steps; ++kb, ++it) {
          const int s = it % kStagesDN;
          if (!ab.wait(&bars->empty[s], ((it / kStagesDN) & 1) ^ 1)) { ok = false; break; }
          mbar_expect_tx(&bars->full[s], kTileB);
          tma_load_2d(ring + s * kDnStage + kTileA, &map_h, kb * kBK, un.z, &bars->full[s]);
        }
        if (!ok) break;
      }
    }
  } else if (warp <= 9) {
    // ---------------- dequant: warp = 16 rows, lane = (row, half of the K step)
    const int wd = warp - 2, row0 = wd * 16;
    int s = 0;
    uint32_t ph = 0;
    auto rows_of = [&](int u) -> const uint8_t* {  // the warp's 16 rows in unit u (nullptr behind the last unit)
      if (u >= n_units) return nullptr;
      const int4 un = units[u];
      const uint8_t* blob = expert_blob ? expert_blob[un.x] : L.slots + int64_t(un.x) * L.blob_stride;
      return blob + L.down_offset + size_t(un.y + row0) * row_bytes;
    };
    uint32_t pre[16];
    const uint8_t* warp_rows = rows_of(blockIdx.x);
    if (warp_rows) raw_prefetch<FMT>(warp_rows, row_bytes, 0, lane, pre);
    for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
      const uint8_t* next_rows = rows_of(u + gridDim.x);  // (read well before its use behind the unit's last column)
      dequant_unit<FMT, kStagesDN>(warp_rows, next_rows, pre, row_bytes, k_steps, raw, row0, ring, kDnStage, 0,
                                                 row0 + (lane >> 1), lane & 1, bars->full, bars->empty, s, ph, ab, seltab);
      warp_rows = next_rows;
    }
  } else {
    const int q = warp & 3, chunk0 = 32 * ((warp - 10) >> 2);  // the warps of a lane quarter take chunks of 32 tokens in turn
    uint32_t ul = 0;
    for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++ul) {
      const int4 un = units[u];
      const int acc = ul & 1;
      if (!ab.wait(&bars->tmem_full[acc], (ul >> 1) & 1)) break;
      tc_fence_after();
      const int n = un.y + q * 32 + lane;
      for (int c0 = chunk0; c0 < un.w; c0 += 8 * kDnEpilogueWarps) {
        uint32_t r[32];
        tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * 256 + c0), r);
        tmem_ld_wait();
        if (y_fixed) {  // the reference's accumulation (src/kernels/moe/moe.h:186-192): y_fixed[token] += fixed(w * v)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c0 + i < un.w) {
              const float v = pair_weight[un.z + c0 + i] * __uint_as_float(r[i]);
              atomicAdd(y_fixed + size_t(pair_token[un.z + c0 + i]) * H + n,
                        static_cast<unsigned long long>(__float2ll_rn(v * 4294967296.0f)));
            }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c0 + i < un.w) yp[size_t(un.z + c0 + i) * H + n] = pair_weight[un.z + c0 + i] * __uint_as_float(r[i]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------ combine
// y[t][n] = sum over token t's ten pairs, in ascending expert id, of yp[pair][n] (+ shared);
// X[t][s][n] += inj[t][s] * y when X is given.
__global__ void __launch_bounds__(256) pf_combine_kernel(const int32_t* __restrict__ topk_e,
                                                         const int32_t* __restrict__ token_pair,
                                                         const float* __restrict__ yp, const float* __restrict__ y_shared,
                                                         const float* __restrict__ inj, float* __restrict__ X,
                                                         float* __restrict__ y_out, const long long* __restrict__ y_fixed) {
  const int t = blockIdx.y;
  if (y_fixed) {  // fixed-point sums: one rounding, the scale is exact (moe_y_fixed_to_float of the reference)
    const int n = blockIdx.x * 256 + threadIdx.x;
    float y = static_cast<float>(y_fixed[size_t(t) * H + n]) * (1.0f / 4294967296.0f);
    if (y_shared) y += y_shared[size_t(t) * H + n];
    if (y_out) y_out[size_t(t) * H + n] = y;
    if (X) {
#pragma unroll
      for (int s = 0; s < 4; ++s) X[(size_t(t) * 4 + s) * H + n] += inj[t * 4 + s] * y;
    }
    return;
  }
  __shared__ int s_order[kTopK];
  if (threadIdx.x < kTopK) {
    // ascending expert id; entries without a local pair (expert-parallel shards) sort last
    auto key = [&](int k) {
      const int e = topk_e[t * kTopK + k];
      return e < 0 ? kExperts + k : e;
    };
    const int mine = key(threadIdx.x);
    int rank = 0;
    for (int k = 0; k < kTopK; ++k) rank += key(k) < mine ? 1 : 0;
    s_order[rank] = token_pair[t * kTopK + threadIdx.x];
  }
  __syncthreads();
  const int n = blockIdx.x * 256 + threadIdx.x;
  float y = 0.0f;
#pragma unroll
  for (int k = 0; k < kTopK; ++k)
    if (s_order[k] >= 0) y += yp[size_t(s_order[k]) * H + n];
  if (y_shared) y += y_shared[size_t(t) * H + n];
  if (y_out) y_out[size_t(t) * H + n] = y;
  if (X) {
#pragma unroll
    for (int s = 0; s < 4; ++s) X[(size_t(t) * 4 + s) * H + n] += inj[t * 4 + s] * y;
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

size_t up256(size_t v) { return (v + 255) & ~size_t(255); }
int max_units(int capacity, int tiles_per_group) {
  return (capacity * kTopK / kTileN + kExperts) * tiles_per_group;
}

struct PfLayout {
  size_t meta, count, offset, cursor, topk_e, topk_w, pair_token, pair_weight, token_pair, units_gu, units_dn, h, yp,
      status, total;
};
PfLayout pf_layout(int capacity, int inter) {
  PfLayout l;
  size_t o = 0;
  auto take = [&](size_t bytes) {
    const size_t at = o;
    o = up256(o + bytes);
    return at;
  };
  const size_t pairs = size_t(capacity) * kTopK;
  l.meta = take(64);
  l.count = take(kExperts * 4);
  l.offset = take((kExperts + 1) * 4);
  l.cursor = take(kExperts * 4);
  l.topk_e = take(pairs * 4);
  l.topk_w = take(pairs * 4);
  l.pair_token = take(pairs * 4);
  l.pair_weight = take(pairs * 4);
  l.token_pair = take(pairs * 4);
  l.units_gu = take(size_t(max_units(capacity, inter / kTileM)) * 16);
  l.units_dn = take(size_t(max_units(capacity, H / kTileM)) * 16);
  l.h = take((pairs + kTileN) * size_t(inter) * 2);  // + one tile so a TMA box never leaves the buffer
  l.yp = take(pairs * size_t(H) * 4);
  l.status = take(64);
  l.total = o;
  return l;
}

bool pf_layout_ok(const fb_moe_expert_layout* L, const void* table) {
  if (!L || (!L->slots && !table)) return false;
  if ((uintptr_t(L->blob_stride) | uintptr_t(L->gate_offset) | uintptr_t(L->up_offset) | uintptr_t(L->down_offset)) & 1)
    return false;
  if (L->inter != 512 && L->inter != 640) return false;
  if (L->gate_up_format != FB_FMT_IQ3_S && L->gate_up_format != FB_FMT_IQ4_NL) return false;
  if (L->down_format == FB_FMT_IQ3_S) return L->inter % 256 == 0;
  return L->down_format == FB_FMT_IQ4_NL;
}

bool pf_ws_ok(const fb_moe_prefill_workspace* ws, int tokens) {
  return ws && ws->meta && ws->h && ws->yp && ws->units_gate_up && ws->units_down && tokens >= 1 &&
         tokens <= ws->capacity;
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" {

size_t fb_moe_prefill_workspace_bytes(int32_t capacity, int32_t inter) {
  if (capacity < 1 || (inter != 512 && inter != 640)) return 0;
  return pf_layout(capacity, inter).total;
}

int32_t fb_moe_prefill_workspace_make(void* base, int32_t capacity, int32_t inter, fb_moe_prefill_workspace* out) {
  if (!base || !out || (reinterpret_cast<uintptr_t>(base) & 255) || capacity < 1 || (inter != 512 && inter != 640))
    return invalid("prefill_workspace_make: bad arguments (base 256-byte aligned, inter 512 or 640)");
  const PfLayout l = pf_layout(capacity, inter);
  uint8_t* b = static_cast<uint8_t*>(base);
  out->capacity = capacity;
  out->inter = inter;
  out->max_units_gate_up = max_units(capacity, inter / kTileM);
  out->max_units_down = max_units(capacity, H / kTileM);
  out->meta = reinterpret_cast<int32_t*>(b + l.meta);
  out->expert_count = reinterpret_cast<int32_t*>(b + l.count);
  out->expert_offset = reinterpret_cast<int32_t*>(b + l.offset);
  out->expert_cursor = reinterpret_cast<int32_t*>(b + l.cursor);
  out->topk_expert = reinterpret_cast<int32_t*>(b + l.topk_e);
  out->topk_weight = reinterpret_cast<float*>(b + l.topk_w);
  out->pair_token = reinterpret_cast<int32_t*>(b + l.pair_token);
  out->pair_weight = reinterpret_cast<float*>(b + l.pair_weight);
  out->token_pair = reinterpret_cast<int32_t*>(b + l.token_pair);
  out->units_gate_up = b + l.units_gu;
  out->units_down = b + l.units_dn;
  out->h = b + l.h;
  out->yp = reinterpret_cast<float*>(b + l.yp);
  out->status = reinterpret_cast<uint32_t*>(b + l.status);
  return 0;
}

// 1: the down projection adds into fixed-point per-token sums (the reference's scheme: exact, order-free,
// no per-pair buffer to write and re-read); 0: it stores fp32 per-pair rows that the combine adds in ascending
// expert order. Both are deterministic. The sums live in the head of the yp buffer.
static int g_prefill_fixed = PREFILL_FIXED_DEFAULT;
int32_t fb_moe_prefill_set_accumulation(int32_t fixed_point) {
  g_prefill_fixed = fixed_point ? 1 : 0;
  return 0;
}
static cudaError_t clear_fixed(const fb_moe_prefill_workspace* ws, int32_t tokens, cudaStream_t s) {
  return g_prefill_fixed ? cudaMemsetAsync(ws->yp, 0, size_t(tokens) * H * 8, s) : cudaSuccess;
}

int32_t fb_moe_route(const float* router_logits, int32_t logits_stride, const void* x, const uint8_t* const* expert_blob,
                     int32_t layer, const uint32_t* seq, void* control, int32_t tokens,
                     const fb_moe_prefill_workspace* ws, void* stream) {
  (void)x;
  (void)expert_blob;
  (void)layer;
  (void)seq;
  if (control) return invalid("route: no CPU expert tier exists behind these kernels; control must be NULL");
  if (!router_logits || logits_stride < kExperts || !pf_ws_ok(ws, tokens)) return invalid("route: bad arguments");
  cudaStream_t s = as_stream(stream);
  cudaError_t e = cudaMemsetAsync(ws->expert_count, 0, kExperts * 4, s);
  if (e == cudaSuccess) e = clear_fixed(ws, tokens, s);
  if (e != cudaSuccess) return check_launch("route: memset");
  pf_topk_kernel<<<(tokens + 7) / 8, 256, 0, s>>>(router_logits, logits_stride, tokens, ws->topk_expert, ws->topk_weight,
                                                  ws->expert_count);
  pf_scan_kernel<<<1, 512, 0, s>>>(ws->expert_count, ws->expert_offset, ws->expert_cursor,
                                   static_cast<int4*>(ws->units_gate_up), static_cast<int4*>(ws->units_down), ws->meta,
                                   ws->inter, ws->max_units_gate_up, ws->max_units_down);
  pf_scatter_kernel<<<(tokens * kTopK + 255) / 256, 256, 0, s>>>(ws->topk_expert, ws->topk_weight, ws->expert_offset,
                                                                 ws->expert_cursor, ws->pair_token, ws->pair_weight,
                                                                 ws->token_pair, tokens);
  return check_launch("route");
}

int32_t fb_moe_topk(const float* router_logits, int32_t logits_stride, int32_t tokens, int32_t* topk_expert,
                    float* topk_weight, void* stream) {
  if (!router_logits || logits_stride < kExperts || tokens < 1 || !topk_expert || !topk_weight)
    return invalid("topk: bad arguments");
  pf_topk_kernel<<<(tokens + 7) / 8, 256, 0, as_stream(stream)>>>(router_logits, logits_stride, tokens, topk_expert,
                                                                 topk_weight, nullptr);
  return check_launch("topk");
}

static int32_t route_ep_impl(const int32_t* topk_expert, const float* topk_weight, int32_t expert_lo, int32_t expert_hi,
                             const int32_t* share, int32_t rows, const fb_moe_prefill_workspace* ws, void* stream);

int32_t fb_moe_route_ep(const int32_t* topk_expert, const float* topk_weight, int32_t expert_lo, int32_t expert_hi,
                        int32_t rows, const fb_moe_prefill_workspace* ws, void* stream) {
  if (!topk_expert || !topk_weight || expert_lo < 0 || expert_hi > kExperts || expert_lo >= expert_hi ||
      !pf_ws_ok(ws, rows))
    return invalid("route_ep: bad arguments");
  return route_ep_impl(topk_expert, topk_weight, expert_lo, expert_hi, nullptr, rows, ws, stream);
}

int32_t fb_moe_route_placed(const int32_t* topk_expert, const float* topk_weight, const int32_t* share, int32_t rows,
                            const fb_moe_prefill_workspace* ws, void* stream) {
  if (!topk_expert || !topk_weight || !share || !pf_ws_ok(ws, rows)) return invalid("route_placed: bad arguments");
  return route_ep_impl(topk_expert, topk_weight, 0, 0, share, rows, ws, stream);
}

static int32_t route_ep_impl(const int32_t* topk_expert, const float* topk_weight, int32_t expert_lo, int32_t expert_hi,
                             const int32_t* share, int32_t rows, const fb_moe_prefill_workspace* ws, void* stream) {
  cudaStream_t s = as_stream(stream);
  cudaError_t e = cudaMemsetAsync(ws->expert_count, 0, kExperts * 4, s);
  if (e == cudaSuccess) e = clear_fixed(ws, rows, s);
  if (e != cudaSuccess) return check_launch("route_ep: memset");
  const int n = rows * kTopK;
  pf_import_kernel<<<(n + 255) / 256, 256, 0, s>>>(topk_expert, topk_weight, expert_lo, expert_hi, share, n,
                                                   ws->topk_expert, ws->topk_weight, ws->expert_count);
  pf_scan_kernel<<<1, 512, 0, s>>>(ws->expert_count, ws->expert_offset, ws->expert_cursor,
                                   static_cast<int4*>(ws->units_gate_up), static_cast<int4*>(ws->units_down), ws->meta,
                                   ws->inter, ws->max_units_gate_up, ws->max_units_down);
  pf_scatter_kernel<<<(n + 255) / 256, 256, 0, s>>>(ws->topk_expert, ws->topk_weight, ws->expert_offset,
                                                    ws->expert_cursor, ws->pair_token, ws->pair_weight, ws->token_pair,
                                                    rows);
  return check_launch("route_ep");
}

int32_t fb_ep_scatter_sum(const float* recv, const int32_t* row_of, int32_t n_ranks, int32_t tokens, float* y,
                          void* stream) {
  if (!recv || !row_of || n_ranks < 1 || tokens < 1 || !y) return invalid("ep_scatter_sum: bad arguments");
  ep_scatter_sum_kernel<<<dim3(H / 256, tokens), 256, 0, as_stream(stream)>>>(recv, row_of, n_ranks, y);
  return check_launch("ep_scatter_sum");
}

int32_t fb_moe_grouped_gate_up(const fb_moe_expert_layout* layout, const uint8_t* const* expert_blob, const void* x_bf16,
                               int32_t tokens, const fb_moe_prefill_workspace* ws, void* stream) {
  if (!pf_layout_ok(layout, expert_blob) || !x_bf16 || !pf_ws_ok(ws, tokens) || layout->inter != ws->inter ||
      (reinterpret_cast<uintptr_t>(x_bf16) & 15))
    return invalid("grouped_gate_up: bad arguments");
  static PerDeviceOnce once;
  const cudaError_t attr = per_device_once(once, [] {
    cudaError_t a = opt_in_smem(grouped_gate_up_kernel<FB_FMT_IQ3_S>, kGuSmem);
    if (a == cudaSuccess) a = opt_in_smem(grouped_gate_up_kernel<FB_FMT_IQ4_NL>, kGuSmem);
    return a;
  });
  if (attr != cudaSuccess) {
    set_error("grouped_gate_up: shared-memory opt-in: %s", cudaGetErrorString(attr));
    return int32_t(attr);
  }
  const int grid = sm_count();
  if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) != 0) return invalid("grouped_gate_up: x must be 16-byte aligned");
  const auto* xb = static_cast<const __nv_bfloat16*>(x_bf16);
  auto* hb = static_cast<__nv_bfloat16*>(ws->h);
  const auto* un = static_cast<const int4*>(ws->units_gate_up);
  if (layout->gate_up_format == FB_FMT_IQ3_S)
    grouped_gate_up_kernel<FB_FMT_IQ3_S><<<grid, kGuThreads, kGuSmem, as_stream(stream)>>>(
        *layout, expert_blob, xb, un, ws->meta, ws->pair_token, hb, ws->status);
  else
    grouped_gate_up_kernel<FB_FMT_IQ4_NL><<<grid, kGuThreads, kGuSmem, as_stream(stream)>>>(
        *layout, expert_blob, xb, un, ws->meta, ws->pair_token, hb, ws->status);
  return check_launch("grouped_gate_up");
}

int32_t fb_moe_grouped_down(const fb_moe_expert_layout* layout, const uint8_t* const* expert_blob, int32_t tokens,
                            const fb_moe_prefill_workspace* ws, void* stream) {
  if (!pf_layout_ok(layout, expert_blob) || !pf_ws_ok(ws, tokens) || layout->inter != ws->inter)
    return invalid("grouped_down: bad arguments");
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    set_error("grouped_down: cuTensorMapEncodeTiled is not available");
    return int32_t(cudaErrorNotSupported);
  }
  // h as a 2-D bf16 tensor [pairs + one tile][inter]; boxes of 64 x 256, 128-byte swizzle
  CUtensorMap map_h;
  const cuuint64_t dims[2] = {cuuint64_t(ws->inter), cuuint64_t(size_t(ws->capacity) * kTopK + kTileN)};
  const cuuint64_t strides[1] = {cuuint64_t(ws->inter) * 2};
  const cuuint32_t box[2] = {cuuint32_t(kBK), cuuint32_t(kTileN)};
  const cuuint32_t elem[2] = {1, 1};
  if (fn(&map_h, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ws->h, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    set_error("grouped_down: cuTensorMapEncodeTiled failed");
    return int32_t(cudaErrorInvalidValue);
  }
  static PerDeviceOnce once;
  const cudaError_t attr = per_device_once(once, [] {
    cudaError_t a = opt_in_smem(grouped_down_kernel<FB_FMT_IQ3_S>, kDnSmem);
    if (a == cudaSuccess) a = opt_in_smem(grouped_down_kernel<FB_FMT_IQ4_NL>, kDnSmem);
    return a;
  });
  if (attr != cudaSuccess) {
    set_error("grouped_down: shared-memory opt-in: %s", cudaGetErrorString(attr));
    return int32_t(attr);
  }
  const int grid = sm_count();
  const auto* un = static_cast<const int4*>(ws->units_down);
  unsigned long long* yf = g_prefill_fixed ? reinterpret_cast<unsigned long long*>(ws->yp) : nullptr;
  if (layout->down_format == FB_FMT_IQ3_S)
    grouped_down_kernel<FB_FMT_IQ3_S><<<grid, kDnThreads, kDnSmem, as_stream(stream)>>>(
        *layout, expert_blob, map_h, un, ws->meta, ws->pair_weight, ws->yp, ws->pair_token, yf, ws->status);
  else
    grouped_down_kernel<FB_FMT_IQ4_NL><<<grid, kDnThreads, kDnSmem, as_stream(stream)>>>(
        *layout, expert_blob, map_h, un, ws->meta, ws->pair_weight, ws->yp, ws->pair_token, yf, ws->status);
  return check_launch("grouped_down");
}

int32_t fb_moe_prefill_combine(const fb_moe_prefill_workspace* ws, const float* y_shared, void* control, int32_t layer,
                               const uint32_t* seq, const float* inj, float* X, float* y_out, int32_t tokens,
                               long long timeout_cycles, const float* ablate_direction, float ablate_scale,
                               void* stream) {
  (void)layer;
  (void)seq;
  (void)timeout_cycles;
  (void)ablate_scale;
  if (control) return invalid("prefill_combine: no CPU expert tier exists behind these kernels; control must be NULL");
  if (ablate_direction) return invalid("prefill_combine: the rank-1 ablation is not built for the prefill path");
  if (!pf_ws_ok(ws, tokens) || (X && !inj) || (!X && !y_out)) return invalid("prefill_combine: bad arguments");
  pf_combine_kernel<<<dim3(H / 256, tokens), 256, 0, as_stream(stream)>>>(
      ws->topk_expert, ws->token_pair, ws->yp, y_shared, inj, X, y_out,
      g_prefill_fixed ? reinterpret_cast<const long long*>(ws->yp) : nullptr);
  return check_launch("prefill_combine");
}

}  // extern "C"
