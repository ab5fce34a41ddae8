// The streaming expert kernel of the decode path (gate/up and down of IQ3_S and of IQ4_NL experts), included
// by moe_decode.cu inside namespace fb's anonymous namespace. Written for IQ3_S, described for IQ3_S; IQ4_NL
// rides the same skeleton with its own tile sizes and block arithmetic (ExpertsCfg<FB_FMT_IQ4_NL>,
// iq4nl_task_terms).
//
// One persistent kernel streams the gate, up and down matrices of every routed expert of a layer:
// first all gate/up tiles (heaviest experts first), then all down tiles, through one three-stage ring
// of 40 KB slots, so the codebook set-up, the work-list copy and the pipeline fill are paid once per
// layer and HBM keeps streaming across the gate/up -> down boundary. A down tile needs its expert's h
// re-quantized, which the warp that finishes the expert's last gate/up tile does and then flags; the
// producer asks for a down tile's weights first and polls that flag (a bounded number of times) only
// before it asks for the activation rows. The same kernel runs one phase alone behind the separate
// gate/up and down entry points.
//
// Shape of the work. A lane owns a weight row; a warp task is one 110-byte block (256 weights) of 32
// rows (gate/up: 16 gate rows + the 16 matching up rows, ten blocks; down: five groups of 32 rows, two
// blocks), so every tile is ten tasks, five on even blocks and five on odd ones, that the consumer
// warps draw from two shared-memory tickets.
//
// Arithmetic per 4 weights (one codebook look-up). The codebook in shared memory holds G = (g - 1) / 2
// for every magnitude g in {1, 3, ..., 15}; with m = 0xFF in the bytes of negative weights, the bytes of
// x = G ^ m are G or -G-1, so that 2 x + 1 = +-g: the signed weight. Hence
//   sum_i s_i g_i a_i = 2 * sum_lookups dp4a(x, a) + sum_i a_i,
// ONE dp4a per look-up and token; the second term is the sum of the sub-block's 32 activation codes,
// which the activation quantizer stores beside the codes (it is Q8_K's bsums, pairwise added). Exact
// integer arithmetic throughout: the block sums are the same integers the reference's CPU tier forms.
#pragma once

// ------------------------------------------------------------------------------ planar activation rows
// Q8_K rows in the workspace and in the staged tiles: codes [k] | block scales float [k/256], padded to
// 64 bytes | sub-block code sums int16 [k/32].
__host__ __device__ constexpr int q8k_planar_asum_off(int k) { return q8k_asum_off(k); }
__host__ __device__ constexpr int q8k_planar_bytes(int k) { return q8k_asum_off(k) + ((k / 32 * 2 + 15) & ~15); }
static_assert(q8k_planar_bytes(2560) <= FB_XQ_STRIDE && q8k_planar_bytes(512) <= FB_HQ_STRIDE, "row strides");
static_assert(q8k_planar_bytes(2560) % 16 == 0 && q8k_planar_bytes(512) % 16 == 0, "bulk copies");

// ------------------------------------------------------------------------------ codebook for the 2x+1 form
// Entry i of lane l at word i*32 + l (as iq3s_tables_fill), bytes (g - 1) / 2.
__device__ __forceinline__ void iq3s_half_tables_fill(uint32_t* gridrep, uint32_t* signtab) {
  // consecutive threads write consecutive 16-byte pieces (eight per entry): no bank conflicts
  for (int i = threadIdx.x; i < 512 * 8; i += blockDim.x) {
    const uint32_t w = (iq3s_grid_entry(i >> 3) >> 1) & 0x07070707u;
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

// One 32-weight sub-block: P = sum over its 8 look-ups of dp4a(G ^ m, a) for each of TT tokens.
// qs_lo/qs_hi = its 8 index bytes, qh = a word whose bits [sh, sh+8) are the ninth index bits, sg = its
// 32 sign bits (nibble l = look-up l). sign_base = shared-window address of the 16-word mask table
// (256-byte aligned, below 2^24): it rides in the upper bytes of the byte-permute that builds the
// table offset, so the mask load needs no address arithmetic.
template <int TT>
__device__ __forceinline__ void iq3s_sub_dot(uint32_t qs_lo, uint32_t qs_hi, uint32_t qh, int sh, uint32_t sg,
                                             const uint32_t* grid_lane, uint32_t sign_base,
                                             const int8_t* const (&act)[TT], int (&P)[TT]) {
  // bit j of a nibble -> byte j (0 or 1): n * (1 + 2^7 + 2^14 + 2^21) has bit j at position 8j
  const uint32_t h_lo = (((qh >> sh) & 0xFu) * 0x00204081u) & 0x01010101u;
  const uint32_t h_hi = (((qh >> (sh + 4)) & 0xFu) * 0x00204081u) & 0x01010101u;
  // sign nibbles pre-scaled by 4 (byte offsets into the mask table)
  const uint32_t s_even = (sg << 2) & 0x3C3C3C3Cu;  // look-ups 0,2,4,6
  const uint32_t s_odd = (sg >> 2) & 0x3C3C3C3Cu;   // look-ups 1,3,5,7
  uint32_t x[8];
#pragma unroll
  for (int l = 0; l < 8; ++l) {
    const int b = l & 3;
    // byte0 = qs byte b, byte1 = spread bit b, bytes 2-3 = 0 (sign-replicate of a 0/1 byte)
    const uint32_t sel = uint32_t(b) | (uint32_t(4 + b) << 4) | (uint32_t(0xC + b) << 8) | (uint32_t(0xC + b) << 12);
    const uint32_t idx = prmt(l < 4 ? qs_lo : qs_hi, l < 4 ? h_lo : h_hi, sel);
    const uint32_t g = grid_lane[idx * 32];
    // byte0 = the pre-scaled nibble of look-up l, bytes 1-3 = the table's address bytes
    // (computing the masks instead - isolate the nibble, one wide multiply that sends bit j to the top of
    // byte j, one sign-replicating byte-permute - frees a third of the shared-memory wavefronts but the
    // multiplies queue up in the dispatch stage: measured 96 us against 80 us per layer launch)
    const uint32_t maddr = prmt((l & 1) ? s_odd : s_even, sign_base, 0x7650u | uint32_t(l >> 1));
    uint32_t m;
    asm("ld.shared.u32 %0, [%1];" : "=r"(m) : "r"(maddr));
    x[l] = g ^ m;
  }
#pragma unroll
  for (int t = 0; t < TT; ++t) {
    const int4 a0 = *reinterpret_cast<const int4*>(act[t]);
    const int4 a1 = *reinterpret_cast<const int4*>(act[t] + 16);
    int p = __dp4a(int(x[0]), a0.x, 0);
    p = __dp4a(int(x[1]), a0.y, p);
    p = __dp4a(int(x[2]), a0.z, p);
    p = __dp4a(int(x[3]), a0.w, p);
    p = __dp4a(int(x[4]), a1.x, p);
    p = __dp4a(int(x[5]), a1.y, p);
    p = __dp4a(int(x[6]), a1.z, p);
    p = __dp4a(int(x[7]), a1.w, p);
    P[t] = p;
  }
}

// Integer dot of one IQ3_S block with TT activation blocks:
//   bsum[t] = sum over its 8 sub-blocks of (2 s + 1) * (2 P + A), exact in int32 (|bsum| < 2^24).
// w = the word that holds the block's fp16 scale (MIS: in its low half, the 27 stream words then sit
// 2 bytes off word alignment; else in its high half and the stream is aligned); act[t] = the 256
// codes of the matching Q8_K block, asum[t] = its 8 sub-block code sums (16-byte aligned).
// |P| <= 32 * 8 * 127 fits 16 bits, so two sub-blocks' P (and their two code sums A) are multiplied by
// their odd multipliers with one two-way dot product each.
template <bool MIS, int TT>
__device__ __forceinline__ void iq3s_block_idot2(const uint32_t* w, const uint32_t* grid_lane, uint32_t sign_base,
                                                 const int8_t* const (&act)[TT], const int16_t* const (&asum)[TT],
                                                 int (&bsum)[TT]) {
  const uint32_t sc = iq3s_stream<MIS>(w, 26);
  // multipliers 2 s + 1 as bytes: even sub-blocks (low nibbles) and odd sub-blocks (high nibbles)
  const uint32_t m_even = ((sc << 1) & 0x1E1E1E1Eu) | 0x01010101u;
  const uint32_t m_odd = ((sc >> 3) & 0x1E1E1E1Eu) | 0x01010101u;
  int4 as[TT];
  int accP[TT], accA[TT];
#pragma unroll
  for (int t = 0; t < TT; ++t) {
    accP[t] = 0;
    as[t] = *reinterpret_cast<const int4*>(asum[t]);
  }
  {  // code-sum part: sum_sb (2 s + 1) * A_sb, four two-way dot products
    const uint32_t mi01 = __byte_perm(m_even, m_odd, 0x5140), mi23 = __byte_perm(m_even, m_odd, 0x7362);
#pragma unroll
    for (int t = 0; t < TT; ++t) {
      int a = __dp2a_lo(as[t].x, int(mi01), 0);
      a = __dp2a_hi(as[t].y, int(mi01), a);
      a = __dp2a_lo(as[t].z, int(mi23), a);
      accA[t] = __dp2a_hi(as[t].w, int(mi23), a);
    }
  }
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    const uint32_t qh = iq3s_stream<MIS>(w, 16 + half);
    // bytes {m(4h), m(4h+1), m(4h+2), m(4h+3)} of this half's four sub-blocks
    const uint32_t mi = __byte_perm(m_even, m_odd, half == 0 ? 0x5140u : 0x7362u);
    int P[4][TT];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int ib = 4 * half + i;
      const int8_t* a[TT];
#pragma unroll
      for (int t = 0; t < TT; ++t) a[t] = act[t] + 32 * ib;
      iq3s_sub_dot<TT>(iq3s_stream<MIS>(w, 2 * ib), iq3s_stream<MIS>(w, 2 * ib + 1), qh, 8 * i,
                       iq3s_stream<MIS>(w, 18 + ib), grid_lane, sign_base, a, P[i]);
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
      const int p01 = int(__byte_perm(uint32_t(P[0][t]), uint32_t(P[1][t]), 0x5410));
      const int p23 = int(__byte_perm(uint32_t(P[2][t]), uint32_t(P[3][t]), 0x5410));
      accP[t] = __dp2a_lo(p01, int(mi), accP[t]);
      accP[t] = __dp2a_hi(p23, int(mi), accP[t]);
    }
  }
#pragma unroll
  for (int t = 0; t < TT; ++t) bsum[t] = 2 * accP[t] + accA[t];
}

// scale of the block, fp16 -> fp32
template <bool MIS>
__device__ __forceinline__ float iq3s_block_d(const uint32_t* w) {
  const uint32_t v = MIS ? (w[0] & 0xFFFFu) : (w[0] >> 16);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(v)));
}

// The 64-byte mask table sits on a 256-byte boundary (its address bytes 1-3 ride in a byte-permute)
// inside an area of kSignArea bytes.
constexpr int kSignArea = 320;
__device__ __forceinline__ uint32_t* sign_table_at(uint8_t* area) {
  return reinterpret_cast<uint32_t*>(area + ((256u - (smem_u32(area) & 255u)) & 255u));
}

// ------------------------------------------------------------------------------ multi-stage ring
template <int S>
struct RingN {
  uint64_t* full;   // [S] count 1 + tx bytes
  uint64_t* empty;  // [S]
  volatile StageMeta* meta;  // [S]
  // number of entries the producer staged in all; INT_MAX while it is still staging; 0 after a time-out
  volatile int* end_seq;
};

// try_wait with a suspend-time hint: the thread may sleep inside the instruction until the phase
// completes or about a microsecond has passed, instead of spinning through issue slots the working
// warps need.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(1000u)
      : "memory");
  return ok != 0;
}
// Bounded: 2^21 tries of at most about a microsecond each.
__device__ __forceinline__ bool mbar_wait_hint(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 21); ++i)
    if (mbar_try_wait_hint(bar, parity)) return true;
  return false;
}

template <int S>
__device__ __forceinline__ void ringn_init(const RingN<S>& r) {
  for (int s = 0; s < S; ++s) {
    mbar_init(&r.full[s], 1);
    mbar_init(&r.empty[s], 1);  // one arrival frees a slot: the warp that finishes the entry's last task
    r.meta[s].tile = -1;
    r.meta[s].seq = -1;
  }
  *r.end_seq = 0x7fffffff;
  mbar_fence_init();
}

// Consumer side: draws the next (entry, task) ticket and waits for that entry's data; returns false
// at the end. A warp may hold a ticket for an entry that is S or more entries ahead of the one its slot
// is being filled with, and the barrier's one-bit phase cannot tell those apart. So the warp first waits
// (polling one shared-memory word, asleep in between) until the producer has written this entry's number
// into the slot, which it does before it arms the barrier; only then is the barrier's current phase the
// entry's own, and the warp can sleep inside try_wait. On a time-out the producer sets end_seq to 0, which
// releases every waiting warp.
template <int S, int TASKS>
__device__ __forceinline__ bool draw_task_n(const RingN<S>& r, int* ticket_ctr, uint32_t* status, int lane, int& s,
                                            int& task) {
  int ticket = 0;
  if (lane == 0) ticket = atomicAdd(ticket_ctr, 1);
  ticket = __shfl_sync(0xffffffffu, ticket, 0);
  const int seq = ticket / TASKS;
  task = ticket - seq * TASKS;
  s = seq % S;
  uint32_t tries = 0;
  while (r.meta[s].seq != seq) {
    if (*r.end_seq <= seq) return false;
    if (++tries > (1u << 20)) {  // bounded: about a second
      *r.end_seq = 0;
      atomicMax(status, uint32_t(FB_STATUS_PIPELINE_TIMEOUT));
      return false;
    }
    // (the producer is behind only at the start of a phase; the nap is short because at one to three tokens this
    // wait sits on the layer's critical path)
    __nanosleep(200);
  }
  const uint32_t parity = (seq / S) & 1;
  for (uint32_t i = 0; i < (1u << 21); ++i) {  // bounded: each try takes at most about a microsecond
    if (mbar_try_wait_hint(&r.full[s], parity)) return true;
    if (*r.end_seq <= seq) return false;
  }
  *r.end_seq = 0;
  atomicMax(status, uint32_t(FB_STATUS_PIPELINE_TIMEOUT));
  return false;
}

// ------------------------------------------------------------------------------ the expert kernel
// Gate/up tile = 16 intermediate rows: 16 gate rows and the 16 matching up rows (17,600 bytes each);
// task b (0..9) = block b of all 32 rows, lanes 0-15 the gate rows, lanes 16-31 the up rows; the warp
// that finishes the tile's last task adds each row's ten block terms in block order, pairs gate with
// up through a shuffle and applies SwiGLU.
// Down tile = 160 output rows (35,200 bytes; a row is two blocks); task 2k + b = block b of rows
// 32k .. 32k+31; the finishing warp adds each row's two block terms and applies the routing weight.
// Both kinds carry the activation rows of the pass behind the weights.
template <int FMT>
struct ExpertsCfg;
template <>
struct ExpertsCfg<FB_FMT_IQ3_S> {
  static constexpr int kWarps = 24, kTasks = 10, kStages = 3, kInter = 512;
  static constexpr int kTaskBytes = 110;  // one block of 256 weights
  static constexpr int kGuRows = 16, kGuRowBytes = 1100, kGuPart = kGuRows * kGuRowBytes;  // 17,600
  static constexpr int kDnRows = 160, kDnRowBytes = 220, kDnTile = kDnRows * kDnRowBytes;  // 35,200
  static constexpr int kAct = FB_ACT_Q8_K;
  static constexpr int kGuAct = q8k_planar_bytes(H), kDnAct = q8k_planar_bytes(kInter);    // 2,784 / 608
  static constexpr int kSlot = 2 * kGuPart + kTT * kGuAct;                                 // 40,768
  static constexpr int kDnTilesPerItem = H / kDnRows;                                      // 16
  static constexpr int kPartialFloats = kStages * kTasks * kTT * 32;
  static constexpr int kTableBytes = kGridRepBytes + kSignArea;  // codebook replica and sign masks
  static constexpr size_t kSmem = size_t(kTableBytes) + size_t(kStages) * kSlot + kPartialFloats * 4 + 128;
};
// IQ4_NL: the same tile and task shapes with a "block" of eight consecutive 18-byte blocks (256 weights, 144
// bytes, 16-byte aligned in every row): gate/up tile = 16 + 16 rows of 1440 bytes, down tile = 160 rows of 288.
// No table: the sixteen levels live in registers.
template <>
struct ExpertsCfg<FB_FMT_IQ4_NL> {
  static constexpr int kWarps = 24, kTasks = 10, kStages = 3, kInter = 512;
  static constexpr int kTaskBytes = 144;
  static constexpr int kGuRows = 16, kGuRowBytes = 1440, kGuPart = kGuRows * kGuRowBytes;  // 23,040
  static constexpr int kDnRows = 160, kDnRowBytes = 288, kDnTile = kDnRows * kDnRowBytes;  // 46,080
  static constexpr int kAct = FB_ACT_Q8_0;
  static constexpr int kGuAct = H + H / 8, kDnAct = kInter + kInter / 8;                    // 2,880 / 576
  static constexpr int kSlot = 2 * kGuPart + kTT * kGuAct;                                 // 51,840
  static constexpr int kDnTilesPerItem = H / kDnRows;
  static constexpr int kPartialFloats = kStages * kTasks * kTT * 32;
  static constexpr int kTableBytes = 0;
  static constexpr size_t kSmem = size_t(kStages) * kSlot + kPartialFloats * 4 + 128;
};
using Experts3 = ExpertsCfg<FB_FMT_IQ3_S>;
template <int FMT>
constexpr bool experts_cfg_ok() {
  using C = ExpertsCfg<FMT>;
  return C::kDnTile + kTT * C::kDnAct <= C::kSlot && C::kSlot % 16 == 0 && C::kGuPart % 16 == 0 && C::kDnTile % 16 == 0 &&
         C::kGuAct % 16 == 0 && C::kDnAct % 16 == 0 && H % C::kDnRows == 0 && C::kDnRows % 32 == 0 &&
         C::kGuRowBytes == C::kTasks * C::kTaskBytes && C::kDnRowBytes == 2 * C::kTaskBytes && C::kTaskBytes % 2 == 0;
}
static_assert(experts_cfg_ok<FB_FMT_IQ3_S>() && experts_cfg_ok<FB_FMT_IQ4_NL>(), "tile shapes, bulk-copy sizes");
// kPhaseSelect: the CTA builds the work list itself from the router logits (SelectArgs) instead of
// reading the device work list a selection kernel left.
enum { kPhaseGateUp = 1, kPhaseDown = 2, kPhaseSelect = 4 };

// One block (256 weights) of the lane's row against the pass's tokens: term[t] = bsum * d * d_act.
template <bool MIS>
__device__ __forceinline__ void expert_block_terms(const uint32_t* w, const uint32_t* grid_lane, uint32_t sign_base,
                                                   const uint8_t* act0, int act_bytes, int k, int blk, int ntp,
                                                   float (&term)[kTT]) {
  const float d = iq3s_block_d<MIS>(w);
  if (ntp == 1) {
    const int8_t* a[1] = {reinterpret_cast<const int8_t*>(act0) + 256 * blk};
    const int16_t* as[1] = {reinterpret_cast<const int16_t*>(act0 + q8k_planar_asum_off(k)) + 8 * blk};
    int bs[1];
    iq3s_block_idot2<MIS, 1>(w, grid_lane, sign_base, a, as, bs);
    term[0] = float(bs[0]) * (d * reinterpret_cast<const float*>(act0 + k)[blk]);
    term[1] = 0.0f;
  } else {
    const uint8_t* act1 = act0 + act_bytes;
    const int8_t* a[2] = {reinterpret_cast<const int8_t*>(act0) + 256 * blk,
                          reinterpret_cast<const int8_t*>(act1) + 256 * blk};
    const int16_t* as[2] = {reinterpret_cast<const int16_t*>(act0 + q8k_planar_asum_off(k)) + 8 * blk,
                            reinterpret_cast<const int16_t*>(act1 + q8k_planar_asum_off(k)) + 8 * blk};
    int bs[2];
    iq3s_block_idot2<MIS, 2>(w, grid_lane, sign_base, a, as, bs);
    term[0] = float(bs[0]) * (d * reinterpret_cast<const float*>(act0 + k)[blk]);
    term[1] = float(bs[1]) * (d * reinterpret_cast<const float*>(act1 + k)[blk]);
  }
}

// IQ4_NL: one task = eight consecutive blocks (144 bytes at `wp`, 16-byte aligned) of the lane's row against
// the pass's tokens; blk0 = index of the first of them in the row. Even blocks start on a word (scale in the
// low half, codes two bytes off: funnel shifts), odd blocks on a half word (scale in the high half, codes
// aligned). term[t] = sum over the eight blocks, in block order, of isum * (d * d_act).
__device__ __forceinline__ void iq4nl_task_terms(const uint8_t* wp, const Iq4nlLevels& lv, const uint8_t* act0,
                                                 int act_bytes, int k, int blk0, int ntp, float (&term)[kTT]) {
  uint32_t w[36];
#pragma unroll
  for (int c = 0; c < 9; ++c) {
    const uint4 v = reinterpret_cast<const uint4*>(wp)[c];
    w[4 * c] = v.x;
    w[4 * c + 1] = v.y;
    w[4 * c + 2] = v.z;
    w[4 * c + 3] = v.w;
  }
  term[0] = term[1] = 0.0f;
  const uint8_t* act1 = act0 + (ntp == 2 ? act_bytes : 0);
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    uint32_t q[4];
    float d;
    if (b % 2 == 0) {
      const int base = 9 * b / 2;
      d = __half2float(__ushort_as_half(static_cast<unsigned short>(w[base] & 0xFFFFu)));
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = __funnelshift_r(w[base + i], w[base + i + 1], 16);
    } else {
      const int base = (18 * b - 2) / 4;
      d = __half2float(__ushort_as_half(static_cast<unsigned short>(w[base] >> 16)));
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = w[base + 1 + i];
    }
    int wq[8];
    iq4nl_decode32(lv, q, wq);
    const int blk = blk0 + b;
    const int s0 = dot32(wq, reinterpret_cast<const int8_t*>(act0) + 32 * blk);
    term[0] = fmaf(float(s0), d * reinterpret_cast<const float*>(act0 + k)[blk], term[0]);
    if (ntp == 2) {
      const int s1 = dot32(wq, reinterpret_cast<const int8_t*>(act1) + 32 * blk);
      term[1] = fmaf(float(s1), d * reinterpret_cast<const float*>(act1 + k)[blk], term[1]);
    }
  }
}

template <int FMT>
__global__ void __launch_bounds__((ExpertsCfg<FMT>::kWarps + 1) * 32, 1)
experts_kernel(fb_moe_expert_layout L, fb_moe_decode_workspace ws, int phases, SelectArgs sel) {
  using C = ExpertsCfg<FMT>;
  constexpr int S = C::kStages;
  constexpr bool kIq3s = FMT == FB_FMT_IQ3_S;
  extern __shared__ __align__(128) uint8_t smem[];
  uint32_t* gridrep = reinterpret_cast<uint32_t*>(smem);
  uint32_t* signtab = kIq3s ? sign_table_at(smem + kGridRepBytes) : nullptr;
  uint8_t* stage0 = smem + C::kTableBytes;
  float* partials = reinterpret_cast<float*>(stage0 + S * C::kSlot);
  uint64_t* bars = reinterpret_cast<uint64_t*>(partials + C::kPartialFloats);
  __shared__ StageMeta s_meta[S];
  __shared__ int s_misc[3 + S];  // [1..2] task tickets (even / odd blocks), [3..] finished tasks per slot
  __shared__ int s_end;
  __shared__ WorkCache s_work;
  RingN<S> ring{bars, bars + S, s_meta, &s_end};

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if constexpr (kIq3s) iq3s_half_tables_fill(gridrep, signtab);
  if (tid == 0) {
    ringn_init(ring);
    for (int i = 1; i < 3 + S; ++i) s_misc[i] = 0;
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait_prior();

  int n_items;
  if (phases & kPhaseSelect) {
    select_block(
        [&](int t, uint2* scratch, int* ids, float* wts) {
          warp_topk10_pruned([&](int e) { return __ldcg(sel.logits + size_t(t) * sel.stride + e); }, scratch, ids, wts);
        },
        sel.slot_of, sel.tokens, ws, nullptr, sel.remote_ok != 0, blockIdx.x == 0, false, s_work);
    n_items = s_work.n_items;
  } else {
    n_items = min(max(ws.work->n_items, 0), kMaxPairs);
  }
  const int I = L.inter;  // gate/up takes 512 or 640; the down phase is for 512 (checked on the host)
  const uint8_t* xq_rows = ws.xq + xq_offset(C::kAct);
  const int gu_tpi = I / C::kGuRows;
  const int n_gu = (phases & kPhaseGateUp) ? n_items * gu_tpi : 0;
  const int n_dn = (phases & kPhaseDown) ? n_items * C::kDnTilesPerItem : 0;

  if (warp == C::kWarps) {
    // ---------------- producer: one lane draws tiles (two steps ahead of their use) and issues their
    // bulk copies into the ring; every pass of kTT tokens of a tile is one ring entry.
    if (!(phases & kPhaseSelect)) {
      work_cache_fill(ws, s_work, n_items);
      __syncwarp();
    }
    if (lane != 0) return;
    int* counter = ws.sched + ((phases & kPhaseGateUp) ? kSchedGateUp : kSchedDown);
    const int n_tiles = n_gu + n_dn;
    int i = 0;
    bool failed = false;
    struct EndMark {  // whichever way the loop is left, waiting consumers learn how many entries exist
      const RingN<S>& r;
      const int& i;
      const bool& failed;
      __device__ ~EndMark() { *r.end_seq = failed ? 0 : i; }
    } end_mark{ring, i, failed};
    auto give_up = [&]() {
      failed = true;
      atomicMax(ws.status, uint32_t(FB_STATUS_PIPELINE_TIMEOUT));
    };
    auto slot_free = [&](int s) -> bool {
      if (*ring.end_seq == 0) return false;  // a consumer gave up
      if (i >= S && !mbar_wait_hint(&ring.empty[s], ((i / S) - 1) & 1)) {
        give_up();
        return false;
      }
      return true;
    };
    // a block's first two tiles need no ticket; the counter hands out the tiles behind those
    const int first_ticket = 2 * int(gridDim.x);
    int next = int(blockIdx.x), next2 = int(blockIdx.x + gridDim.x);
    while (true) {
      const int tile = next;
      if (tile >= n_tiles) break;
      next = next2;
      next2 = first_ticket + atomicAdd(counter, 1);
      const bool down = tile >= n_gu;
      const int tl = down ? tile - n_gu : tile;
      const int pos = down ? tl / C::kDnTilesPerItem : I == 512 ? tl >> 5 : tl / (640 / C::kGuRows);  // (no run-time division)
      const int sub = down ? tl - pos * C::kDnTilesPerItem : tl - pos * gu_tpi;
      const int item = s_work.order[pos];
      const int pb = s_work.pair_begin[item];
      const int ntok = s_work.pair_begin[item + 1] - pb;
      const uint8_t* blob = L.slots + int64_t(s_work.slot[item]) * L.blob_stride;
      bool ready = !down || !(phases & kPhaseGateUp);  // a down-only launch runs behind a finished gate/up launch
      for (int tok0 = 0; tok0 < ntok; tok0 += kTT, ++i) {
        const int s = i % S;
        if (!slot_free(s)) return;
        const int ntp = min(kTT, ntok - tok0);
        volatile StageMeta* m = &ring.meta[s];
        m->seq = i;
        m->tile = down ? 1 : 0;  // entry kind
        m->pair0 = pb + tok0;
        m->ntp = ntp;
        m->row0 = sub * (down ? C::kDnRows : C::kGuRows);
        m->item = item;
        m->item_pair0 = pb;
        m->item_tok = ntok;
        for (int t = 0; t < kTT; ++t) m->wgt[t] = tok0 + t < ntok ? s_work.pair_weight[pb + tok0 + t] : 0.0f;
        uint8_t* st = stage0 + s * C::kSlot;
        if (!down) {
          mbar_expect_tx(&ring.full[s], uint32_t(2 * C::kGuPart + ntp * C::kGuAct));
          const size_t off = size_t(sub) * C::kGuPart;
          bulk_g2s(st, blob + L.gate_offset + off, C::kGuPart, &ring.full[s]);
          bulk_g2s(st + C::kGuPart, blob + L.up_offset + off, C::kGuPart, &ring.full[s]);
          for (int t = 0; t < ntp; ++t)
            bulk_g2s(st + 2 * C::kGuPart + t * C::kGuAct,
                     xq_rows + size_t(s_work.pair_token[pb + tok0 + t]) * FB_XQ_STRIDE, C::kGuAct, &ring.full[s]);
        } else {
          mbar_expect_tx(&ring.full[s], uint32_t(C::kDnTile + ntp * C::kDnAct));
          bulk_g2s(st, blob + L.down_offset + size_t(sub) * C::kDnTile, C::kDnTile, &ring.full[s]);
          if (!ready) {  // the item's h must have been re-quantized (bounded poll of its flag)
            const int* flag = ws.item_done + item;
            uint32_t tries = 0;
            while (true) {
              int v;
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
              if (v & kItemReady) break;
              if (++tries > (1u << 22) || *ring.end_seq == 0) {
                give_up();
                break;
              }
              __nanosleep(200);
            }
            ready = true;
            // the rows were written by another SM's ordinary stores and are read by bulk copies
            asm volatile("fence.proxy.async.global;" ::: "memory");
          }
          for (int t = 0; t < ntp; ++t)
            bulk_g2s(st + C::kDnTile + t * C::kDnAct, ws.hq + size_t(pb + tok0 + t) * FB_HQ_STRIDE, C::kDnAct,
                     &ring.full[s]);
          if (failed) {  // nobody will use the entry: see its copies land (bounded), then leave
            mbar_wait_hint(&ring.full[s], (i / S) & 1);
            return;
          }
        }
      }
    }
    return;
  }

  // ---------------- consumers
  const uint32_t* grid_lane = gridrep + lane;
  const uint32_t sign_base = kIq3s ? smem_u32(signtab) : 0u;
  const Iq4nlLevels lv = iq4nl_levels();
  const int gu_row_off = (lane >> 4) * C::kGuPart + (lane & 15) * C::kGuRowBytes;
  // Even blocks start on a word boundary (their 27-word stream is 2 bytes off), odd blocks the other
  // way round: two code paths. A warp keeps to one parity, and since warp w issues on scheduler w % 4,
  // each scheduler's instruction cache sees one path only.
  const int parity = warp & 1;
  const int down_act = act_of(L.down_format);
  while (true) {
    int s, k;
    if (!draw_task_n<S, C::kTasks / 2>(ring, &s_misc[1 + parity], ws.status, lane, s, k)) break;
    const int task = 2 * k + parity;
    const int ntp = ring.meta[s].ntp;
    const bool down = ring.meta[s].tile != 0;
    uint8_t* st = stage0 + s * C::kSlot;
    // the lane's block, the activation rows, and which of their blocks it meets
    const uint8_t* blk = down ? st + (32 * k + lane) * C::kDnRowBytes + parity * C::kTaskBytes
                              : st + gu_row_off + task * C::kTaskBytes;
    const uint8_t* act0 = st + (down ? C::kDnTile : 2 * C::kGuPart);
    const int act_bytes = down ? C::kDnAct : C::kGuAct, act_k = down ? C::kInter : H, ablk = down ? parity : task;
    float term[kTT];
    if constexpr (!kIq3s)
      iq4nl_task_terms(blk, lv, act0, act_bytes, act_k, 8 * ablk, ntp, term);
    else if (parity == 0)
      expert_block_terms<true>(reinterpret_cast<const uint32_t*>(blk), grid_lane, sign_base, act0, act_bytes, act_k, ablk,
                               ntp, term);
    else
      expert_block_terms<false>(reinterpret_cast<const uint32_t*>(blk - 2), grid_lane, sign_base, act0, act_bytes, act_k,
                                ablk, ntp, term);
    float* part = partials + (s * C::kTasks + task) * (kTT * 32);
    part[lane] = term[0];
    part[32 + lane] = term[1];
    // The warp that finishes the entry's last task adds the block terms of every row in a fixed
    // order, finishes the rows and hands the slot back to the producer.
    __threadfence_block();
    __syncwarp();
    int done = 0;
    if (lane == 0) done = atomicAdd(&s_misc[3 + s], 1);
    done = __shfl_sync(0xffffffffu, done, 0);
    if (done != C::kTasks - 1) continue;
    __threadfence_block();
    const int pair0 = ring.meta[s].pair0, r0 = ring.meta[s].row0;
    const float* pt = partials + s * C::kTasks * (kTT * 32);
    if (!down) {
      const int item = ring.meta[s].item, ipb = ring.meta[s].item_pair0, itok = ring.meta[s].item_tok;
      for (int t = 0; t < ntp; ++t) {
        float v = 0.0f;
#pragma unroll
        for (int b = 0; b < C::kTasks; ++b) v += pt[(b * kTT + t) * 32 + lane];
        const float u = __shfl_down_sync(0xffffffffu, v, 16);
        if (lane < 16) ws.h[size_t(pair0 + t) * I + r0 + lane] = silu_mul(v, u);
      }
      __syncwarp();
      if (lane == 0) {
        s_misc[3 + s] = 0;
        mbar_arrive(&ring.empty[s]);
      }
      item_contribution_done(ws, item, ipb, itok, gu_tpi * ((itok + kTT - 1) / kTT), down_act, I, lane);
    } else {
      const float w0 = ring.meta[s].wgt[0], w1 = ring.meta[s].wgt[1];
#pragma unroll
      for (int g = 0; g < C::kDnRows / 32; ++g) {
        const float v0 = pt[((2 * g) * kTT + 0) * 32 + lane] + pt[((2 * g + 1) * kTT + 0) * 32 + lane];
        ws.partial[size_t(pair0) * H + r0 + 32 * g + lane] = w0 * v0;
        if (ntp == 2) {
          const float v1 = pt[((2 * g) * kTT + 1) * 32 + lane] + pt[((2 * g + 1) * kTT + 1) * 32 + lane];
          ws.partial[size_t(pair0 + 1) * H + r0 + 32 * g + lane] = w1 * v1;
        }
      }
      __syncwarp();
      if (lane == 0) {
        s_misc[3 + s] = 0;
        mbar_arrive(&ring.empty[s]);
      }
    }
  }
}
