// IQ3_S streaming kernels of the decode path (gate/up and down), included by moe_decode.cu inside
// namespace fb's anonymous namespace.
//
// Shape of the work. A lane owns a weight row; a warp task is one 110-byte block (256 weights) of 32
// rows (gate/up: 16 gate rows + the 16 matching up rows; down: 32 rows, both blocks of the row), so a
// staged tile splits into many small tasks that sixteen consumer warps draw from a shared-memory
// ticket. Tiles are small (35 KB gate/up, 28 KB down) and the ring is three / five stages deep: at any
// time two / four tiles are in flight from HBM while one is being consumed, and enough tasks are
// resident that no scheduler runs out of warps (a two-stage ring of 70 KB tiles left the consumer
// warps waiting on the full barriers for 40 % of their time).
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
__host__ __device__ constexpr int q8k_planar_scales_off(int k) { return k; }
__host__ __device__ constexpr int q8k_planar_asum_off(int k) { return k + 64; }
__host__ __device__ constexpr int q8k_planar_bytes(int k) { return k + 64 + ((k / 32 * 2 + 15) & ~15); }
static_assert(q8k_planar_bytes(2560) <= FB_XQ_STRIDE && q8k_planar_bytes(512) <= FB_HQ_STRIDE, "row strides");
static_assert(q8k_planar_bytes(2560) % 16 == 0 && q8k_planar_bytes(512) % 16 == 0, "bulk copies");

// ------------------------------------------------------------------------------ codebook for the 2x+1 form
// Entry i of lane l at word i*32 + l (as iq3s_tables_fill), bytes (g - 1) / 2.
__device__ __forceinline__ void iq3s_half_tables_fill(uint32_t* gridrep, uint32_t* signtab) {
  for (int i = threadIdx.x; i < 512; i += blockDim.x) {
    const uint32_t w = (iq3s_grid_entry(i) >> 1) & 0x07070707u;
    uint4 v = make_uint4(w, w, w, w);
    uint4* dst = reinterpret_cast<uint4*>(gridrep + i * 32);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = v;
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
template <bool MIS, int TT>
__device__ __forceinline__ void iq3s_block_idot2(const uint32_t* w, const uint32_t* grid_lane, uint32_t sign_base,
                                                 const int8_t* const (&act)[TT], const int16_t* const (&asum)[TT],
                                                 int (&bsum)[TT]) {
  const uint32_t sc = iq3s_stream<MIS>(w, 26);
  int4 as[TT];
#pragma unroll
  for (int t = 0; t < TT; ++t) {
    bsum[t] = 0;
    as[t] = *reinterpret_cast<const int4*>(asum[t]);
  }
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    const uint32_t qh = iq3s_stream<MIS>(w, 16 + half);
    const uint32_t sch = sc >> (16 * half);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int ib = 4 * half + i;
      const int8_t* a[TT];
#pragma unroll
      for (int t = 0; t < TT; ++t) a[t] = act[t] + 32 * ib;
      int P[TT];
      iq3s_sub_dot<TT>(iq3s_stream<MIS>(w, 2 * ib), iq3s_stream<MIS>(w, 2 * ib + 1), qh, 8 * i,
                       iq3s_stream<MIS>(w, 18 + ib), grid_lane, sign_base, a, P);
      const int mult = 2 * int((sch >> (4 * i)) & 0xFu) + 1;
#pragma unroll
      for (int t = 0; t < TT; ++t) {
        // the two sums of this half's sub-blocks sit in words (x, y) / (z, w) of the int4, 16 bits each
        const int pair = half == 0 ? (i < 2 ? as[t].x : as[t].y) : (i < 2 ? as[t].z : as[t].w);
        const int A = (i & 1) ? (pair >> 16) : int(short(pair & 0xFFFF));
        bsum[t] += mult * (2 * P[t] + A);
      }
    }
  }
}

// scale of the block, fp16 -> fp32
template <bool MIS>
__device__ __forceinline__ float iq3s_block_d(const uint32_t* w) {
  const uint32_t v = MIS ? (w[0] & 0xFFFFu) : (w[0] >> 16);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(v)));
}

// ------------------------------------------------------------------------------ multi-stage ring
template <int S>
struct RingN {
  uint64_t* full;   // [S] count 1 + tx bytes
  uint64_t* empty;  // [S]
  volatile StageMeta* meta;  // [S]
  volatile int* abort;
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
  }
  *r.abort = 0;
  mbar_fence_init();
}

// Producer loop of one CTA (one thread): draws tiles from `counter`, stages every pass of each tile
// through issue(slot, ...), and finally posts the end marker in every slot.
template <int S, class IssueF>
__device__ __forceinline__ void producer_loop_n(const RingN<S>& r, const fb_moe_decode_workspace& ws, int* counter,
                                                int n_tiles, int tiles_per_item, int rows_per_tile, IssueF issue) {
  const fb_moe_decode_work* work = ws.work;
  int i = 0;
  auto slot_free = [&](int s) -> bool {
    if (*r.abort) return false;
    if (i >= S && !mbar_wait_hint(&r.empty[s], ((i / S) - 1) & 1)) {
      *r.abort = 1;
      atomicMax(ws.status, uint32_t(FB_STATUS_PIPELINE_TIMEOUT));
      return false;
    }
    return true;
  };
  int next = atomicAdd(counter, 1);  // drawn one step ahead of its use
  while (true) {
    const int tile = next;
    if (tile >= n_tiles) break;
    next = atomicAdd(counter, 1);
    const int pos = tile / tiles_per_item;
    const int item = ws.sched[kSchedOrder + pos];
    const int sub = tile - pos * tiles_per_item;
    const int pb = work->item_pair_begin[item];
    const int ntok = work->item_pair_begin[item + 1] - pb;
    const int slot_id = work->item_slot[item];
    for (int tok0 = 0; tok0 < ntok; tok0 += kTT, ++i) {
      const int s = i % S;
      if (!slot_free(s)) return;
      volatile StageMeta* m = &r.meta[s];
      m->tile = tile;
      m->pair0 = pb + tok0;
      m->ntp = min(kTT, ntok - tok0);
      m->row0 = sub * rows_per_tile;
      m->item = item;
      m->item_pair0 = pb;
      m->item_tok = ntok;
      for (int t = 0; t < kTT; ++t) m->wgt[t] = tok0 + t < ntok ? work->pair_weight[pb + tok0 + t] : 0.0f;
      issue(s, slot_id, sub, pb + tok0, min(kTT, ntok - tok0));
    }
  }
  for (int e = 0; e < S; ++e, ++i) {  // end marker in every slot: every waiting warp sees it
    const int s = i % S;
    if (!slot_free(s)) return;
    r.meta[s].tile = -1;
    mbar_arrive(&r.full[s]);
  }
}

// Consumer side: draws the next (entry, task) ticket; returns false at the end.
template <int S, int TASKS>
__device__ __forceinline__ bool draw_task_n(const RingN<S>& r, int* ticket_ctr, uint32_t* status, int lane, int& s,
                                            int& task) {
  int ticket = 0;
  if (lane == 0) ticket = atomicAdd(ticket_ctr, 1);
  ticket = __shfl_sync(0xffffffffu, ticket, 0);
  const int seq = ticket / TASKS;
  task = ticket - seq * TASKS;
  s = seq % S;
  if (*r.abort) return false;
  if (!mbar_wait_hint(&r.full[s], (seq / S) & 1)) {
    *r.abort = 1;
    atomicMax(status, uint32_t(FB_STATUS_PIPELINE_TIMEOUT));
    return false;
  }
  return r.meta[s].tile >= 0;
}

// ------------------------------------------------------------------------------ gate/up, IQ3_S
// Tile = 16 intermediate rows: 16 gate rows and the 16 matching up rows (17,600 bytes each) plus the
// activation rows of the pass. Task b (0..9) = block b of all 32 rows: lanes 0-15 the gate rows, lanes
// 16-31 the up rows. The warp that finishes a tile's last task adds each row's ten block terms in block
// order, pairs gate with up through a shuffle, applies SwiGLU and frees the slot.
struct GateUp3 {
  static constexpr int kJ = 16, kRowBytes = 1100, kWarps = 16, kTasks = 10, kStages = 3;
  static constexpr int kPart = kJ * kRowBytes;                 // 17,600
  static constexpr int kActBytes = q8k_planar_bytes(H);        // 2,784
  static constexpr int kStage = 2 * kPart + kTT * kActBytes;   // 40,768
  static constexpr int kPartialFloats = kStages * kTasks * kTT * 32;
  static constexpr size_t kSmem = size_t(kGridRepBytes) + 256 + size_t(kStages) * kStage + kPartialFloats * 4 + 128;
};
static_assert(GateUp3::kStage % 16 == 0 && GateUp3::kPart % 16 == 0, "bulk copy alignment");

__global__ void __launch_bounds__((GateUp3::kWarps + 1) * 32, 1)
gate_up_iq3s_kernel(fb_moe_expert_layout L, fb_moe_decode_workspace ws) {
  using C = GateUp3;
  constexpr int S = C::kStages;
  extern __shared__ __align__(256) uint8_t smem[];
  uint32_t* gridrep = reinterpret_cast<uint32_t*>(smem);
  uint32_t* signtab = reinterpret_cast<uint32_t*>(smem + kGridRepBytes);  // 256-byte aligned
  uint8_t* stage0 = smem + kGridRepBytes + 256;
  float* partials = reinterpret_cast<float*>(stage0 + S * C::kStage);
  uint64_t* bars = reinterpret_cast<uint64_t*>(partials + C::kPartialFloats);
  __shared__ StageMeta s_meta[S];
  __shared__ int s_misc[2 + S];  // [0] abort, [1] task ticket, [2..] finished tasks per slot
  RingN<S> ring{bars, bars + S, s_meta, s_misc};

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  iq3s_half_tables_fill(gridrep, signtab);
  if (tid == 0) {
    ringn_init(ring);
    for (int i = 1; i < 2 + S; ++i) s_misc[i] = 0;
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait_prior();

  const fb_moe_decode_work* work = ws.work;
  const int n_items = min(max(work->n_items, 0), kMaxPairs);
  const int I = L.inter;
  const int tpi = I / C::kJ;
  const int n_tiles = n_items * tpi;
  const int down_act = act_of(L.down_format);

  if (warp == C::kWarps) {
    // ---------------- producer: one lane draws tiles and issues their bulk copies into the ring.
    if (lane == 0) {
      producer_loop_n<S>(ring, ws, ws.sched + kSchedGateUp, n_tiles, tpi, C::kJ,
                         [&](int s, int slot_id, int sub, int pair0, int ntp) {
                           const uint8_t* blob = L.slots + int64_t(slot_id) * L.blob_stride;
                           uint8_t* st = stage0 + s * C::kStage;
                           mbar_expect_tx(&ring.full[s], uint32_t(2 * C::kPart + ntp * C::kActBytes));
                           const size_t off = size_t(sub) * C::kPart;
                           bulk_g2s(st, blob + L.gate_offset + off, C::kPart, &ring.full[s]);
                           bulk_g2s(st + C::kPart, blob + L.up_offset + off, C::kPart, &ring.full[s]);
                           for (int t = 0; t < ntp; ++t)
                             bulk_g2s(st + 2 * C::kPart + t * C::kActBytes,
                                      ws.xq + size_t(work->pair_token[pair0 + t]) * FB_XQ_STRIDE, C::kActBytes,
                                      &ring.full[s]);
                         });
    }
    return;
  }

  // ---------------- consumers
  const uint32_t* grid_lane = gridrep + lane;
  const uint32_t sign_base = smem_u32(signtab);
  const int row_off = (lane >> 4) * C::kPart + (lane & 15) * C::kRowBytes;
  while (true) {
    int s, task;
    if (!draw_task_n<S, C::kTasks>(ring, &s_misc[1], ws.status, lane, s, task)) break;
    const int ntp = ring.meta[s].ntp;
    uint8_t* st = stage0 + s * C::kStage;
    const uint8_t* act0 = st + 2 * C::kPart;
    const uint8_t* blk = st + row_off + task * 110;
    float* part = partials + (s * C::kTasks + task) * (kTT * 32);
    const bool mis = (task & 1) == 0;  // even blocks start on a word boundary: their stream is 2 bytes off
    const uint32_t* w = reinterpret_cast<const uint32_t*>(blk - (mis ? 0 : 2));
    if (ntp == 1) {
      const int8_t* a[1] = {reinterpret_cast<const int8_t*>(act0) + 256 * task};
      const int16_t* as[1] = {reinterpret_cast<const int16_t*>(act0 + q8k_planar_asum_off(H)) + 8 * task};
      int bs[1];
      float d;
      if (mis) {
        iq3s_block_idot2<true, 1>(w, grid_lane, sign_base, a, as, bs);
        d = iq3s_block_d<true>(w);
      } else {
        iq3s_block_idot2<false, 1>(w, grid_lane, sign_base, a, as, bs);
        d = iq3s_block_d<false>(w);
      }
      part[lane] = float(bs[0]) * (d * reinterpret_cast<const float*>(act0 + H)[task]);
    } else {
      const uint8_t* act1 = act0 + C::kActBytes;
      const int8_t* a[2] = {reinterpret_cast<const int8_t*>(act0) + 256 * task,
                            reinterpret_cast<const int8_t*>(act1) + 256 * task};
      const int16_t* as[2] = {reinterpret_cast<const int16_t*>(act0 + q8k_planar_asum_off(H)) + 8 * task,
                              reinterpret_cast<const int16_t*>(act1 + q8k_planar_asum_off(H)) + 8 * task};
      int bs[2];
      float d;
      if (mis) {
        iq3s_block_idot2<true, 2>(w, grid_lane, sign_base, a, as, bs);
        d = iq3s_block_d<true>(w);
      } else {
        iq3s_block_idot2<false, 2>(w, grid_lane, sign_base, a, as, bs);
        d = iq3s_block_d<false>(w);
      }
      part[lane] = float(bs[0]) * (d * reinterpret_cast<const float*>(act0 + H)[task]);
      part[32 + lane] = float(bs[1]) * (d * reinterpret_cast<const float*>(act1 + H)[task]);
    }
    // The warp that finishes the entry's last task adds the ten block terms of every row (fixed
    // order), applies SwiGLU and hands the slot back to the producer.
    __threadfence_block();
    __syncwarp();
    int done = 0;
    if (lane == 0) done = atomicAdd(&s_misc[2 + s], 1);
    done = __shfl_sync(0xffffffffu, done, 0);
    if (done == C::kTasks - 1) {
      __threadfence_block();
      const int pair0 = ring.meta[s].pair0, j0 = ring.meta[s].row0;
      const int item = ring.meta[s].item, ipb = ring.meta[s].item_pair0, itok = ring.meta[s].item_tok;
      const float* pt = partials + s * C::kTasks * (kTT * 32);
      for (int t = 0; t < ntp; ++t) {
        float v = 0.0f;
#pragma unroll
        for (int b = 0; b < C::kTasks; ++b) v += pt[(b * kTT + t) * 32 + lane];
        const float u = __shfl_down_sync(0xffffffffu, v, 16);
        if (lane < 16) ws.h[size_t(pair0 + t) * I + j0 + lane] = silu_mul(v, u);
      }
      __syncwarp();
      if (lane == 0) {
        s_misc[2 + s] = 0;
        mbar_arrive(&ring.empty[s]);
      }
      item_contribution_done(ws, item, ipb, itok, tpi * ((itok + kTT - 1) / kTT), down_act, lane);
    }
  }
}

// ------------------------------------------------------------------------------ down, IQ3_S, inter 512
// A row is two blocks (220 bytes); tile = 128 rows = four tasks of 32 rows, one row per lane, no
// cross-warp reduction.
struct Down3 {
  static constexpr int kRows = 128, kRowBytes = 220, kWarps = 16, kTasks = 4, kStages = 5, kInter = 512;
  static constexpr int kTile = kRows * kRowBytes;              // 28,160
  static constexpr int kActBytes = q8k_planar_bytes(kInter);   // 608
  static constexpr int kStage = kTile + kTT * kActBytes;       // 29,376
  static constexpr size_t kSmem = size_t(kGridRepBytes) + 256 + size_t(kStages) * kStage + 128;
};
static_assert(Down3::kStage % 16 == 0 && Down3::kTile % 16 == 0, "bulk copy alignment");

__global__ void __launch_bounds__((Down3::kWarps + 1) * 32, 1)
down_iq3s_kernel(fb_moe_expert_layout L, fb_moe_decode_workspace ws) {
  using C = Down3;
  constexpr int S = C::kStages;
  extern __shared__ __align__(256) uint8_t smem[];
  uint32_t* gridrep = reinterpret_cast<uint32_t*>(smem);
  uint32_t* signtab = reinterpret_cast<uint32_t*>(smem + kGridRepBytes);
  uint8_t* stage0 = smem + kGridRepBytes + 256;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage0 + S * C::kStage);
  __shared__ StageMeta s_meta[S];
  __shared__ int s_misc[2 + S];
  RingN<S> ring{bars, bars + S, s_meta, s_misc};

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  iq3s_half_tables_fill(gridrep, signtab);
  if (tid == 0) {
    ringn_init(ring);
    for (int i = 1; i < 2 + S; ++i) s_misc[i] = 0;
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait_prior();

  const fb_moe_decode_work* work = ws.work;
  const int n_items = min(max(work->n_items, 0), kMaxPairs);
  constexpr int tpi = H / C::kRows;
  const int n_tiles = n_items * tpi;

  if (warp == C::kWarps) {
    if (lane == 0) {
      producer_loop_n<S>(ring, ws, ws.sched + kSchedDown, n_tiles, tpi, C::kRows,
                         [&](int s, int slot_id, int sub, int pair0, int ntp) {
                           const uint8_t* blob = L.slots + int64_t(slot_id) * L.blob_stride;
                           uint8_t* st = stage0 + s * C::kStage;
                           mbar_expect_tx(&ring.full[s], uint32_t(C::kTile + ntp * C::kActBytes));
                           bulk_g2s(st, blob + L.down_offset + size_t(sub) * C::kTile, C::kTile, &ring.full[s]);
                           for (int t = 0; t < ntp; ++t)
                             bulk_g2s(st + C::kTile + t * C::kActBytes, ws.hq + size_t(pair0 + t) * FB_HQ_STRIDE,
                                      C::kActBytes, &ring.full[s]);
                         });
    }
    return;
  }

  const uint32_t* grid_lane = gridrep + lane;
  const uint32_t sign_base = smem_u32(signtab);
  while (true) {
    int s, task;
    if (!draw_task_n<S, C::kTasks>(ring, &s_misc[1], ws.status, lane, s, task)) break;
    const int ntp = ring.meta[s].ntp, pair0 = ring.meta[s].pair0, r0 = ring.meta[s].row0;
    const float w0 = ring.meta[s].wgt[0], w1 = ring.meta[s].wgt[1];
    uint8_t* st = stage0 + s * C::kStage;
    const uint8_t* act0 = st + C::kTile;
    const int row = 32 * task + lane;
    const uint32_t* unit = reinterpret_cast<const uint32_t*>(st + row * C::kRowBytes);
    const uint32_t* wB = unit + 27;  // the word whose high half holds the second block's scale
    if (ntp == 1) {
      const int8_t* a[1] = {reinterpret_cast<const int8_t*>(act0)};
      const int16_t* as[1] = {reinterpret_cast<const int16_t*>(act0 + q8k_planar_asum_off(C::kInter))};
      const float* da = reinterpret_cast<const float*>(act0 + C::kInter);
      int bs[1];
      iq3s_block_idot2<true, 1>(unit, grid_lane, sign_base, a, as, bs);
      float acc = float(bs[0]) * (iq3s_block_d<true>(unit) * da[0]);
      const int8_t* a2[1] = {a[0] + 256};
      const int16_t* as2[1] = {as[0] + 8};
      iq3s_block_idot2<false, 1>(wB, grid_lane, sign_base, a2, as2, bs);
      acc = fmaf(float(bs[0]), iq3s_block_d<false>(wB) * da[1], acc);
      ws.partial[size_t(pair0) * H + r0 + row] = w0 * acc;
    } else {
      const uint8_t* act1 = act0 + C::kActBytes;
      const int8_t* a[2] = {reinterpret_cast<const int8_t*>(act0), reinterpret_cast<const int8_t*>(act1)};
      const int16_t* as[2] = {reinterpret_cast<const int16_t*>(act0 + q8k_planar_asum_off(C::kInter)),
                              reinterpret_cast<const int16_t*>(act1 + q8k_planar_asum_off(C::kInter))};
      const float* da0 = reinterpret_cast<const float*>(act0 + C::kInter);
      const float* da1 = reinterpret_cast<const float*>(act1 + C::kInter);
      int bs[2];
      iq3s_block_idot2<true, 2>(unit, grid_lane, sign_base, a, as, bs);
      const float dA = iq3s_block_d<true>(unit);
      float acc0 = float(bs[0]) * (dA * da0[0]), acc1 = float(bs[1]) * (dA * da1[0]);
      const int8_t* a2[2] = {a[0] + 256, a[1] + 256};
      const int16_t* as2[2] = {as[0] + 8, as[1] + 8};
      iq3s_block_idot2<false, 2>(wB, grid_lane, sign_base, a2, as2, bs);
      const float dB = iq3s_block_d<false>(wB);
      acc0 = fmaf(float(bs[0]), dB * da0[1], acc0);
      acc1 = fmaf(float(bs[1]), dB * da1[1], acc1);
      ws.partial[size_t(pair0) * H + r0 + row] = w0 * acc0;
      ws.partial[size_t(pair0 + 1) * H + r0 + row] = w1 * acc1;
    }
    __syncwarp();
    if (lane == 0) {
      const int done = atomicAdd(&s_misc[2 + s], 1);
      if (done == C::kTasks - 1) {  // the tile's last task hands the slot back to the producer
        s_misc[2 + s] = 0;
        mbar_arrive(&ring.empty[s]);
      }
    }
  }
}
