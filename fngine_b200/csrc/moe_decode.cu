// Decode-width (T <= 16) routed-expert kernels on native GGUF expert bytes.
//
//   route    router projection, once-per-token activation quantization
//   select   top-10 and the sorted work list (stand-alone from given logits, or inside the expert kernel)
//   gate_up  h[pair][j] = silu(gate_j . x) * (up_j . x)
//   down     partial[pair][n] = w_pair * (down_n . q8(h[pair]))
//   combine  y[t] = sum of token t's partials in slot order (+ shared, + residual write)
//
// gate_up and down of IQ3_S and IQ4_NL experts are one persistent kernel, one CTA per SM
// (moe_decode_iq3s.cuh): a producer thread streams tiles of the expert blob into a three-stage
// shared-memory ring with 1-D bulk async copies (TMA, no multicast) signalled through mbarriers;
// consumer warps decode the blocks from shared memory and accumulate exact int8 dot products (dp4a).
// (IQ4_NL down at intermediate 640 keeps an earlier two-stage kernel; the other formats have plain
// kernels, moe_decode_generic.cuh.) Numerics are those of the
// reference's CPU expert tier (src/cpu/iq_cpu.h:12-40 of the reference project): Q8_K activations
// for IQ3_S weights, Q8_0 for IQ4_NL, integer sums per block, one fp32 scale step per block.
#include "iq_decode.cuh"

#include <cstring>

#include <cuda_bf16.h>

namespace fb {
namespace {

constexpr int H = FB_HIDDEN;
constexpr int kTopK = FB_TOPK;
constexpr int kExperts = FB_EXPERTS;
constexpr int kMaxTok = FB_DECODE_MAX_TOKENS;
constexpr int kMaxPairs = FB_DECODE_MAX_PAIRS;
constexpr int kTT = 2;  // tokens of one work item handled per pass over a staged tile
// ws.sched: [0] gate/up tile counter, [1] down tile counter, [8..168) item order
constexpr int kSchedOrderBase = 8;
constexpr int kEpMaxRanks = FB_EP_MAX_RANKS;
constexpr uint32_t kPeerSpinLimit = 1u << 20;  // default polls of a peer-written flag before giving up (about a second)

// Flag-in-data exchange lines (the low-latency protocol of collective libraries): 16 bytes =
// {value 0, step, value 1, step}, written by ONE 16-byte store, so a reader that sees the step
// number of the current step in both flag words holds both values - no fence, no separate flag.
__device__ __forceinline__ void ll_store(uint4* line, float v0, float v1, uint32_t step) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(line), "r"(__float_as_uint(v0)), "r"(step),
               "r"(__float_as_uint(v1)), "r"(step)
               : "memory");
}
// Polls the line (at most `limit` times) until both halves carry `step`.
__device__ __forceinline__ float2 ll_read(const uint4* line, uint32_t step, uint32_t* status, uint32_t limit) {
  uint4 v;
  for (uint32_t i = 0; i < limit; ++i) {
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(line)
                 : "memory");
    if (v.y == step && v.w == step) return make_float2(__uint_as_float(v.x), __uint_as_float(v.z));
    // once any reader of this launch has given up, the others stop waiting too (checked rarely)
    if ((i & 1023u) == 1023u && *reinterpret_cast<volatile uint32_t*>(status) >= uint32_t(FB_STATUS_PIPELINE_TIMEOUT))
      return make_float2(0.0f, 0.0f);
    __nanosleep(100);
  }
  atomicMax(status, uint32_t(FB_STATUS_PIPELINE_TIMEOUT));
  return make_float2(0.0f, 0.0f);
}
constexpr int kSchedInts = 256;

__host__ __device__ constexpr int act_row_bytes_planar(int act, int k) {
  return act == FB_ACT_Q8_K ? k + 64 : k + k / 8;
}
__host__ __device__ constexpr int act_of(int fmt) {
  return fmt == FB_FMT_IQ4_NL || fmt == FB_FMT_Q2_0 ? FB_ACT_Q8_0 : FB_ACT_Q8_K;
}
// gate/up formats without a streaming kernel (plain kernels in moe_decode_generic.cuh)
__host__ __device__ constexpr bool plain_gate_up(int fmt) {
  return fmt == FB_FMT_IQ3_XXS || fmt == FB_FMT_IQ2_S || fmt == FB_FMT_IQ4_XS;
}
// ws.xq holds [2][16][FB_XQ_STRIDE]: the Q8_K rows of the step's tokens, then their Q8_0 rows. A workspace
// made for a layout gets the one its gate/up format needs; one made without a layout gets both from
// the stand-alone selection (which does not see the layout).
__host__ __device__ constexpr size_t xq_offset(int act) { return act == FB_ACT_Q8_0 ? size_t(kMaxTok) * FB_XQ_STRIDE : 0; }

__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + expf(-g)) * u; }

// Planar Q8_K rows: codes [k] | block scales float [k/256] (64 bytes reserved) | code sums of every 32
// codes, int16 [k/32] (Q8_K's bsums added in pairs; the IQ3_S kernels use them, see moe_decode_iq3s.cuh).
__host__ __device__ constexpr int q8k_asum_off(int k) { return k + 64; }

// Stores block b of a planar Q8_K row from the calling warp's quantizer output (lane l holds codes
// 8l..8l+7 of the block in q, pair_sum the sum of its 16-code group).
__device__ __forceinline__ void store_q8k_block_planar(uint8_t* out, int k, int b, const int (&q)[8], int pair_sum,
                                                       float d) {
  const int lane = threadIdx.x & 31;
  uint2 pk;
  pk.x = uint32_t(uint8_t(q[0])) | (uint32_t(uint8_t(q[1])) << 8) | (uint32_t(uint8_t(q[2])) << 16) |
         (uint32_t(uint8_t(q[3])) << 24);
  pk.y = uint32_t(uint8_t(q[4])) | (uint32_t(uint8_t(q[5])) << 8) | (uint32_t(uint8_t(q[6])) << 16) |
         (uint32_t(uint8_t(q[7])) << 24);
  *reinterpret_cast<uint2*>(out + 256 * b + 8 * lane) = pk;
  const int sum32 = pair_sum + __shfl_xor_sync(0xffffffffu, pair_sum, 2);  // lanes 4j..4j+3 hold sub-block j
  if ((lane & 3) == 0) reinterpret_cast<int16_t*>(out + q8k_asum_off(k))[8 * b + (lane >> 2)] = int16_t(sum32);
  if (lane == 0) reinterpret_cast<float*>(out + k)[b] = d;
}

// ------------------------------------------------------------------------------ activation rows
// One row of k values -> planar codes + scales, by the calling block (any number of warps).
// Q8_K: codes [k], scales float[k/256]. Q8_0: codes [k] (interleaved per block), scales float[k/32].
template <class LoadF>
__device__ __forceinline__ void quantize_row_planar(int act, int k, LoadF load, uint8_t* out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  if (act == FB_ACT_Q8_K) {
    for (int b = warp; b < k / 256; b += warps) {
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = load(256 * b + 8 * lane + i);
      int q[8], ps;
      const float d = q8k_block_warp(v, q, ps);
      store_q8k_block_planar(out, k, b, q, ps, d);
    }
  } else {
    float* scales = reinterpret_cast<float*>(out + k);
    for (int b = warp; b < k / 32; b += warps) {
      unsigned short dh;
      const int q = q8_0_block_warp(load(32 * b + lane), dh);
      out[32 * b + q8_0_interleave_index(lane)] = uint8_t(int8_t(q));
      if (lane == 0) scales[b] = __half2float(__ushort_as_half(dh));
    }
  }
}

// ------------------------------------------------------------------------------ router
// logits[t][r] = sum_k W[r][k] * x[t][k]; one warp per row (four rows per block), the row's
// weights held in registers, tokens taken four at a time so that their loads overlap; the 32 lane
// sums are added by a butterfly. Fixed order: repeated calls are bitwise identical.
template <bool XBF16>
__global__ void __launch_bounds__(128) router_kernel(const __nv_bfloat16* __restrict__ w, int rows,
                                                     const void* __restrict__ xv, int tokens,
                                                     float* __restrict__ logits, int stride) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  pdl_wait_prior();
  if (row >= rows) return;
  float wr[80];
  {
    const uint4* wp = reinterpret_cast<const uint4*>(w + size_t(row) * H);
#pragma unroll
    for (int c = 0; c < 10; ++c) {
      const uint4 v = wp[c * 32 + lane];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        wr[8 * c + 2 * i] = __uint_as_float(u[i] << 16);
        wr[8 * c + 2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
      }
    }
  }
  for (int t0 = 0; t0 < tokens; t0 += 4) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int c = 0; c < 10; ++c) {
#pragma unroll
      for (int tt = 0; tt < 4; ++tt) {
        const int t = min(t0 + tt, tokens - 1);  // clamped rows are computed and dropped
        float xs[8];
        if constexpr (XBF16) {
          const uint4 v =
              reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(xv) + size_t(t) * H)[c * 32 + lane];
          const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            xs[2 * i] = __uint_as_float(u[i] << 16);
            xs[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
          }
        } else {
          const float4* xp =
              reinterpret_cast<const float4*>(static_cast<const float*>(xv) + size_t(t) * H) + (c * 32 + lane) * 2;
          const float4 a = xp[0], b = xp[1];
          xs[0] = a.x; xs[1] = a.y; xs[2] = a.z; xs[3] = a.w;
          xs[4] = b.x; xs[5] = b.y; xs[6] = b.z; xs[7] = b.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[tt] = fmaf(wr[8 * c + i], xs[i], acc[tt]);
      }
    }
#pragma unroll
    for (int tt = 0; tt < 4; ++tt) {
      float v = acc[tt];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && t0 + tt < tokens) logits[size_t(t0 + tt) * stride + row] = v;
    }
  }
}

// The part of the work list a producer needs, in shared memory: the producer is a single thread, and a
// chain of dependent global loads per tile (visiting order -> item -> its pairs -> their tokens and
// weights, about two microseconds) would pace the whole kernel. Either copied from the device work list
// (work_cache_fill) or built in place by the CTA's own selection (select_block).
struct WorkCache {
  int order[kMaxPairs];
  int pair_begin[kMaxPairs + 1];
  int slot[kMaxPairs];
  int pair_token[kMaxPairs];
  float pair_weight[kMaxPairs];
  int n_items;
};
// Called by the 32 lanes of the producer warp (the only reader) after the wait on the preceding kernel;
// the caller follows with __syncwarp().
__device__ __forceinline__ void work_cache_fill(const fb_moe_decode_workspace& ws, WorkCache& c, int n_items) {
  const fb_moe_decode_work* work = ws.work;
  for (int i = threadIdx.x & 31; i < kMaxPairs; i += 32) {
    const bool live = i < n_items;
    c.order[i] = live ? ws.sched[kSchedOrderBase + i] : 0;
    c.slot[i] = live ? work->item_slot[i] : 0;
    c.pair_begin[i] = i <= n_items ? work->item_pair_begin[i] : 0;
    c.pair_token[i] = work->pair_token[i];
    c.pair_weight[i] = work->pair_weight[i];
  }
  if ((threadIdx.x & 31) == 0) {
    c.pair_begin[kMaxPairs] = n_items == kMaxPairs ? work->item_pair_begin[kMaxPairs] : 0;
    c.n_items = n_items;
  }
}

// ------------------------------------------------------------------------------ select
// topk(t, scratch, ids, weights): the calling warp writes token t's top-10 (ids and softmax weights, rank
// order) to ids / weights in shared memory; scratch = 32 entries of shared memory for that warp.
// Called by every thread of a block of 512 or more threads. The work list goes to `wc` in shared memory
// (complete when the call returns) and, with `publish`, to the device work list as well; `reset` clears
// the tile and item counters of the streaming kernels (only where no such kernel can be running). The
// list is a function of the logits alone: every block that runs this on the same logits builds the same
// list. Every CTA of a decode step waits for this, so it is kept a short chain of six barriers: token
// masks per physical slot (shared-memory atomics), a scan over the 512 slots (thread = slot), the pairs
// placed from the scan, and the items ranked by a counting sort on their token counts (warp votes). Few
// warps do this work and a warp on its own retires an instruction every few cycles: what counts here is the
// number of instructions on the longest chain, not the arithmetic. (Up to three tokens: one warp, shuffles.)
//   items  = distinct selected experts held on this rank, in physical-slot order
//   pairs  = (item, token), tokens ascending inside an item
//   order  = items by token count, most first, ties by item index (the streaming kernels' visiting order)
template <class TopkF>
__device__ __forceinline__ void select_block(TopkF topk, const int32_t* slot_of, int T,
                                             const fb_moe_decode_workspace& ws, uint32_t* counts, bool remote_ok,
                                             bool publish, bool reset, WorkCache& wc) {
  static_assert(kMaxPairs % 32 == 0 && kMaxTok % 4 == 0, "the ranking below votes by whole warps and reads 16-byte groups");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __shared__ int s_id[kMaxTok][kTopK];
  __shared__ float s_w[kMaxTok][kTopK];
  __shared__ int s_pair[kMaxTok][kTopK];
  __shared__ uint32_t s_tok[kExperts];  // physical slot -> mask of the tokens that chose it
  __shared__ int s_begin[kExperts];     // physical slot -> first pair of its item
  __shared__ int s_scan[2][kExperts / 32];
  __shared__ __align__(16) int s_item_cnt[kMaxPairs];
  __shared__ __align__(16) int s_hist[kMaxPairs / 32][kMaxTok];  // [warp of items][token count - 1] -> items
  __shared__ uint2 s_cand[kMaxTok][32];
  fb_moe_decode_work* work = ws.work;
  if (tid < kExperts) s_tok[tid] = 0;
  if (reset) {
    if (tid < kMaxPairs) ws.item_done[tid] = 0;
    if (tid < kSchedOrderBase) ws.sched[tid] = 0;
  }
  if (warp < T) topk(warp, s_cand[warp], s_id[warp], s_w[warp]);
  __syncthreads();
  const int np = T * kTopK;
  if (np <= 32) {
    // Up to three tokens: the pairs fit one warp, which builds the whole list through shuffles (lane = pair),
    // two barriers in all instead of five. Same list as the general path below.
    if (warp == 0) {
      const bool pv = lane < np;
      const int t = lane / kTopK, k = lane - t * kTopK;
      const int e = pv ? s_id[t][k] : 0;
      int slot = !pv ? -1 : slot_of ? slot_of[e] : e;
      if (slot >= kExperts) slot = -1;
      const float wt = pv ? s_w[t][k] : 0.0f;
      const int key = slot >= 0 ? slot * kMaxTok + t : 0x7fffffff;  // pairs not held here sort last
      // (a lone warp runs at a few cycles per instruction: the loops below take np turns, not 32, and a single
      // token, whose ten pairs are ten different experts, needs only the first)
      int idx = 0, trank = 0, cnt = 0;
#pragma unroll 2
      for (int j = 0; j < np; ++j) {
        const int kj = __shfl_sync(0xffffffffu, key, j);
        const bool same = kj != 0x7fffffff && (kj / kMaxTok) == slot;
        idx += kj < key ? 1 : 0;
        cnt += same ? 1 : 0;
        trank += same && kj < key ? 1 : 0;
      }
      const bool hot = slot >= 0, first = hot && trank == 0;
      const uint32_t hot_m = __ballot_sync(0xffffffffu, hot), first_m = __ballot_sync(0xffffffffu, first);
      const int n_pairs = __popc(hot_m), n_items = __popc(first_m);
      int item = idx, rank = idx;  // one token: every held pair is an item of one token, in key order
      if (T > 1) {
        item = 0;  // distinct slots below this pair's slot = first pairs with a smaller key
#pragma unroll 2
        for (int j = 0; j < np; ++j) {
          const int kj = __shfl_sync(0xffffffffu, key, j);
          item += ((first_m >> j) & 1u) && (kj / kMaxTok) < slot ? 1 : 0;
        }
        rank = 0;  // visiting order among the items: more tokens first, then lower item index
#pragma unroll 2
        for (int j = 0; j < np; ++j) {
          const int cj = __shfl_sync(0xffffffffu, cnt, j), ij = __shfl_sync(0xffffffffu, item, j);
          rank += ((first_m >> j) & 1u) && (cj > cnt || (cj == cnt && ij < item)) ? 1 : 0;
        }
      }
      if (hot) {
        wc.pair_token[idx] = t;
        wc.pair_weight[idx] = wt;
        if (publish) {
          work->pair_token[idx] = t;
          work->pair_weight[idx] = wt;
        }
      }
      if (first) {
        wc.slot[item] = slot;
        wc.pair_begin[item] = idx;
        wc.order[rank] = item;
        if (publish) {
          work->item_slot[item] = slot;
          work->item_pair_begin[item] = idx;
          ws.sched[kSchedOrderBase + rank] = item;
        }
      }
      if (lane == 0) {
        wc.pair_begin[n_items] = n_pairs;
        wc.n_items = n_items;
      }
      if (pv && counts) atomicAdd(&counts[e], 1u);
      if (publish) {
        if (pv) {
          work->topk_expert[t][k] = e;
          work->topk_weight[t][k] = wt;
        }
        // a token's held pairs in pair order (= slot order)
        int prank = idx, nh = n_pairs;
        if (T > 1) {
          prank = nh = 0;
#pragma unroll 2
          for (int j = 0; j < np; ++j) {
            const int kj = __shfl_sync(0xffffffffu, key, j), ixj = __shfl_sync(0xffffffffu, idx, j);
            const bool mine = j / kTopK == t && kj != 0x7fffffff;
            nh += mine ? 1 : 0;
            prank += mine && ixj < idx ? 1 : 0;
          }
        }
        if (hot) work->token_pairs[t][prank] = idx;
        if (pv && k == 0) {
          work->token_pair_count[t] = nh;
          work->token_cold_count[t] = kTopK - nh;
        }
        if (lane == 0) {
          work->item_pair_begin[n_items] = n_pairs;
          work->n_items = n_items;
          work->n_pairs = n_pairs;
          work->n_cold = np - n_pairs;
          work->tokens = T;
          if (np - n_pairs && !remote_ok) atomicMax(ws.status, uint32_t(FB_STATUS_BAD_WORK));
        }
      }
    }
    __syncthreads();
    return;
  }
  const bool valid = tid < np;
  const int pt = tid / kTopK, pk = tid - pt * kTopK;
  int my_e = 0, my_slot = -1;
  if (valid) {
    my_e = s_id[pt][pk];
    my_slot = slot_of ? slot_of[my_e] : my_e;
    if (my_slot >= kExperts) my_slot = -1;
    if (my_slot >= 0) atomicOr(&s_tok[my_slot], 1u << pt);
    if (counts) atomicAdd(&counts[my_e], 1u);
  }
  __syncthreads();
  // inclusive scans of (tokens, chosen flag) over the 512 slots: inside the warps first
  const int c = tid < kExperts ? __popc(s_tok[tid]) : 0;
  int incl_c = c, incl_n = c > 0 ? 1 : 0;
  if (tid < kExperts) {  // (whole warps)
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, incl_c, o), y = __shfl_up_sync(0xffffffffu, incl_n, o);
      if (lane >= o) {
        incl_c += x;
        incl_n += y;
      }
    }
    if (lane == 31) {
      s_scan[0][warp] = incl_c;
      s_scan[1][warp] = incl_n;
    }
  }
  __syncthreads();
  int base_c = 0, base_n = 0, n_pairs = 0, n_items = 0;
#pragma unroll
  for (int i = 0; i < kExperts / 32; ++i) {
    const int sc = s_scan[0][i], sn = s_scan[1][i];
    base_c += i < warp ? sc : 0;
    base_n += i < warp ? sn : 0;
    n_pairs += sc;
    n_items += sn;
  }
  if (c > 0) {  // thread = a chosen slot = an item
    const int item = base_n + incl_n - 1, pair_begin = base_c + incl_c - c;
    s_begin[tid] = pair_begin;
    s_item_cnt[item] = c;
    wc.slot[item] = tid;
    wc.pair_begin[item] = pair_begin;
    if (publish) {
      work->item_slot[item] = tid;
      work->item_pair_begin[item] = pair_begin;
    }
  }
  if (tid == 0) {
    wc.pair_begin[n_items] = n_pairs;
    wc.n_items = n_items;
    if (publish) {
      work->item_pair_begin[n_items] = n_pairs;
      work->n_items = n_items;
      work->n_pairs = n_pairs;
      work->n_cold = np - n_pairs;
      work->tokens = T;
      if (np - n_pairs && !remote_ok) atomicMax(ws.status, uint32_t(FB_STATUS_BAD_WORK));
    }
  }
  __syncthreads();
  if (valid) {
    int idx = -1;
    if (my_slot >= 0) {
      idx = s_begin[my_slot] + __popc(s_tok[my_slot] & ((1u << pt) - 1u));  // tokens ascending inside an item
      wc.pair_token[idx] = pt;
      wc.pair_weight[idx] = s_w[pt][pk];
      if (publish) {
        work->pair_token[idx] = pt;
        work->pair_weight[idx] = s_w[pt][pk];
      }
    }
    s_pair[pt][pk] = idx;
    if (publish) {
      work->topk_expert[pt][pk] = my_e;
      work->topk_weight[pt][pk] = s_w[pt][pk];
    }
  }
  // Visiting order: rank of an item = items with more tokens + items with as many tokens and a lower index.
  // A counting sort on the token count (1..16): every warp of items votes its histogram, then an item adds the
  // counts above its own, the earlier warps' share of its own count, and its place among its warp's equals.
  {
    const bool live = tid < n_items;
    const int mine = live ? s_item_cnt[tid] : 0;
    uint32_t equals = 0;
    if (tid < kMaxPairs) {  // (whole warps: kMaxPairs is a multiple of 32)
#pragma unroll
      for (int cnt = 1; cnt <= kMaxTok; ++cnt) {
        const uint32_t b = __ballot_sync(0xffffffffu, mine == cnt);
        equals = mine == cnt ? b : equals;
        if (lane == cnt - 1) s_hist[warp][cnt - 1] = __popc(b);
      }
    }
    __syncthreads();
    if (live) {
      int rank = __popc(equals & ((1u << lane) - 1u));
#pragma unroll
      for (int wv = 0; wv < kMaxPairs / 32; ++wv) {
        const int4* hp = reinterpret_cast<const int4*>(s_hist[wv]);
#pragma unroll
        for (int g = 0; g < kMaxTok / 4; ++g) {
          const int4 hv = hp[g];
          const int hc[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int cnt = 4 * g + i + 1;
            rank += (cnt > mine || (cnt == mine && wv < warp)) ? hc[i] : 0;
          }
        }
      }
      wc.order[rank] = tid;
      if (publish) ws.sched[kSchedOrderBase + rank] = tid;
    }
  }
  __syncthreads();
  if (publish && tid < T) {
    int idx10[kTopK];
#pragma unroll
    for (int k = 0; k < kTopK; ++k) idx10[k] = s_pair[tid][k];
    int nh = 0;
#pragma unroll
    for (int k = 0; k < kTopK; ++k) {
      if (idx10[k] >= 0) {
        int rank = 0;
#pragma unroll
        for (int k2 = 0; k2 < kTopK; ++k2) rank += (idx10[k2] >= 0 && idx10[k2] < idx10[k]) ? 1 : 0;
        work->token_pairs[tid][rank] = idx10[k];  // slot order == pair order
        ++nh;
      }
    }
    work->token_pair_count[tid] = nh;
    work->token_cold_count[tid] = kTopK - nh;
  }
}

// What a streaming kernel needs to run the selection itself (the fused layer call): every CTA builds the
// work list in its own shared memory from the logits the route kernel stored, and block 0 also writes the
// device work list for the combine kernel and the host.
struct SelectArgs {
  const float* logits;  // [tokens][stride]
  int stride;
  const int32_t* slot_of;
  int tokens;
  int remote_ok;
};

// Stand-alone selection (the reference's moe_select_publish): block 0 routes, blocks 1..T quantize
// one token's activations each.
template <bool XBF16>
__global__ void __launch_bounds__(512) select_kernel(const float* __restrict__ logits, int logits_stride,
                                                     const void* __restrict__ xv, const int32_t* __restrict__ slot_of,
                                                     int T, fb_moe_decode_workspace ws,
                                                     uint32_t* __restrict__ counts) {
  pdl_launch_dependents();
  pdl_wait_prior();
  if (blockIdx.x > 0) {
    const int t = blockIdx.x - 1;
    auto load = [&](int i) -> float {
      if constexpr (XBF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(xv)[size_t(t) * H + i]);
      else return static_cast<const float*>(xv)[size_t(t) * H + i];
    };
    for (int act = FB_ACT_Q8_K; act <= FB_ACT_Q8_0; ++act)
      if (ws.gate_up_format == 0 || act_of(ws.gate_up_format) == act)
        quantize_row_planar(act, H, load, ws.xq + xq_offset(act) + size_t(t) * FB_XQ_STRIDE);
    return;
  }
  __shared__ WorkCache s_work;  // the streaming kernels of this path read the device work list instead
  select_block(
      [&](int t, uint2* scratch, int* ids, float* wts) {
        warp_topk10_pruned([&](int e) { return logits[size_t(t) * logits_stride + e]; }, scratch, ids, wts);
      },
      slot_of, T, ws, counts, false, true, true, s_work);
}

// The selection alone, from logits a route kernel stored (one block): for layers whose gate/up format has
// only plain kernels, which read the device work list.
__global__ void __launch_bounds__(512) select_only_kernel(SelectArgs sel, fb_moe_decode_workspace ws) {
  pdl_launch_dependents();
  pdl_wait_prior();
  __shared__ WorkCache s_work;
  select_block(
      [&](int t, uint2* scratch, int* ids, float* wts) {
        warp_topk10_pruned([&](int e) { return __ldcg(sel.logits + size_t(t) * sel.stride + e); }, scratch, ids, wts);
      },
      sel.slot_of, sel.tokens, ws, nullptr, sel.remote_ok != 0, true, false, s_work);
}

// What route_kernel needs for an expert-parallel step with peer-memory exchange (n_ranks == 0: none).
struct EpRouteArgs {
  fb_ep_peers peers;
  const float* x_local;  // this rank's rows, fp32 [tpr][2560]
  int tpr;               // tokens per rank
  int parity;
  uint32_t step;
  uint32_t spin_limit;  // polls per awaited line
  int act;              // activation format the layer's gate/up weights pair with (set for every launch)
};

// Router projection and activation quantization in one launch (the head of the fused layer call; the
// selection runs inside the streaming kernel that follows, see SelectArgs). 128 blocks in sixteen
// clusters of eight: cluster g owns router rows 32g..32g+31, its CTA q the K slice [320q, 320q+320). The
// x slice of all tokens sits in the CTA's shared memory (sixteen CTAs read each slice: no line of x is
// wanted by all SMs at once), one warp per row pair (every x value read from shared memory feeds two
// rows), all tokens in flight at once. The eight slice sums of a logit meet through distributed shared
// memory: after a cluster barrier CTA q adds the slices of rows 4q..4q+3 in order 0..7 (fixed: repeated
// calls are bitwise identical) and stores the logits. No block waits on device memory for another. Every
// warp of the grid also quantizes a share of the activation blocks, and block 0 clears the counters of
// the streaming kernels (none can be running: this kernel waited for its predecessor).
constexpr int kRouteSplits = 8, kRouteSlice = H / kRouteSplits;  // 320
constexpr int kRouteGroups = kExperts / 32;                      // 16
constexpr int kRouteBlocks = kRouteGroups * kRouteSplits;
static_assert(kRouteSlice == 320, "lane layout below: two 128-element chunks and a 64-element tail");

template <bool XBF16, bool EP>
__global__ void __launch_bounds__(512) route_kernel(const __nv_bfloat16* __restrict__ w, const void* __restrict__ xv,
                                                    int T, float* __restrict__ logits, int stride,
                                                    fb_moe_decode_workspace ws, EpRouteArgs ep) {
  pdl_launch_dependents();
  pdl_wait_prior();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr bool ep_mode = EP;  // the single-GPU instantiation carries none of the exchange code
  const uint4* x_lines = nullptr;  // this rank's copy of all tokens' rows, as exchange lines
  if constexpr (EP) {
    // Expert-parallel step: this rank's own rows go to every rank as flag-in-data lines (block b
    // serves rank b % R with slice b / R of the rows); readers below poll the lines they need.
    const int R = ep.peers.n_ranks, d = int(blockIdx.x) % R, slice = int(blockIdx.x) / R, n_slices = int(gridDim.x) / R;
    // (the host refuses rank counts that do not divide the grid; the clamp keeps a stray block inside the rows)
    const int total = ep.tpr * (H / 4), lo = min(total, int(int64_t(total) * slice / n_slices)),
              hi = min(total, int(int64_t(total) * (slice + 1) / n_slices));
    uint4* dst = static_cast<uint4*>(ep.peers.x_all[d]) +
                 (size_t(ep.parity) * kMaxTok + size_t(ep.peers.rank) * ep.tpr) * (H / 2);
    const float4* src = reinterpret_cast<const float4*>(ep.x_local);
    for (int i = lo + tid; i < hi; i += 512) {
      const float4 v = src[i];
      ll_store(dst + 2 * i, v.x, v.y, ep.step);
      ll_store(dst + 2 * i + 1, v.z, v.w, ep.step);
    }
    x_lines = static_cast<const uint4*>(ep.peers.x_all[ep.peers.rank]) + size_t(ep.parity) * kMaxTok * (H / 2);
  }
  if (blockIdx.x == 0) {
    if (tid < kMaxPairs) ws.item_done[tid] = 0;
    if (tid < kSchedOrderBase) ws.sched[tid] = 0;
  }
  __shared__ __align__(16) float s_x[kMaxTok][kRouteSlice];  // x slice [token][320]
  __shared__ float s_part[32][kMaxTok];                       // this slice's sums [row of the group][token]
  const int g = blockIdx.x / kRouteSplits, q = int(cluster_cta_rank());  // (clusters are eight consecutive blocks)
  for (int i = tid; i < T * (kRouteSlice / 4); i += 512) {
    const int t = i / (kRouteSlice / 4), c = i - t * (kRouteSlice / 4);
    float4 v;
    if constexpr (ep_mode) {
      const uint4* ln = x_lines + (size_t(t) * H + q * kRouteSlice) / 2 + 2 * c;
      const float2 a = ll_read(ln, ep.step, ws.status, ep.spin_limit),
                   b2 = ll_read(ln + 1, ep.step, ws.status, ep.spin_limit);
      v = make_float4(a.x, a.y, b2.x, b2.y);
    } else if constexpr (XBF16) {
      const uint2 u = reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(xv) + size_t(t) * H +
                                                     q * kRouteSlice)[c];
      v = make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u), __uint_as_float(u.y << 16),
                      __uint_as_float(u.y & 0xFFFF0000u));
    } else {
      v = reinterpret_cast<const float4*>(static_cast<const float*>(xv) + size_t(t) * H + q * kRouteSlice)[c];
    }
    reinterpret_cast<float4*>(&s_x[t][0])[c] = v;
  }
  const int row0 = g * 32 + 2 * warp;
  float wr[2][10];  // lane holds elements 128c + 4 lane .. +3 (c = 0, 1) and 256 + 2 lane, +1 of the slice
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const __nv_bfloat16* wrow = w + size_t(row0 + r) * H + q * kRouteSlice;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint2 u = reinterpret_cast<const uint2*>(wrow)[c * 32 + lane];
      wr[r][4 * c + 0] = __uint_as_float(u.x << 16);
      wr[r][4 * c + 1] = __uint_as_float(u.x & 0xFFFF0000u);
      wr[r][4 * c + 2] = __uint_as_float(u.y << 16);
      wr[r][4 * c + 3] = __uint_as_float(u.y & 0xFFFF0000u);
    }
    const uint32_t u = reinterpret_cast<const uint32_t*>(wrow + 256)[lane];
    wr[r][8] = __uint_as_float(u << 16);
    wr[r][9] = __uint_as_float(u & 0xFFFF0000u);
  }
  __syncthreads();
  {
    float acc[2 * kMaxTok];  // [row of the pair][token]
#pragma unroll
    for (int t = 0; t < kMaxTok; ++t) {
      float a0 = 0.0f, a1 = 0.0f;
      if (t < T) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const float4 x4 = reinterpret_cast<const float4*>(&s_x[t][0])[c * 32 + lane];
          a0 = fmaf(wr[0][4 * c + 0], x4.x, a0);
          a1 = fmaf(wr[1][4 * c + 0], x4.x, a1);
          a0 = fmaf(wr[0][4 * c + 1], x4.y, a0);
          a1 = fmaf(wr[1][4 * c + 1], x4.y, a1);
          a0 = fmaf(wr[0][4 * c + 2], x4.z, a0);
          a1 = fmaf(wr[1][4 * c + 2], x4.z, a1);
          a0 = fmaf(wr[0][4 * c + 3], x4.w, a0);
          a1 = fmaf(wr[1][4 * c + 3], x4.w, a1);
        }
        const float2 x2 = reinterpret_cast<const float2*>(&s_x[t][256])[lane];
        a0 = fmaf(wr[0][8], x2.x, a0);
        a1 = fmaf(wr[1][8], x2.x, a1);
        a0 = fmaf(wr[0][9], x2.y, a0);
        a1 = fmaf(wr[1][9], x2.y, a1);
      }
      acc[t] = a0;
      acc[kMaxTok + t] = a1;
    }
    // Sum over the 32 lanes by the butterfly xor 16, 8, 4, 2, 1, halving the values a lane carries
    // at each step: 31 shuffles for the 32 (row, token) sums. Lane l ends with row l >> 4, token l & 15.
#pragma unroll
    for (int n = 16, o = 16; n >= 1; n >>= 1, o >>= 1) {
      const bool hi = (lane & o) != 0;
#pragma unroll
      for (int i = 0; i < n; ++i) {
        const float send = hi ? acc[i] : acc[i + n], keep = hi ? acc[i + n] : acc[i];
        acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
      }
    }
    s_part[2 * warp + (lane >> 4)][lane & 15] = acc[0];
  }
  cluster_sync();
  if (tid < 4 * kMaxTok) {
    const int r = 4 * q + (tid >> 4), t = tid & 15;
    if (t < T) {
      float v = 0.0f;
#pragma unroll
      for (int qq = 0; qq < kRouteSplits; ++qq) v += ld_cluster_f32(&s_part[r][t], uint32_t(qq));
      logits[size_t(t) * stride + g * 32 + r] = v;
    }
  }
  // activation quantization, one warp per ggml block, strided over every warp of the grid (spread over
  // the blocks first: a single token's ten blocks go to ten different SMs)
  {
    const int act = ep.act;
    const int per_tok = act == FB_ACT_Q8_K ? H / 256 : H / 32;
    const int n_warps = gridDim.x * 16;
    for (int task = warp * gridDim.x + blockIdx.x; task < T * per_tok; task += n_warps) {
      const int t = task / per_tok, b = task - t * per_tok;
      auto load = [&](int i) -> float {
        if constexpr (XBF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(xv)[size_t(t) * H + i]);
        else return static_cast<const float*>(xv)[size_t(t) * H + i];
      };
      uint8_t* out = ws.xq + xq_offset(act) + size_t(t) * FB_XQ_STRIDE;
      float* scales = reinterpret_cast<float*>(out + H);
      if (act == FB_ACT_Q8_K) {
        float v[8];
        if constexpr (EP) {
          const uint4* ln = x_lines + (size_t(t) * H + 256 * b + 8 * lane) / 2;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = ll_read(ln + i, ep.step, ws.status, ep.spin_limit);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = load(256 * b + 8 * lane + i);
        }
        int qv[8], ps;
        const float d = q8k_block_warp(v, qv, ps);
        store_q8k_block_planar(out, H, b, qv, ps, d);
      } else {
        unsigned short dh;
        float xv1;
        if constexpr (EP) {
          const float2 f = ll_read(x_lines + (size_t(t) * H + 32 * b + lane) / 2, ep.step, ws.status, ep.spin_limit);
          xv1 = (lane & 1) ? f.y : f.x;
        } else {
          xv1 = load(32 * b + lane);
        }
        const int qv = q8_0_block_warp(xv1, dh);
        out[32 * b + q8_0_interleave_index(lane)] = uint8_t(int8_t(qv));
        if (lane == 0) scales[b] = __half2float(__ushort_as_half(dh));
      }
    }
  }
  cluster_sync();  // no CTA of the cluster leaves while another may still read its slice sums
}

// ------------------------------------------------------------------------------ streaming skeleton
// Tiles are handed out dynamically: the producer lane of each CTA takes the next tile index from a
// device counter (reset by the select kernel), so a CTA that drew an expert with many tokens simply
// takes fewer tiles. Work items are visited heaviest first (ws.sched[8..]). An expert with more
// than kTT tokens is staged once per group of kTT tokens (its weights come back from L2). Every
// output element is still written by exactly one thread after a fixed-order reduction: results do
// not depend on which CTA or warp ran which piece.
constexpr int kSchedGateUp = 0, kSchedDown = 1, kSchedOrder = kSchedOrderBase;

// What the producer tells the consumers about the entry staged in a ring slot (shared memory).
struct StageMeta {
  int tile;        // -1: no more work
  int pair0;       // first pair (row of h / partial) of this pass
  int ntp;         // tokens in this pass (1..kTT)
  int row0;        // first intermediate row (gate/up) or output row (down) of the tile
  int item;        // work item
  int item_pair0;  // first pair of the item
  int item_tok;    // tokens of the item
  int seq;         // entry number of this CTA (the multi-stage rings check it)
  float wgt[kTT];  // routing weights of the pass's pairs (down)
};

struct Ring {
  uint64_t* full;   // [2] count 1 + tx bytes
  uint64_t* empty;  // [2]
  volatile StageMeta* meta;  // [2]
  volatile int* abort;
};

// After a wait has run out every later wait is skipped and all loops end at their next check, so
// the kernel drains quickly with the status word set; nothing ever waits without a limit.
__device__ __forceinline__ bool ring_aborted(const Ring& r) { return *r.abort != 0; }
__device__ __forceinline__ void ring_timeout(const Ring& r, uint32_t* status) {
  *r.abort = 1;
  atomicMax(status, uint32_t(FB_STATUS_PIPELINE_TIMEOUT));
}

__device__ __forceinline__ void ring_init(const Ring& r, int empty_count) {
  mbar_init(&r.full[0], 1);
  mbar_init(&r.full[1], 1);
  mbar_init(&r.empty[0], empty_count);
  mbar_init(&r.empty[1], empty_count);
  r.meta[0].tile = -1;
  r.meta[1].tile = -1;
  *r.abort = 0;
  mbar_fence_init();
}

// Producer loop of one CTA (one thread): draws tiles from `counter`, stages every pass of each
// tile through issue(meta, slot), and finally posts the end marker in both slots.
template <class IssueF>
__device__ __forceinline__ void producer_loop(const Ring& r, const fb_moe_decode_workspace& ws, const WorkCache& wc,
                                              int* counter, int n_tiles, int tiles_per_item, int rows_per_tile,
                                              IssueF issue) {
  int i = 0;
  auto slot_free = [&](int s) -> bool {
    if (ring_aborted(r)) return false;
    if (i >= 2 && !mbar_wait(&r.empty[s], ((i >> 1) - 1) & 1)) {
      ring_timeout(r, ws.status);
      return false;
    }
    return true;
  };
  int next = int(blockIdx.x);  // a block's first tile needs no ticket; later ones are drawn one step ahead of their use
  while (true) {
    const int tile = next;
    if (tile >= n_tiles) break;
    next = int(gridDim.x) + atomicAdd(counter, 1);
    const int pos = tile / tiles_per_item;
    const int item = wc.order[pos];
    const int sub = tile - pos * tiles_per_item;
    const int pb = wc.pair_begin[item];
    const int ntok = wc.pair_begin[item + 1] - pb;
    const int slot_id = wc.slot[item];
    for (int tok0 = 0; tok0 < ntok; tok0 += kTT, ++i) {
      const int s = i & 1;
      if (!slot_free(s)) return;
      volatile StageMeta* m = &r.meta[s];
      m->tile = tile;
      m->pair0 = pb + tok0;
      m->ntp = min(kTT, ntok - tok0);
      m->row0 = sub * rows_per_tile;
      m->item = item;
      m->item_pair0 = pb;
      m->item_tok = ntok;
      for (int t = 0; t < kTT; ++t) m->wgt[t] = tok0 + t < ntok ? wc.pair_weight[pb + tok0 + t] : 0.0f;
      issue(s, slot_id, sub, pb + tok0, min(kTT, ntok - tok0));
    }
  }
  for (int e = 0; e < 2; ++e, ++i) {  // end marker in both slots: every waiting warp sees it
    const int s = i & 1;
    if (!slot_free(s)) return;
    r.meta[s].tile = -1;
    mbar_arrive(&r.full[s]);
  }
}

// ------------------------------------------------------------------------------ per-format tile math
// One 36-byte IQ4_NL unit (two blocks) against TT interleaved Q8_0 rows; ublk = index of the
// unit's first block within the row.
template <int TT>
__device__ __forceinline__ void iq4nl_unit_dot(const uint32_t* unit, const Iq4nlLevels& L,
                                               const uint8_t* const (&actrow)[TT], int ublk, int act_k,
                                               float (&acc)[TT]) {
  int w[8];
  {
    const uint32_t q[4] = {ld4<2>(unit), ld4<6>(unit), ld4<10>(unit), ld4<14>(unit)};
    iq4nl_decode32(L, q, w);
    const float d = ld_fp16<0>(unit);
#pragma unroll
    for (int t = 0; t < TT; ++t) {
      const int s = dot32(w, reinterpret_cast<const int8_t*>(actrow[t]) + 32 * ublk);
      acc[t] = fmaf(float(s), d * reinterpret_cast<const float*>(actrow[t] + act_k)[ublk], acc[t]);
    }
  }
  {
    const uint32_t q[4] = {unit[5], unit[6], unit[7], unit[8]};
    iq4nl_decode32(L, q, w);
    const float d = ld_fp16<18>(unit);
#pragma unroll
    for (int t = 0; t < TT; ++t) {
      const int s = dot32(w, reinterpret_cast<const int8_t*>(actrow[t]) + 32 * (ublk + 1));
      acc[t] = fmaf(float(s), d * reinterpret_cast<const float*>(actrow[t] + act_k)[ublk + 1], acc[t]);
    }
  }
}

// One IQ4_NL block (18 bytes at row + 18 b, two-byte aligned) against TT interleaved Q8_0 rows, for
// the gate/up kernel where eight lanes share a row and lane q takes blocks q, q + 8, ...: the
// block's parity, hence its alignment, is a lane constant (`odd`), so the five aligned words that
// cover it are read directly and the four code words come out of one PRMT each. The eight lanes
// read eight consecutive 32-byte activation blocks; lanes 4-7 (`swap`) take the two 16-byte halves in
// the other order, which puts the eight 128-bit loads of an instruction in eight different bank
// groups. Integer sums do not depend on that order.
template <int TT>
__device__ __forceinline__ void iq4nl_block_dot(const uint8_t* row, int b, bool odd, bool swap, const Iq4nlLevels& L,
                                                const uint8_t* const (&actrow)[TT], int act_k, float (&acc)[TT]) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(row + 18 * b - (odd ? 2 : 0));
  const uint32_t u0 = u[0], u1 = u[1], u2 = u[2], u3 = u[3], u4 = u[4];
  const uint32_t sel = odd ? 0x7654u : 0x5432u;
  const uint32_t q[4] = {__byte_perm(u0, u1, sel), __byte_perm(u1, u2, sel), __byte_perm(u2, u3, sel),
                         __byte_perm(u3, u4, sel)};
  const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(odd ? (u0 >> 16) : (u0 & 0xFFFFu))));
  int w[8];
  iq4nl_decode32(L, q, w);
  int wa[4], wb[4];  // weights of the half read first / second
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    wa[i] = swap ? w[4 + i] : w[i];
    wb[i] = swap ? w[i] : w[4 + i];
  }
  const int off_a = 32 * b + (swap ? 16 : 0), off_b = 32 * b + (swap ? 0 : 16);
#pragma unroll
  for (int t = 0; t < TT; ++t) {
    const int4 a = *reinterpret_cast<const int4*>(actrow[t] + off_a);
    const int4 c = *reinterpret_cast<const int4*>(actrow[t] + off_b);
    int sum = __dp4a(wa[0], a.x, 0);
    sum = __dp4a(wa[1], a.y, sum);
    sum = __dp4a(wa[2], a.z, sum);
    sum = __dp4a(wa[3], a.w, sum);
    sum = __dp4a(wb[0], c.x, sum);
    sum = __dp4a(wb[1], c.y, sum);
    sum = __dp4a(wb[2], c.z, sum);
    sum = __dp4a(wb[3], c.w, sum);
    acc[t] = fmaf(float(sum), d * reinterpret_cast<const float*>(actrow[t] + act_k)[b], acc[t]);
  }
}

// h of one finished work item -> planar activation rows for the down projection (one warp).
__device__ __forceinline__ void quantize_item_h(const fb_moe_decode_workspace& ws, int pair_begin, int n_tok,
                                                int down_act, int I) {
  const int lane = threadIdx.x & 31;
  for (int p = pair_begin; p < pair_begin + n_tok; ++p) {
    const float* h = ws.h + size_t(p) * I;
    uint8_t* out = ws.hq + size_t(p) * FB_HQ_STRIDE;
    if (down_act == FB_ACT_Q8_K) {
      for (int b0 = 0; b0 < I / 256; b0 += 2) {  // two blocks' loads in flight: the finishing warp waits on this chain
        const int nb = min(2, I / 256 - b0);
        float4 a[2], c[2];
#pragma unroll
        for (int i = 0; i < 2; ++i)
          if (i < nb) {
            a[i] = __ldcg(reinterpret_cast<const float4*>(h + 256 * (b0 + i) + 8 * lane));
            c[i] = __ldcg(reinterpret_cast<const float4*>(h + 256 * (b0 + i) + 8 * lane) + 1);
          }
#pragma unroll
        for (int i = 0; i < 2; ++i)
          if (i < nb) {
            float v[8] = {a[i].x, a[i].y, a[i].z, a[i].w, c[i].x, c[i].y, c[i].z, c[i].w};
            int q[8], ps;
            const float d = q8k_block_warp(v, q, ps);
            store_q8k_block_planar(out, I, b0 + i, q, ps, d);
          }
      }
    } else {
      float* scales = reinterpret_cast<float*>(out + I);
      for (int b = 0; b < I / 32; ++b) {
        unsigned short dh;
        const int q = q8_0_block_warp(__ldcg(h + 32 * b + lane), dh);
        out[32 * b + q8_0_interleave_index(lane)] = uint8_t(int8_t(q));
        if (lane == 0) scales[b] = __half2float(__ushort_as_half(dh));
      }
    }
  }
}

// Counts one finished contribution to an item's h; the last one re-quantizes that item's h for the
// down projection and then sets kItemReady in the item's counter (a fused gate/up + down launch polls
// it before staging the item's rows). `expected` = contributions per item.
constexpr int kItemReady = 0x40000000;
__device__ __forceinline__ void item_contribution_done(const fb_moe_decode_workspace& ws, int item, int pair_begin,
                                                       int n_tok, int expected, int down_act, int inter, int lane) {
  __threadfence();
  __syncwarp();
  int ticket = 0;
  if (lane == 0) ticket = atomicAdd(&ws.item_done[item], 1);
  ticket = __shfl_sync(0xffffffffu, ticket, 0);
  if (ticket == expected - 1) {
    __threadfence();
    quantize_item_h(ws, pair_begin, n_tok, down_act, inter);
    __threadfence();
    __syncwarp();
    if (lane == 0) atomicOr(&ws.item_done[item], kItemReady);
  }
}

// Consumer side of the task scheme: draws the next (entry, task) ticket; returns false at the end.
// seq = entry number of this CTA, s = its ring slot.
template <int TASKS>
__device__ __forceinline__ bool draw_task(const Ring& r, int* ticket_ctr, uint32_t* status, int lane, int& s,
                                          int& task) {
  int ticket = 0;
  if (lane == 0) ticket = atomicAdd(ticket_ctr, 1);
  ticket = __shfl_sync(0xffffffffu, ticket, 0);
  const int seq = ticket / TASKS;
  task = ticket - seq * TASKS;
  s = seq & 1;
  if (ring_aborted(r)) return false;
  if (!mbar_wait(&r.full[s], (seq >> 1) & 1)) {
    ring_timeout(r, status);
    return false;
  }
  return r.meta[s].tile >= 0;
}

// ------------------------------------------------------------------------------ down kernel
template <int FMT, int INTER>
struct Down;
// IQ4_NL, inter 512: a row is eight 36-byte units, eight lanes per row, four rows per warp step.
template <>
struct Down<FB_FMT_IQ4_NL, 512> {
  static constexpr int kRows = 320, kRowBytes = 288, kWarps = 16, kTasks = 16, kAct = FB_ACT_Q8_0,
                       kActBytes = 512 + 64;
  static constexpr int kLanesPerRow = 8, kUnitsPerLane = 1, kUnitA = 1, kUnitB = 0;
};
// IQ4_NL, inter 640: a row is ten units, two lanes per row with five consecutive units each.
template <>
struct Down<FB_FMT_IQ4_NL, 640> {
  static constexpr int kRows = 256, kRowBytes = 360, kWarps = 16, kTasks = 16, kAct = FB_ACT_Q8_0,
                       kActBytes = 640 + 80;
  static constexpr int kLanesPerRow = 2, kUnitsPerLane = 5, kUnitA = 5, kUnitB = 1;
};

template <int FMT, int INTER>
__global__ void __launch_bounds__((Down<FMT, INTER>::kWarps + 1) * 32, 1)
down_kernel(fb_moe_expert_layout L, fb_moe_decode_workspace ws) {
  using C = Down<FMT, INTER>;
  constexpr int kW = C::kWarps, kStageW = C::kRows * C::kRowBytes;
  constexpr int kStage = kStageW + kTT * C::kActBytes;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* p = smem;
  uint8_t* stage0 = p;
  p += 2 * kStage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p);
  __shared__ StageMeta s_meta[2];
  __shared__ int s_misc[4];
  __shared__ WorkCache s_work;
  Ring ring{bars, bars + 2, s_meta, s_misc};

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    ring_init(ring, 1);  // one arrival frees a slot: the warp that finishes the entry's last task
    s_misc[1] = 0;
    s_misc[2] = 0;
    s_misc[3] = 0;
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait_prior();

  const fb_moe_decode_work* work = ws.work;
  const int n_items = min(max(work->n_items, 0), kMaxPairs);
  constexpr int tpi = H / C::kRows;
  const int n_tiles = n_items * tpi;

  if (warp == kW) {
    work_cache_fill(ws, s_work, n_items);
    __syncwarp();
    if (lane == 0) {
      producer_loop(ring, ws, s_work, ws.sched + kSchedDown, n_tiles, tpi, C::kRows,
                    [&](int s, int slot_id, int sub, int pair0, int ntp) {
                      const uint8_t* blob = L.slots + int64_t(slot_id) * L.blob_stride;
                      uint8_t* st = stage0 + s * kStage;
                      mbar_expect_tx(&ring.full[s], uint32_t(kStageW + ntp * C::kActBytes));
                      bulk_g2s(st, blob + L.down_offset + size_t(sub) * kStageW, kStageW, &ring.full[s]);
                      for (int t = 0; t < ntp; ++t)
                        bulk_g2s(st + kStageW + t * C::kActBytes, ws.hq + size_t(pair0 + t) * FB_HQ_STRIDE,
                                 C::kActBytes, &ring.full[s]);
                    });
    }
    return;
  }

  {
    const Iq4nlLevels lv = iq4nl_levels();
    while (true) {  // sixteen tasks per tile, drawn from the ticket: task k takes row steps k, k + 16, ...
      int s, task;
      if (!draw_task<C::kTasks>(ring, &s_misc[1], ws.status, lane, s, task)) break;
      const int ntp = ring.meta[s].ntp, pair0 = ring.meta[s].pair0, r0 = ring.meta[s].row0;
      const float wgt[kTT] = {ring.meta[s].wgt[0], ring.meta[s].wgt[1]};
      uint8_t* st = stage0 + s * kStage;
      const uint8_t* actbase = st + kStageW;
      constexpr int LPR = C::kLanesPerRow, RPS = 32 / LPR;
      const int q = lane % LPR, r = lane / LPR;
      for (int step = task; step < C::kRows / RPS; step += C::kTasks) {
        const int row = step * RPS + r;
        const uint8_t* rowp = st + row * C::kRowBytes;
        float acc[kTT] = {0.0f, 0.0f};
        if constexpr (INTER == 512) {
          // eight lanes per row, lane q takes blocks q and q + 8 (conflict-free weight and activation reads)
          const bool odd = (q & 1) != 0, swap = (q & 4) != 0;
          if (ntp == 1) {
            const uint8_t* ar[1] = {actbase};
            float a1[1] = {0.0f};
            iq4nl_block_dot<1>(rowp, q, odd, swap, lv, ar, INTER, a1);
            iq4nl_block_dot<1>(rowp, q + 8, odd, swap, lv, ar, INTER, a1);
            acc[0] = a1[0];
          } else {
            const uint8_t* ar[2] = {actbase, actbase + C::kActBytes};
            iq4nl_block_dot<2>(rowp, q, odd, swap, lv, ar, INTER, acc);
            iq4nl_block_dot<2>(rowp, q + 8, odd, swap, lv, ar, INTER, acc);
          }
        } else if (ntp == 1) {
          const uint8_t* ar[1] = {actbase};
          float a1[1] = {0.0f};
#pragma unroll
          for (int it = 0; it < C::kUnitsPerLane; ++it) {
            const int u = q * C::kUnitA + it * C::kUnitB;
            iq4nl_unit_dot<1>(reinterpret_cast<const uint32_t*>(rowp + 36 * u), lv, ar, 2 * u, INTER, a1);
          }
          acc[0] = a1[0];
        } else {
          const uint8_t* ar[2] = {actbase, actbase + C::kActBytes};
#pragma unroll
          for (int it = 0; it < C::kUnitsPerLane; ++it) {
            const int u = q * C::kUnitA + it * C::kUnitB;
            iq4nl_unit_dot<2>(reinterpret_cast<const uint32_t*>(rowp + 36 * u), lv, ar, 2 * u, INTER, acc);
          }
        }
#pragma unroll
        for (int t = 0; t < kTT; ++t) {
          float v = acc[t];
#pragma unroll
          for (int o = 1; o < LPR; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (t < ntp && q == 0) ws.partial[size_t(pair0 + t) * H + r0 + row] = wgt[t] * v;
        }
      }
      __syncwarp();
      int done = 0;
      if (lane == 0) done = atomicAdd(&s_misc[2 + s], 1);
      done = __shfl_sync(0xffffffffu, done, 0);
      if (done == C::kTasks - 1 && lane == 0) {
        s_misc[2 + s] = 0;
        mbar_arrive(&ring.empty[s]);
      }
    }
  }
}

#include "moe_decode_iq3s.cuh"
#define FB_MOE_DECODE_TU
#include "moe_decode_generic.cuh"

// ------------------------------------------------------------------------------ combine
// y[t][n] = partials of token t in slot order (+ y_shared); optional rank-1 ablation of the routed
// part; X[t][s][n] += inj[t][s] * y (4 residual streams) when X is given; y_out optional.
// One block per (token, 256-column slice): the projection r . y_routed needs the whole row, so
// with ablation a block first reduces the row (only then).
__global__ void __launch_bounds__(256) combine_kernel(fb_moe_decode_workspace ws, const float* __restrict__ y_shared,
                                                      const float* __restrict__ inj, float* __restrict__ X,
                                                      float* __restrict__ y_out, const float* __restrict__ ablate,
                                                      float ablate_scale) {
  pdl_launch_dependents();
  pdl_wait_prior();
  const int t = blockIdx.y;
  const fb_moe_decode_work* work = ws.work;
  const int np = min(max(work->token_pair_count[t], 0), kTopK);
  __shared__ float s_red[8];
  __shared__ float s_proj;
  float proj = 0.0f;
  if (ablate) {
    float loc = 0.0f;
    for (int n = threadIdx.x; n < H; n += 256) {
      float y = 0.0f;
      for (int k = 0; k < np; ++k) y += ws.partial[size_t(work->token_pairs[t][k]) * H + n];
      loc = fmaf(ablate[n], y, loc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) loc += __shfl_xor_sync(0xffffffffu, loc, o);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = loc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.0f;
      for (int i = 0; i < 8; ++i) s += s_red[i];
      s_proj = s;
    }
    __syncthreads();
    proj = s_proj;
  }
  const int n = blockIdx.x * 256 + threadIdx.x;
  float y = 0.0f;
  for (int k = 0; k < np; ++k) y += ws.partial[size_t(work->token_pairs[t][k]) * H + n];
  if (ablate) y -= ablate_scale * ablate[n] * proj;
  if (y_shared) y += y_shared[size_t(t) * H + n];
  if (y_out) y_out[size_t(t) * H + n] = y;
  if (X) {
#pragma unroll
    for (int s = 0; s < 4; ++s) X[(size_t(t) * 4 + s) * H + n] += inj[t * 4 + s] * y;
  }
}

// ------------------------------------------------------------------------------ expert-parallel combine
// y[r][n] = parts[0][r][n] + parts[1][r][n] + ... in rank order (deterministic).
__global__ void __launch_bounds__(256) sum_ranks_kernel(const float* __restrict__ parts, int n_ranks, int64_t elems,
                                                        float* __restrict__ y) {
  const int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= elems) return;
  float v = 0.0f;
  for (int r = 0; r < n_ranks; ++r) v += parts[int64_t(r) * elems + i];
  y[i] = v;
}

// ------------------------------------------------------------------------------ peer-memory exchange
// Expert-parallel decode without a collective library call in the step: ranks write flag-in-data
// lines (ll_store) straight into each other's buffers over NVLink and readers poll the lines they
// need in their OWN memory, a bounded number of times. No fence, no ticket, no separate flag sits
// between the data and its arrival. Buffers are double-buffered by step parity: a rank can be at
// most one step ahead of a peer (it needs that peer's partial rows to finish a step), so the lines
// of step k+2 never overwrite lines of step k that someone still reads, and a stale line (step
// k-2) never passes for a current one.
//   x_all   [2][16][1280] lines         all tokens of the step, rows written by their owners
//   y_parts [2][8][16][1280] lines      [parity][source rank][local token]: partial rows for this rank's tokens

// The combine of an expert-parallel step. Thread = (token t, two adjacent columns): token t's partial
// row over the local pairs (slot order) goes straight into its owner's y_parts; threads of tokens
// this rank owns then read the partial rows of all ranks and add them in rank order.
__global__ void __launch_bounds__(256) ep_combine_exchange_kernel(fb_moe_decode_workspace ws, fb_ep_peers peers, int tpr,
                                                                  int parity, uint32_t step, uint32_t spin_limit,
                                                                  float* __restrict__ y_local) {
  pdl_launch_dependents();
  pdl_wait_prior();
  const int t = blockIdx.y;
  const fb_moe_decode_work* work = ws.work;
  const int np = min(max(work->token_pair_count[t], 0), kTopK);
  const int c = blockIdx.x * 256 + threadIdx.x;  // line = columns 2c, 2c+1
  float y0 = 0.0f, y1 = 0.0f;
  for (int k = 0; k < np; ++k) {
    const float2 v = *reinterpret_cast<const float2*>(ws.partial + size_t(work->token_pairs[t][k]) * H + 2 * c);
    y0 += v.x;
    y1 += v.y;
  }
  const int d = t / tpr, i = t - d * tpr;
  ll_store(static_cast<uint4*>(peers.y_parts[d]) + ((size_t(parity) * kEpMaxRanks + peers.rank) * kMaxTok + i) * (H / 2) + c,
           y0, y1, step);
  if (d != peers.rank) return;
  const uint4* mine = static_cast<const uint4*>(peers.y_parts[peers.rank]);
  float a0 = 0.0f, a1 = 0.0f;
  for (int s = 0; s < peers.n_ranks; ++s) {
    const float2 v =
        ll_read(mine + ((size_t(parity) * kEpMaxRanks + s) * kMaxTok + i) * (H / 2) + c, step, ws.status, spin_limit);
    a0 += v.x;
    a1 += v.y;
  }
  *reinterpret_cast<float2*>(y_local + size_t(i) * H + 2 * c) = make_float2(a0, a1);
}

// ------------------------------------------------------------------------------ host side
template <int FMT, int INTER>
constexpr size_t down_smem() {
  using C = Down<FMT, INTER>;
  return 2 * size_t(C::kRows * C::kRowBytes + kTT * C::kActBytes) + 64;
}

bool layout_ok(const fb_moe_expert_layout* L) {
  if (!L || !L->slots) return false;
  if ((reinterpret_cast<uintptr_t>(L->slots) | uintptr_t(L->blob_stride) | uintptr_t(L->gate_offset) |
       uintptr_t(L->up_offset) | uintptr_t(L->down_offset)) & 15)
    return false;
  if (L->inter != 512 && L->inter != 640) return false;
  if (L->gate_up_format != FB_FMT_IQ3_S && L->gate_up_format != FB_FMT_IQ4_NL && !plain_gate_up(L->gate_up_format))
    return false;
  if (L->down_format == FB_FMT_IQ3_S) return L->inter % 256 == 0;
  return L->down_format == FB_FMT_IQ4_NL || L->down_format == FB_FMT_Q2_0;
}

// Polls a reader gives a peer-written exchange line before it records FB_STATUS_PIPELINE_TIMEOUT.
uint32_t g_peer_wait_polls = kPeerSpinLimit;

// A workspace made for a layout must be used with that layout; one made without (formats 0) fits all.
bool ws_fits(const fb_moe_decode_workspace* ws, const fb_moe_expert_layout* L, bool gate_up, bool down) {
  if (ws->inter && ws->inter != L->inter) return false;
  if (gate_up && ws->gate_up_format && ws->gate_up_format != L->gate_up_format) return false;
  if (down && ws->down_format && ws->down_format != L->down_format) return false;
  return true;
}

bool ws_ok(const fb_moe_decode_workspace* ws) {
  return ws && ws->work && ws->xq && ws->h && ws->hq && ws->partial && ws->item_done && ws->sched && ws->status;
}

// The streaming expert kernel of a format (IQ3_S or IQ4_NL) over the given phases.
template <int FMT>
int32_t launch_experts_fmt(const fb_moe_expert_layout* layout, const fb_moe_decode_workspace* ws, int phases,
                           void* stream, const char* what, const SelectArgs* sel) {
  using C = ExpertsCfg<FMT>;
  static PerDeviceOnce once;
  const cudaError_t attr = per_device_once(once, [] { return opt_in_smem(experts_kernel<FMT>, C::kSmem); });
  if (attr != cudaSuccess) {
    set_error("%s: shared-memory opt-in: %s", what, cudaGetErrorString(attr));
    return int32_t(attr);
  }
  const cudaError_t e = launch_pdl(experts_kernel<FMT>, dim3(sm_count()), dim3((C::kWarps + 1) * 32), C::kSmem,
                                   as_stream(stream), *layout, *ws, sel ? (phases | kPhaseSelect) : phases,
                                   sel ? *sel : SelectArgs{});
  if (e != cudaSuccess) return check_launch(what);
  return 0;
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" {

size_t fb_moe_decode_workspace_bytes(int32_t inter) {
  (void)inter;
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  return up(sizeof(fb_moe_decode_work)) + up(size_t(2 * kMaxTok) * FB_XQ_STRIDE) + up(size_t(kMaxPairs) * 640 * 4) +
         up(size_t(kMaxPairs) * FB_HQ_STRIDE) + up(size_t(kMaxPairs) * H * 4) + up(kMaxPairs * 4) +
         up(kSchedInts * 4) + 256;
}

int32_t fb_moe_decode_workspace_make(void* base, const fb_moe_expert_layout* layout, fb_moe_decode_workspace* out) {
  if (!base || !out || (reinterpret_cast<uintptr_t>(base) & 255)) return invalid("decode workspace: base must be 256-byte aligned");
  if (layout && !layout_ok(layout)) return invalid("decode workspace: unsupported expert layout");
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  uint8_t* p = static_cast<uint8_t*>(base);
  out->work = reinterpret_cast<fb_moe_decode_work*>(p);
  p += up(sizeof(fb_moe_decode_work));
  out->xq = p;
  p += up(size_t(2 * kMaxTok) * FB_XQ_STRIDE);
  out->h = reinterpret_cast<float*>(p);
  p += up(size_t(kMaxPairs) * 640 * 4);
  out->hq = p;
  p += up(size_t(kMaxPairs) * FB_HQ_STRIDE);
  out->partial = reinterpret_cast<float*>(p);
  p += up(size_t(kMaxPairs) * H * 4);
  out->item_done = reinterpret_cast<int32_t*>(p);
  p += up(kMaxPairs * 4);
  out->sched = reinterpret_cast<int32_t*>(p);
  p += up(kSchedInts * 4);
  out->status = reinterpret_cast<uint32_t*>(p);
  out->gate_up_format = layout ? layout->gate_up_format : 0;  // 0: any (the selection quantizes x both ways)
  out->down_format = layout ? layout->down_format : 0;
  out->inter = layout ? layout->inter : 0;
  out->reserved = 0;
  return 0;
}

int32_t fb_router_logits(const void* w_bf16, int32_t rows, const void* x, int32_t x_dtype, int32_t tokens,
                         float* logits, int32_t logits_stride, void* stream) {
  if (!w_bf16 || !x || !logits || rows <= 0 || tokens <= 0 || logits_stride < rows)
    return invalid("router_logits: bad arguments");
  const dim3 grid((rows + 3) / 4), block(128);
  cudaError_t e = x_dtype == FB_DT_BF16
                      ? launch_pdl(router_kernel<true>, grid, block, 0, as_stream(stream),
                                   static_cast<const __nv_bfloat16*>(w_bf16), rows, x, tokens, logits, logits_stride)
                      : launch_pdl(router_kernel<false>, grid, block, 0, as_stream(stream),
                                   static_cast<const __nv_bfloat16*>(w_bf16), rows, x, tokens, logits, logits_stride);
  if (e != cudaSuccess) return check_launch("router_logits");
  return 0;
}

int32_t fb_moe_select_publish(const float* router_logits, int32_t logits_stride, const void* x, int32_t x_dtype,
                              const int32_t* slot_of, int32_t layer, const uint32_t* seq, void* exchange,
                              int32_t tokens, const fb_moe_decode_workspace* ws, void* stream,
                              uint32_t* routing_counts) {
  (void)layer;
  (void)seq;
  if (exchange) return invalid("select_publish: no CPU expert tier exists behind these kernels; exchange must be NULL");
  if (!router_logits || !x || !ws_ok(ws) || tokens < 1 || tokens > kMaxTok || logits_stride < kExperts)
    return invalid("select_publish: bad arguments (tokens must be 1..16)");
  cudaError_t e = x_dtype == FB_DT_BF16
                      ? launch_pdl(select_kernel<true>, dim3(1 + tokens), dim3(512), 0, as_stream(stream),
                                   router_logits, logits_stride, x, slot_of, tokens, *ws, routing_counts)
                      : launch_pdl(select_kernel<false>, dim3(1 + tokens), dim3(512), 0, as_stream(stream),
                                   router_logits, logits_stride, x, slot_of, tokens, *ws, routing_counts);
  if (e != cudaSuccess) return check_launch("select_publish");
  return 0;
}

// The IQ3_S expert kernel: gate/up tiles, down tiles, or both in one launch (down needs inter 512).
static int32_t launch_experts_iq3s(const fb_moe_expert_layout* layout, const fb_moe_decode_workspace* ws, int phases,
                                   void* stream, const char* what, const SelectArgs* sel = nullptr) {
  return launch_experts_fmt<FB_FMT_IQ3_S>(layout, ws, phases, stream, what, sel);
}

// `sel`: the kernel runs the selection itself (the fused layer call), else it reads the device work list.
static int32_t launch_gate_up(const fb_moe_expert_layout* layout, const fb_moe_decode_workspace* ws, void* stream,
                              const SelectArgs* sel) {
  if (layout->gate_up_format == FB_FMT_IQ3_S)
    return launch_experts_iq3s(layout, ws, kPhaseGateUp, stream, "hot_gate_up", sel);
  if (plain_gate_up(layout->gate_up_format)) {  // plain kernels: they read the device work list (sel is not for them)
    const dim3 pgrid(sm_count() * 8);
    cudaError_t pe;
    if (layout->gate_up_format == FB_FMT_IQ3_XXS)
      pe = launch_pdl(gate_up_generic_kernel<FB_FMT_IQ3_XXS>, pgrid, dim3(256), 0, as_stream(stream), *layout, *ws);
    else if (layout->gate_up_format == FB_FMT_IQ2_S)
      pe = launch_pdl(gate_up_generic_kernel<FB_FMT_IQ2_S>, pgrid, dim3(256), 0, as_stream(stream), *layout, *ws);
    else
      pe = launch_pdl(gate_up_generic_kernel<FB_FMT_IQ4_XS>, pgrid, dim3(256), 0, as_stream(stream), *layout, *ws);
    if (pe == cudaSuccess)  // the down projection wants h re-quantized: one warp per pair
      pe = launch_pdl(requant_h_kernel, dim3(kMaxPairs / 8), dim3(256), 0, as_stream(stream), *layout, *ws);
    if (pe != cudaSuccess) return check_launch("hot_gate_up");
    return 0;
  }
  if (layout->gate_up_format == FB_FMT_IQ4_NL)
    return launch_experts_fmt<FB_FMT_IQ4_NL>(layout, ws, kPhaseGateUp, stream, "hot_gate_up", sel);
  return invalid("hot_gate_up: unsupported gate/up format");
}

int32_t fb_moe_hot_gate_up(const fb_moe_expert_layout* layout, int32_t tokens, const fb_moe_decode_workspace* ws,
                           void* stream) {
  if (!layout_ok(layout) || !ws_ok(ws) || tokens < 1 || tokens > kMaxTok) return invalid("hot_gate_up: bad arguments");
  if (!ws_fits(ws, layout, true, true))
    return invalid("hot_gate_up: workspace was made for a different layout");
  return launch_gate_up(layout, ws, stream, nullptr);
}

static int32_t launch_down(const fb_moe_expert_layout* layout, const fb_moe_decode_workspace* ws, void* stream);

// Both projections of every routed expert: one launch for IQ3_S experts, a gate/up and a down launch otherwise.
static int32_t launch_experts(const fb_moe_expert_layout* layout, const fb_moe_decode_workspace* ws, void* stream,
                              const SelectArgs* sel) {
  if (layout->gate_up_format == FB_FMT_IQ3_S && layout->down_format == FB_FMT_IQ3_S)
    return launch_experts_iq3s(layout, ws, kPhaseGateUp | kPhaseDown, stream, "hot_experts", sel);
  if (layout->gate_up_format == FB_FMT_IQ4_NL && layout->down_format == FB_FMT_IQ4_NL && layout->inter == 512)
    return launch_experts_fmt<FB_FMT_IQ4_NL>(layout, ws, kPhaseGateUp | kPhaseDown, stream, "hot_experts", sel);
  const int32_t st = launch_gate_up(layout, ws, stream, sel);
  return st ? st : launch_down(layout, ws, stream);
}


int32_t fb_moe_hot_experts(const fb_moe_expert_layout* layout, int32_t tokens, const fb_moe_decode_workspace* ws,
                           void* stream) {
  if (!layout_ok(layout) || !ws_ok(ws) || tokens < 1 || tokens > kMaxTok) return invalid("hot_experts: bad arguments");
  if (!ws_fits(ws, layout, true, true))
    return invalid("hot_experts: workspace was made for a different layout");
  return launch_experts(layout, ws, stream, nullptr);
}

static int32_t launch_down(const fb_moe_expert_layout* layout, const fb_moe_decode_workspace* ws, void* stream) {
  if (layout->down_format == FB_FMT_IQ3_S) return launch_experts_iq3s(layout, ws, kPhaseDown, stream, "hot_down");
  if (layout->down_format == FB_FMT_Q2_0) {
    if (launch_pdl(down_q2_0_kernel, dim3(sm_count() * 8), dim3(256), 0, as_stream(stream), *layout, *ws) != cudaSuccess)
      return check_launch("hot_down");
    return 0;
  }
  if (layout->inter == 512) return launch_experts_fmt<FB_FMT_IQ4_NL>(layout, ws, kPhaseDown, stream, "hot_down", nullptr);
  static PerDeviceOnce once;
  const cudaError_t attr = per_device_once(once, [] {
    cudaError_t a = opt_in_smem(down_kernel<FB_FMT_IQ4_NL, 512>, down_smem<FB_FMT_IQ4_NL, 512>());
    if (a == cudaSuccess) a = opt_in_smem(down_kernel<FB_FMT_IQ4_NL, 640>, down_smem<FB_FMT_IQ4_NL, 640>());
    return a;
  });
  if (attr != cudaSuccess) {
    set_error("hot_down: shared-memory opt-in: %s", cudaGetErrorString(attr));
    return int32_t(attr);
  }
  const dim3 grid(sm_count());
  cudaError_t e;
  if (layout->inter == 512)
    e = launch_pdl(down_kernel<FB_FMT_IQ4_NL, 512>, grid, dim3((Down<FB_FMT_IQ4_NL, 512>::kWarps + 1) * 32),
                   down_smem<FB_FMT_IQ4_NL, 512>(), as_stream(stream), *layout, *ws);
  else
    e = launch_pdl(down_kernel<FB_FMT_IQ4_NL, 640>, grid, dim3((Down<FB_FMT_IQ4_NL, 640>::kWarps + 1) * 32),
                   down_smem<FB_FMT_IQ4_NL, 640>(), as_stream(stream), *layout, *ws);
  if (e != cudaSuccess) return check_launch("hot_down");
  return 0;
}

int32_t fb_moe_hot_down(const fb_moe_expert_layout* layout, int32_t tokens, const fb_moe_decode_workspace* ws,
                        void* stream) {
  if (!layout_ok(layout) || !ws_ok(ws) || tokens < 1 || tokens > kMaxTok) return invalid("hot_down: bad arguments");
  if (!ws_fits(ws, layout, false, true))
    return invalid("hot_down: workspace was made for a different layout");
  return launch_down(layout, ws, stream);
}

int32_t fb_moe_combine(const fb_moe_decode_workspace* ws, const float* y_shared, void* exchange, int32_t layer,
                       const uint32_t* seq, const float* inj, float* X, float* y_out, int32_t tokens,
                       long long timeout_cycles, const float* ablate_direction, float ablate_scale, void* stream) {
  (void)layer;
  (void)seq;
  (void)timeout_cycles;
  if (exchange) return invalid("combine: no CPU expert tier exists behind these kernels; exchange must be NULL");
  if (!ws_ok(ws) || tokens < 1 || tokens > kMaxTok || (X && !inj) || (!X && !y_out))
    return invalid("combine: bad arguments");
  cudaError_t e = launch_pdl(combine_kernel, dim3(H / 256, tokens), dim3(256), 0, as_stream(stream), *ws, y_shared, inj,
                             X, y_out, ablate_direction, ablate_scale);
  if (e != cudaSuccess) return check_launch("combine");
  return 0;
}

static int32_t layer_decode_impl(const void* router_w_bf16, const fb_moe_expert_layout* layout,
                                 const int32_t* slot_of, bool remote_ok, const void* x, int32_t x_dtype,
                                 int32_t tokens, const fb_moe_decode_workspace* ws, float* logits_scratch, float* y_out,
                                 void* stream, const EpRouteArgs* ep = nullptr) {
  const bool with_combine = ep == nullptr;
  EpRouteArgs era{};
  if (ep) era = *ep;
  era.act = layout_ok(layout) ? act_of(layout->gate_up_format) : FB_ACT_Q8_K;
  // Three launches for IQ3_S experts (four otherwise): route (router projection + activation quantization),
  // the expert kernel (every CTA runs the selection on the stored logits, then gate/up and down tiles in
  // one persistent launch; the other formats take a gate/up and a down launch), combine. The expert
  // arithmetic is that of the separate entry points. The route kernel sums a logit as eight K slices of
  // 320 added in slice order, where fb_router_logits sums 80 values per lane and then the lanes: the two
  // projections agree to fp32 rounding (a few ulp), not bit for bit, so a near-tie between the tenth and
  // eleventh expert may resolve differently. Only rows 0..511 of logits_scratch are written: row 512
  // (the shared-expert gate) is not produced here.
  if (!router_w_bf16 || !x || (!y_out && with_combine) || !logits_scratch || !layout_ok(layout) || !ws_ok(ws) ||
      tokens < 1 || tokens > kMaxTok)
    return invalid("layer_decode: bad arguments (tokens must be 1..16, logits scratch [tokens][513] required)");
  if (!ws_fits(ws, layout, true, true))
    return invalid("layer_decode: workspace was made for a different layout");
  const dim3 grid(kRouteBlocks), block(512);
  auto launch = [&](auto kernel) {
    return launch_pdl_cluster(kernel, grid, block, 0, as_stream(stream), unsigned(kRouteSplits),
                              static_cast<const __nv_bfloat16*>(router_w_bf16), x, tokens, logits_scratch,
                              int(FB_ROUTER_ROWS), *ws, era);
  };
  cudaError_t e = ep                       ? launch(route_kernel<false, true>)
                  : x_dtype == FB_DT_BF16 ? launch(route_kernel<true, false>)
                                          : launch(route_kernel<false, false>);
  if (e != cudaSuccess) return check_launch("layer_decode: route");
  const SelectArgs sel{logits_scratch, int(FB_ROUTER_ROWS), slot_of, tokens, remote_ok ? 1 : 0};
  int32_t st;
  if (plain_gate_up(layout->gate_up_format)) {  // no streaming kernel to select inside: one more launch
    if (launch_pdl(select_only_kernel, dim3(1), dim3(512), 0, as_stream(stream), sel, *ws) != cudaSuccess)
      return check_launch("layer_decode: select");
    st = launch_experts(layout, ws, stream, nullptr);
  } else {
    st = launch_experts(layout, ws, stream, &sel);  // selection + both projections of every routed expert
  }
  if (st || !with_combine) return st;
  return fb_moe_combine(ws, nullptr, nullptr, 0, nullptr, nullptr, nullptr, y_out, tokens, 0, nullptr, 0.0f, stream);
}

int32_t fb_moe_layer_decode(const void* router_w_bf16, const fb_moe_expert_layout* layout, const void* x,
                            int32_t x_dtype, int32_t tokens, const fb_moe_decode_workspace* ws, float* logits_scratch,
                            float* y_out, void* stream) {
  return layer_decode_impl(router_w_bf16, layout, nullptr, false, x, x_dtype, tokens, ws, logits_scratch, y_out,
                           stream);
}

int32_t fb_moe_layer_decode_ep(const void* router_w_bf16, const fb_moe_expert_layout* layout,
                               const int32_t* slot_of, const void* x, int32_t x_dtype, int32_t tokens,
                               const fb_moe_decode_workspace* ws, float* logits_scratch, float* y_partial,
                               void* stream) {
  if (!slot_of) return invalid("layer_decode_ep: slot_of (expert -> local slot, -1 = another rank) is required");
  return layer_decode_impl(router_w_bf16, layout, slot_of, true, x, x_dtype, tokens, ws, logits_scratch, y_partial,
                           stream);
}

int32_t fb_moe_layer_decode_ep_p2p(const void* router_w_bf16, const fb_moe_expert_layout* layout,
                                   const int32_t* slot_of, const float* x_local, int32_t tokens,
                                   const fb_ep_peers* peers, uint32_t step, const fb_moe_decode_workspace* ws,
                                   float* logits_scratch, float* y_local, void* stream) {
  if (!slot_of || !x_local || !y_local || !peers || peers->n_ranks < 1 || peers->n_ranks > kEpMaxRanks ||
      peers->rank < 0 || peers->rank >= peers->n_ranks || tokens < peers->n_ranks || tokens > kMaxTok ||
      tokens % peers->n_ranks || step == 0)
    return invalid("layer_decode_ep_p2p: bad arguments (tokens a multiple of the rank count, at most 16; step >= 1)");
  // the route kernel hands its blocks out to the ranks in equal shares
  if (kRouteBlocks % peers->n_ranks)
    return invalid("layer_decode_ep_p2p: the rank count must be 1, 2, 4 or 8");
  for (int d = 0; d < peers->n_ranks; ++d)
    if (!peers->x_all[d] || !peers->y_parts[d])
      return invalid("layer_decode_ep_p2p: a peer buffer address is missing");
  const int R = peers->n_ranks, tpr = tokens / R, parity = int(step & 1u);
  cudaStream_t s = as_stream(stream);
  // Four launches, chained like the single-GPU layer: route (publishes this rank's rows, waits for
  // everyone's), gate/up, down, combine (sends partial rows, waits, sums).
  EpRouteArgs era{};
  era.peers = *peers;
  era.x_local = x_local;
  era.tpr = tpr;
  era.parity = parity;
  era.step = step;
  era.spin_limit = g_peer_wait_polls;
  // (the route kernel reads every x row through the exchange lines; x_local only satisfies the argument check)
  int32_t st = layer_decode_impl(router_w_bf16, layout, slot_of, true, x_local, FB_DT_F32, tokens, ws, logits_scratch,
                                 nullptr, stream, &era);
  if (st) return st;
  const cudaError_t e = launch_pdl(ep_combine_exchange_kernel, dim3(H / 512, tokens), dim3(256), 0, s, *ws, *peers, tpr,
                                   parity, step, g_peer_wait_polls, y_local);
  if (e != cudaSuccess) return check_launch("layer_decode_ep_p2p: combine");
  return check_launch("layer_decode_ep_p2p");
}

// Exchange buffers of fb_moe_layer_decode_ep_p2p. They are allocated here (cudaMalloc, so a CUDA IPC
// handle names exactly the buffer) and opened by the peers in the context of THEIR OWN device with
// lazy peer access, the way collective libraries map each other's memory.
constexpr size_t kEpBytes[2] = {size_t(2) * kMaxTok * (H / 2) * 16, size_t(2) * kEpMaxRanks * kMaxTok * (H / 2) * 16};

int32_t fb_ep_exchange_create(void** x_all, void** y_parts, uint8_t* handles) {
  if (!x_all || !y_parts || !handles) return invalid("ep_exchange_create: NULL argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == FB_EP_HANDLE_BYTES, "handle size");
  void** out[2] = {x_all, y_parts};
  for (int k = 0; k < 2; ++k) {
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, kEpBytes[k]);
    if (e == cudaSuccess) e = cudaMemset(p, 0, kEpBytes[k]);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
      cudaGetLastError();
      set_error("ep_exchange_create: %s", cudaGetErrorString(e));
      return int32_t(e);
    }
    memcpy(handles + k * FB_EP_HANDLE_BYTES, &h, FB_EP_HANDLE_BYTES);
    *out[k] = p;
  }
  return int32_t(cudaDeviceSynchronize());
}

int32_t fb_ep_exchange_open(const uint8_t* handles, void** x_all, void** y_parts) {
  if (!x_all || !y_parts || !handles) return invalid("ep_exchange_open: NULL argument");
  void** out[2] = {x_all, y_parts};
  for (int k = 0; k < 2; ++k) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + k * FB_EP_HANDLE_BYTES, FB_EP_HANDLE_BYTES);
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      set_error("ep_exchange_open: %s", cudaGetErrorString(e));
      return int32_t(e);
    }
    *out[k] = p;
  }
  return 0;
}

int32_t fb_ep_exchange_close(void* x_all, void* y_parts, int32_t own) {
  void* p[2] = {x_all, y_parts};
  int32_t st = 0;
  for (int k = 0; k < 2; ++k) {
    if (!p[k]) continue;
    const cudaError_t e = own ? cudaFree(p[k]) : cudaIpcCloseMemHandle(p[k]);
    if (e != cudaSuccess) {
      cudaGetLastError();
      st = int32_t(e);
    }
  }
  return st;
}

void fb_ep_set_wait_limit(uint32_t polls) { g_peer_wait_polls = polls ? polls : kPeerSpinLimit; }

size_t fb_ep_exchange_bytes(int32_t which) { return which == 0 ? kEpBytes[0] : which == 1 ? kEpBytes[1] : 0; }

int32_t fb_ep_sum_ranks(const float* parts, int32_t n_ranks, int32_t rows, float* y, void* stream) {
  if (!parts || !y || n_ranks < 1 || rows < 1) return invalid("ep_sum_ranks: bad arguments");
  const int64_t elems = int64_t(rows) * H;
  sum_ranks_kernel<<<unsigned((elems + 255) / 256), 256, 0, as_stream(stream)>>>(parts, n_ranks, elems, y);
  return check_launch("ep_sum_ranks");
}

int32_t fb_moe_layer_decode_host(const void* router_w_bf16, const fb_moe_expert_layout* layout, const void* x_host,
                                 int32_t x_dtype, int32_t tokens, const fb_moe_decode_workspace* ws,
                                 float* logits_scratch, void* x_dev, float* y_dev, float* y_host, void* stream) {
  if (!x_host || !x_dev || !y_dev || !y_host || tokens < 1 || tokens > kMaxTok)
    return invalid("layer_decode_host: bad arguments");
  const size_t xb = size_t(tokens) * H * (x_dtype == FB_DT_BF16 ? 2 : 4);
  cudaError_t e = cudaMemcpyAsync(x_dev, x_host, xb, cudaMemcpyHostToDevice, as_stream(stream));
  if (e != cudaSuccess) return check_launch("layer_decode_host: copy in");
  // A pinned result buffer is written by the combine kernel itself (page-locked host memory has a device address
  // under unified addressing): one copy operation and its launch less per call. Pageable memory takes the copy.
  cudaPointerAttributes pa{};
  const bool direct = cudaPointerGetAttributes(&pa, y_host) == cudaSuccess && pa.type == cudaMemoryTypeHost &&
                      pa.devicePointer != nullptr;
  if (!direct) (void)cudaGetLastError();  // (an unregistered pointer reports an error on older drivers: not ours to keep)
  float* y_target = direct ? static_cast<float*>(pa.devicePointer) : y_dev;
  int32_t st = fb_moe_layer_decode(router_w_bf16, layout, x_dev, x_dtype, tokens, ws, logits_scratch, y_target, stream);
  if (st) return st;
  if (!direct) {
    e = cudaMemcpyAsync(y_host, y_dev, size_t(tokens) * H * 4, cudaMemcpyDeviceToHost, as_stream(stream));
    if (e != cudaSuccess) return check_launch("layer_decode_host: copy out");
  }
  e = cudaStreamSynchronize(as_stream(stream));
  if (e != cudaSuccess) {
    set_error("layer_decode_host: %s", cudaGetErrorString(e));
    return int32_t(e);
  }
  return 0;
}


// ---------------------------------------------------------------------------------------------
// fb_moe_layer_decode_static: the whole decode layer without any caller-provided scratch.
//
// Some hosts of this library may not allocate device memory at the point where they run a layer:
// an engine whose memory plan is frozen after start-up (every byte of HBM already handed to
// weights and KV cache), a plug-in that is only given tensor pointers, or code running where a
// cudaMalloc would serialize the device. For them the layer's scratch - work list, quantized
// activations, h, partial sums, router logits - lives in one array inside the library image.
// Every GPU that loads the library carries these kStaticScratchBytes until the process exits.
//
// The array's name is only a host-side handle; its device address comes from
// cudaGetSymbolAddress, taken once per device on that device's first call (so make that first
// call outside any stream capture). All calls on a device share the array and it keeps the last
// call's contents: the entry point clears the one word that must start at zero, and two calls
// that overlap on the same GPU (different streams) race on it - serialize them.
// fb_moe_layer_decode_static_status reads the status word of the last call back to the host (a
// stream-ordered copy out of the array and a wait on that stream; it allocates nothing either).
namespace {
constexpr size_t kStaticWorkspaceBytes = 2304 * 1024;  // >= fb_moe_decode_workspace_bytes(640), checked at set-up
constexpr size_t kStaticLogitsBytes = size_t(FB_DECODE_MAX_TOKENS) * FB_ROUTER_ROWS * 4;
constexpr size_t kStaticScratchBytes = kStaticWorkspaceBytes + ((kStaticLogitsBytes + 255) & ~size_t(255));
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticScratch {
  bool ready = false;
  unsigned char* base = nullptr;
  uint32_t* status = nullptr;  // the workspace's status word inside the array (set by the first layer call)
};
StaticScratch g_static[64];
}  // namespace

int32_t fb_moe_layer_decode_static(const void* router_w_bf16, const fb_moe_expert_layout* layout, const void* x,
                                   int32_t x_dtype, int32_t tokens, float* y_out, void* stream) {
  if (tokens < 1 || tokens > kMaxTok)
    return invalid("layer_decode_static: tokens must be 1..%d (the static scratch is sized for that)", kMaxTok);
  if (!layout_ok(layout)) return invalid("layer_decode_static: unsupported expert layout");
  if (fb_moe_decode_workspace_bytes(layout->inter) > kStaticWorkspaceBytes)
    return invalid("layer_decode_static: layout needs more scratch than the %zu static bytes", kStaticWorkspaceBytes);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("layer_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    return e != cudaSuccess ? int32_t(e) : int32_t(cudaErrorInvalidDevice);
  }
  StaticScratch& sc = g_static[dev];
  if (!sc.ready) {  // first call on this device: resolve the array's device address
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      set_error("layer_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return e != cudaSuccess ? int32_t(e) : int32_t(cudaErrorInvalidSymbol);
    }
    sc.base = static_cast<unsigned char*>(p);
    sc.ready = true;
  }
  fb_moe_decode_workspace ws;
  int32_t st = fb_moe_decode_workspace_make(sc.base, layout, &ws);
  if (st) return st;
  sc.status = ws.status;
  float* logits = reinterpret_cast<float*>(sc.base + kStaticWorkspaceBytes);
  // the sticky status word and the scheduler words (tile counters, route tickets) are the only state a call inherits
  e = cudaMemsetAsync(ws.status, 0, sizeof(uint32_t), as_stream(stream));
  if (e == cudaSuccess) e = cudaMemsetAsync(ws.sched, 0, kSchedInts * sizeof(int32_t), as_stream(stream));
  if (e != cudaSuccess) {
    set_error("layer_decode_static: clearing scratch state: %s", cudaGetErrorString(e));
    return int32_t(e);
  }
  return fb_moe_layer_decode(router_w_bf16, layout, x, x_dtype, tokens, &ws, logits, y_out, stream);
}

int32_t fb_moe_layer_decode_static_status(uint32_t* status_host, void* stream) {
  if (!status_host) return invalid("layer_decode_static_status: status_host is NULL");
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64 || !g_static[dev].status)
    return invalid("layer_decode_static_status: fb_moe_layer_decode_static has not run on this device");
  e = cudaMemcpyAsync(status_host, g_static[dev].status, sizeof(uint32_t), cudaMemcpyDeviceToHost, as_stream(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(as_stream(stream));
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error("layer_decode_static_status: %s", cudaGetErrorString(e));
    return int32_t(e);
  }
  return 0;
}

}  // extern "C"
