/* fngine_b200 -- C ABI of the B200 (sm_100a) quantized-expert kernels.
 *
 * Every entry point replaces one function of the reference engine's kernel interface for the
 * routed-expert MoE path and the FP8-row dense projection; the comment above each declaration
 * names the reference declaration it stands in for (paths relative to the reference project).
 * The reference exposes these as C++ free functions (namespace fngine::kernels); the translation unit
 * fngine_b200/binding/fngine_kernels_b200.cpp defines those C++ names on top of this ABI.
 *
 * Conventions (same as the reference, src/kernels/moe/moe.h:19-24, src/kernels/linear/linear.h:46-47):
 *  - all tensor arguments are raw device pointers owned by the caller; kernels never allocate and
 *    never synchronize; everything is ordered on the `stream` argument (a cudaStream_t passed as
 *    void*); `tokens` is a host value.
 *  - return value: 0 on success, otherwise a cudaError_t value (cudaErrorInvalidValue = 1 for bad
 *    arguments). fb_last_error_string() describes the last failure on the calling thread.
 *  - there is no CPU fallback: without a CUDA device every compute entry point fails.
 *
 * Differences from the reference interface, all additive:
 *  - `inter` (expert intermediate size) is a run-time field (512 or 640), the reference fixes 640
 *    at compile time (src/core/model_dims.h:60);
 *  - IQ3_S is accepted as a down-projection format (needs inter % 256 == 0);
 *  - activations follow the reference's CPU tier: Q8_K blocks for IQ3_S weights, Q8_0 blocks for
 *    IQ4_NL weights (src/cpu/iq_cpu.h:12-21), not the GPU tier's per-32 fp32-scale variant;
 *  - there is no CPU expert tier behind these kernels: `exchange`/`control` must be NULL and every
 *    routed expert must be resident (slot_of[e] >= 0), which the reference API already permits
 *    (src/kernels/moe/moe.h:119-121, :198-200).
 */
#ifndef FNGINE_B200_H
#define FNGINE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids of the expert formats (src/kernels/moe/moe.h:48-55). IQ3_S and IQ4_NL have the streaming
 * decode kernels and the prefill kernels; IQ3_XXS, IQ2_S and IQ4_XS (gate/up) and Q2_0 (down) run at decode
 * width through plain, untuned kernels (no prefill path). */
enum { FB_FMT_IQ3_XXS = 18, FB_FMT_IQ4_NL = 20, FB_FMT_IQ3_S = 21, FB_FMT_IQ2_S = 22, FB_FMT_IQ4_XS = 23, FB_FMT_Q2_0 = 42 };
/* element types of activation inputs */
enum { FB_DT_F32 = 0, FB_DT_BF16 = 1 };
/* activation block formats (src/cpu/iq_cpu.h:44) */
enum { FB_ACT_Q8_K = 0, FB_ACT_Q8_0 = 1 };

enum {
  FB_HIDDEN = 2560,           /* src/core/model_dims.h:9 */
  FB_EXPERTS = 512,           /* :58 */
  FB_TOPK = 10,               /* :59 */
  FB_ROUTER_ROWS = 513,       /* :62 router | shared-expert gate */
  FB_DECODE_MAX_TOKENS = 16,  /* src/kernels/moe/moe.h:81 */
  FB_DECODE_MAX_PAIRS = 160   /* :82 */
};

/* Device-side status word values written by kernels whose bounded waits ran out. */
enum { FB_STATUS_OK = 0, FB_STATUS_PIPELINE_TIMEOUT = 1, FB_STATUS_BAD_WORK = 2 };

const char* fb_last_error_string(void);
/* Library/ABI version and the SM architecture the kernels were compiled for (100). */
int32_t fb_abi_version(void);
int32_t fb_compiled_sm(void);

/* ---------------------------------------------------------------- formats and layout */
/* moe_row_bytes, src/kernels/moe/moe.h:58 (src/kernels/moe/moe_format.cpp:5-15). 0 if unsupported. */
int64_t fb_moe_row_bytes(int32_t format, int32_t k);
/* Activation block format a weight format pairs with (format_info().act, src/cpu/iq_cpu.cpp:467-478). */
int32_t fb_moe_act_format(int32_t format);
/* Bytes of one activation row of k values in ggml layout (act_row_bytes, src/cpu/iq_cpu.h:66). */
int64_t fb_act_row_bytes(int32_t act_format, int32_t k);

/* MoeExpertLayout, src/kernels/moe/moe.h:62-71, plus the run-time `inter`. */
typedef struct fb_moe_expert_layout {
  const uint8_t* slots; /* device base of the layer's slot array */
  int64_t blob_stride;  /* bytes between consecutive slots (multiple of 16) */
  int64_t gate_offset;  /* byte offsets of gate / up / down inside a blob (multiples of 16) */
  int64_t up_offset;
  int64_t down_offset;
  int32_t gate_up_format;
  int32_t down_format;
  int32_t inter; /* 512 or 640 */
  int32_t reserved;
} fb_moe_expert_layout;

/* make_moe_expert_layout, src/kernels/moe/moe.h:75-76: gate | up | down packed back to back. */
int32_t fb_moe_expert_layout_make(const uint8_t* slots, int64_t blob_stride, int32_t gate_up_format,
                                  int32_t down_format, int32_t inter, fb_moe_expert_layout* out);
/* Bytes of one packed blob for these formats (gate + up + down). */
int64_t fb_moe_blob_bytes(int32_t gate_up_format, int32_t down_format, int32_t inter);

/* ---------------------------------------------------------------- decode (T <= 16) */
/* MoeDecodeWork, src/kernels/moe/moe.h:91-105 (same fields, same meaning; every pair is hot). */
typedef struct fb_moe_decode_work {
  int32_t n_items;
  int32_t n_pairs;
  int32_t n_cold;
  int32_t tokens;
  int32_t item_slot[FB_DECODE_MAX_PAIRS];
  int32_t item_pair_begin[FB_DECODE_MAX_PAIRS + 1];
  int32_t pair_token[FB_DECODE_MAX_PAIRS];
  float pair_weight[FB_DECODE_MAX_PAIRS];
  int32_t token_pair_count[FB_DECODE_MAX_TOKENS];
  int32_t token_pairs[FB_DECODE_MAX_TOKENS][FB_TOPK];
  int32_t token_cold_count[FB_DECODE_MAX_TOKENS];
  int32_t topk_expert[FB_DECODE_MAX_TOKENS][FB_TOPK];
  float topk_weight[FB_DECODE_MAX_TOKENS][FB_TOPK];
} fb_moe_decode_work;

/* MoeDecodeWorkspace, src/kernels/moe/moe.h:108-115. Activations are kept in a planar form of
 * the ggml blocks the CPU tier uses (Q8_K for IQ3_S weights, Q8_0 for IQ4_NL): per row the int8
 * codes first, then the block scales as fp32 (Q8_0 scales are the fp16-rounded values widened;
 * Q8_0 codes are stored per block in the order 2*(e%16) + e/16 that the IQ4_NL nibble decode
 * produces). `hq` is h re-quantized for the down projection, `item_done` counts finished gate/up
 * tiles per work item, `sched` holds the dynamic tile counters ([0] gate/up, [1] down) and from
 * [8] on the work items ordered by token count (heaviest first), `status` is one device word set
 * when a bounded wait runs out. */
typedef struct fb_moe_decode_workspace {
  fb_moe_decode_work* work;
  uint8_t* xq;        /* [2][16][FB_XQ_STRIDE]: Q8_K rows, then Q8_0 rows */
  float* h;           /* [160 pairs][inter] fp32 silu(g)*u */
  uint8_t* hq;        /* [160 pairs][FB_HQ_STRIDE] */
  float* partial;     /* [160 pairs][2560], routing weight applied */
  int32_t* item_done; /* [160] */
  int32_t* sched;     /* [8 + 160] */
  uint32_t* status;   /* FB_STATUS_* */
  int32_t gate_up_format;
  int32_t down_format;
  int32_t inter;
  int32_t reserved;
} fb_moe_decode_workspace;
enum { FB_XQ_STRIDE = 2880, FB_HQ_STRIDE = 720 };

/* moe_decode_workspace_bytes / make_moe_decode_workspace, src/kernels/moe/moe.h:116-117.
 * `base` is 256-byte aligned device memory of at least the returned size, zero-filled once. The carve
 * depends on `base` only (`work` is the first region). `layout` may be NULL, as the reference's
 * make_moe_decode_workspace(base) has none: the workspace then fits every supported layout, and
 * fb_moe_select_publish, which does not see the layout either, quantizes x for both activation
 * formats (Q8_K and Q8_0) instead of the one the layout's gate/up format needs. */
size_t fb_moe_decode_workspace_bytes(int32_t inter);
int32_t fb_moe_decode_workspace_make(void* base, const fb_moe_expert_layout* layout,
                                     fb_moe_decode_workspace* out);

/* Router projection feeding the selection: logits[t][r] = sum_k W[r][k] * x[t][k], W bf16
 * [rows][2560], fp32 accumulation, fp32 out with row stride `logits_stride` (linear_bf16 with the
 * (513, 2560) StoreF32 registry entry, src/kernels/linear/linear.h:20,170-172). */
int32_t fb_router_logits(const void* w_bf16, int32_t rows, const void* x, int32_t x_dtype, int32_t tokens,
                         float* logits, int32_t logits_stride, void* stream);

/* moe_select_publish, src/kernels/moe/moe.h:127-131. Router top-10 (ties to the lower id),
 * renormalised softmax weights, sorted work list, and the once-per-token activation quantization
 * of x (dtype FB_DT_F32 or FB_DT_BF16, [tokens][2560]). `slot_of` may be NULL (slot == expert).
 * `exchange` must be NULL. `routing_counts` optional device u32[512]. */
int32_t fb_moe_select_publish(const float* router_logits, int32_t logits_stride, const void* x, int32_t x_dtype,
                              const int32_t* slot_of, int32_t layer, const uint32_t* seq, void* exchange,
                              int32_t tokens, const fb_moe_decode_workspace* ws, void* stream,
                              uint32_t* routing_counts);
/* moe_hot_gate_up, src/kernels/moe/moe.h:136-137: h[pair][j] = silu(gate_j . x) * (up_j . x). */
int32_t fb_moe_hot_gate_up(const fb_moe_expert_layout* layout, int32_t tokens, const fb_moe_decode_workspace* ws,
                           void* stream);
/* moe_hot_down, src/kernels/moe/moe.h:141-142: partial[pair][n] = w_pair * (down_n . q8(h[pair])). */
int32_t fb_moe_hot_down(const fb_moe_expert_layout* layout, int32_t tokens, const fb_moe_decode_workspace* ws,
                        void* stream);
/* moe_hot_gate_up followed by moe_hot_down as ONE launch where the formats allow it (IQ3_S gate/up and
 * down: a persistent kernel streams all gate/up tiles and then all down tiles through one pipeline, an
 * expert's down tiles waiting for its re-quantized h); otherwise the two launches. Same results as the
 * two calls, bit for bit. No counterpart in the reference as a single function. */
int32_t fb_moe_hot_experts(const fb_moe_expert_layout* layout, int32_t tokens, const fb_moe_decode_workspace* ws,
                           void* stream);
/* moe_combine, src/kernels/moe/moe.h:154-158: y[t] = sum of token t's partials in slot order
 * + y_shared[t] (optional); X[t][s][d] += inj[t][s] * y[t][d] when X is given; y_out optional.
 * `exchange` must be NULL (no CPU tier), so timeout_cycles is unused; the rank-1 ablation of the
 * routed part is applied when ablate_direction is given. */
int32_t fb_moe_combine(const fb_moe_decode_workspace* ws, const float* y_shared, void* exchange, int32_t layer,
                       const uint32_t* seq, const float* inj, float* X, float* y_out, int32_t tokens,
                       long long timeout_cycles, const float* ablate_direction, float ablate_scale, void* stream);

/* One whole decode MoE layer: router projection -> select -> gate/up -> down -> combine, the call
 * sequence of Forward::moe's decode branch (src/model/forward.cpp:333,358-375) without the shared
 * expert. x: device [tokens][2560]; y_out: device fp32 [tokens][2560]. No reference counterpart
 * as a single function. logits_scratch is fp32 [tokens][513]; only columns 0..511 are written (the
 * shared-expert gate, row 512 of a 513-row router, is not projected here). The fused router
 * projection adds a logit's products in a different order than fb_router_logits: the two agree to
 * fp32 rounding, not bit for bit. */
int32_t fb_moe_layer_decode(const void* router_w_bf16, const fb_moe_expert_layout* layout, const void* x,
                            int32_t x_dtype, int32_t tokens, const fb_moe_decode_workspace* ws, float* logits_scratch,
                            float* y_out, void* stream);
/* Same with HOST x and y: copies x in, runs the layer, copies y back and waits for it. `x_dev`
 * ([tokens][2560] of x_dtype) and `y_dev` (fp32) are caller-owned device staging buffers. */
int32_t fb_moe_layer_decode_host(const void* router_w_bf16, const fb_moe_expert_layout* layout, const void* x_host,
                                 int32_t x_dtype, int32_t tokens, const fb_moe_decode_workspace* ws,
                                 float* logits_scratch, void* x_dev, float* y_dev, float* y_host, void* stream);

/* ---------------------------------------------------------------- prefill (eager, T up to the workspace capacity)
 * MoePrefillWorkspace, src/kernels/moe/moe.h:167-184. Differences: the work list holds the units
 * of both grouped GEMMs ({expert, first weight row of a 128-row tile, first pair, tokens}, up to 256
 * tokens per unit) instead of 64-token tiles; the per-pair results go to `yp` (fp32, routing weight
 * applied) and the combine adds a token's ten rows in ascending-expert order, which replaces the
 * reference's 64-bit fixed-point atomics (moe.h:186-192) as the mechanism that makes the prefill sum
 * independent of scheduling; `token_pair` maps (token, rank) to its pair. */
typedef struct fb_moe_prefill_workspace {
  int32_t capacity;
  int32_t inter;
  int32_t max_units_gate_up;
  int32_t max_units_down;
  int32_t* meta;          /* [0] gate/up units [1] down units [2] pairs */
  int32_t* expert_count;  /* [512] */
  int32_t* expert_offset; /* [513] */
  int32_t* expert_cursor; /* [512] */
  int32_t* topk_expert;   /* [capacity][10] */
  float* topk_weight;     /* [capacity][10] */
  int32_t* pair_token;    /* [capacity*10] pairs grouped by expert */
  float* pair_weight;     /* [capacity*10] */
  int32_t* token_pair;    /* [capacity][10] */
  void* units_gate_up;    /* int4 [max_units_gate_up] */
  void* units_down;       /* int4 [max_units_down] */
  void* h;                /* bf16 [capacity*10 + 256][inter] */
  float* yp;              /* [capacity*10][2560] */
  uint32_t* status;       /* FB_STATUS_* */
} fb_moe_prefill_workspace;

/* moe_prefill_workspace_bytes / make_moe_prefill_workspace, src/kernels/moe/moe.h:193-194. */
size_t fb_moe_prefill_workspace_bytes(int32_t capacity, int32_t inter);
int32_t fb_moe_prefill_workspace_make(void* base, int32_t capacity, int32_t inter, fb_moe_prefill_workspace* out);
/* moe_route, src/kernels/moe/moe.h:201-204: top-10 for `tokens` tokens, per-expert pair lists, unit
 * lists. `control` must be NULL (no CPU tier); x and expert_blob are accepted for signature parity
 * and not read (every expert is resident). */
int32_t fb_moe_route(const float* router_logits, int32_t logits_stride, const void* x, const uint8_t* const* expert_blob,
                     int32_t layer, const uint32_t* seq, void* control, int32_t tokens,
                     const fb_moe_prefill_workspace* ws, void* stream);
/* moe_grouped_gate_up, src/kernels/moe/moe.h:209-211: h[pair] = bf16(silu(gate . x) * (up . x)), x bf16
 * [tokens][2560]. `expert_blob` is the device table of blob addresses ([512]) or NULL to address
 * expert e at layout->slots + e * blob_stride. */
int32_t fb_moe_grouped_gate_up(const fb_moe_expert_layout* layout, const uint8_t* const* expert_blob, const void* x_bf16,
                               int32_t tokens, const fb_moe_prefill_workspace* ws, void* stream);
/* moe_grouped_down, src/kernels/moe/moe.h:213-214: yp[pair] = w_pair * (down . h[pair]). */
int32_t fb_moe_grouped_down(const fb_moe_expert_layout* layout, const uint8_t* const* expert_blob, int32_t tokens,
                            const fb_moe_prefill_workspace* ws, void* stream);
/* moe_prefill_combine, src/kernels/moe/moe.h:221-226: y[t] = sum of token t's pair rows (ascending
 * expert id) + y_shared[t]; X[t][s] += inj[t][s] * y[t]; y_out optional. `control` must be NULL; the
 * rank-1 ablation is not built for this path (ablate_direction must be NULL). */
int32_t fb_moe_prefill_combine(const fb_moe_prefill_workspace* ws, const float* y_shared, void* control, int32_t layer,
                               const uint32_t* seq, const float* inj, float* X, float* y_out, int32_t tokens,
                               long long timeout_cycles, const float* ablate_direction, float ablate_scale,
                               void* stream);

/* ---------------------------------------------------------------- expert parallel (no reference counterpart)
 * The reference is single-GPU. Here the 512 experts of a layer are sharded over the ranks of one
 * node; a rank's slot array holds only its own experts and `slot_of[e]` is the local slot of expert
 * e or -1 when another rank owns it (the role the reference gives to "cold" experts,
 * src/kernels/moe/moe.h:119-121). */
/* Prefill, expert parallel. The owner of a token sends its bf16 row once to every rank that holds
 * at least one of the token's ten experts, together with the token's (expert, weight) lists;
 * fb_moe_topk makes those lists on the owner (the same top-10 rule as fb_moe_route), fb_moe_route_ep
 * builds the receiving rank's pair and unit lists from them, keeping only experts in
 * [expert_lo, expert_hi) (the others take no part: their pairs are skipped by the grouped kernels
 * and by fb_moe_prefill_combine, whose output is then the partial sum over this rank's experts, in
 * ascending expert order). `expert_blob` of the grouped kernels must be the [512] table of blob
 * addresses indexed by GLOBAL expert id. fb_ep_scatter_sum adds, on the owner, the partial rows the
 * ranks returned: y[t] = sum over d in rank order of recv[row_of[t][d]] (row_of < 0: rank d holds none
 * of the token's experts). */
int32_t fb_moe_topk(const float* router_logits, int32_t logits_stride, int32_t tokens, int32_t* topk_expert,
                    float* topk_weight, void* stream);
int32_t fb_moe_route_ep(const int32_t* topk_expert, const float* topk_weight, int32_t expert_lo, int32_t expert_hi,
                        int32_t rows, const fb_moe_prefill_workspace* ws, void* stream);
int32_t fb_ep_scatter_sum(const float* recv, const int32_t* row_of, int32_t n_ranks, int32_t tokens, float* y,
                          void* stream);
/* How fb_moe_grouped_down hands its results to fb_moe_prefill_combine. fixed_point != 0: the reference's scheme
 * (src/kernels/moe/moe.h:186-192): every addend w * (down . h) is rounded once to 2^-32 fixed point and added to
 * a 64-bit per-token sum with integer atomics: exact, independent of the order, no per-pair buffer. 0: fp32 rows
 * per pair, added by the combine in ascending expert order. Process-wide; set it before a layer's route call. */
int32_t fb_moe_prefill_set_accumulation(int32_t fixed_point);
/* fb_moe_route_ep for a placement that is not contiguous and may hold several copies of a hot expert
 * (the cross-GPU counterpart of the reference's routing-EMA expert placement, src/model/routing_counts.h:
 * there the hottest experts move to the GPU, here they are spread, and the very hottest copied, so that the
 * ranks get equal shares of the pairs). share [512]: -1 = this rank does not hold the expert; otherwise
 * (n << 8) | i, 0 <= i < n <= 255: this rank holds copy i of n and takes the pairs of rows r with
 * r % n == i. Rows are numbered as they are passed in, so the n copies split an expert's pairs without
 * overlap only when every rank is given the same rows in the same order (the dense exchange). */
int32_t fb_moe_route_placed(const int32_t* topk_expert, const float* topk_weight, const int32_t* share, int32_t rows,
                            const fb_moe_prefill_workspace* ws, void* stream);
/* One decode layer over this rank's experts: x holds ALL tokens of the step (after dispatch),
 * y_partial[t] = sum over token t's LOCAL experts, in slot order; pairs of other ranks are skipped
 * and counted in the work list's n_cold. */
int32_t fb_moe_layer_decode_ep(const void* router_w_bf16, const fb_moe_expert_layout* layout,
                               const int32_t* slot_of, const void* x, int32_t x_dtype, int32_t tokens,
                               const fb_moe_decode_workspace* ws, float* logits_scratch, float* y_partial,
                               void* stream);
/* The same step with the exchange done by the kernels themselves over peer-mapped memory (NVLink
 * stores, no collective library call): every rank owns tokens / n_ranks consecutive tokens.
 * x_all[d] and y_parts[d] are the addresses, valid in THIS process, of rank d's two exchange buffers
 * (entry `rank` is this rank's own memory). Data travels as 16-byte lines {value, step, value, step}
 * written by one store each, so a reader that finds the current step number in both flag words has
 * the values: there is no fence and no separate flag. A step: the route kernel writes the rank's x
 * rows into every rank's x_all and reads all rows of the step from its own x_all, polling lines
 * that have not arrived yet; the layer runs over the local experts; the combine writes every
 * token's partial row into its owner's y_parts, and the owner adds the n_ranks partial rows in rank
 * order into y_local [tokens / n_ranks][2560]. `step` must be 1, 2, 3, ... in call order and equal
 * on all ranks; polls are bounded (about a second, see fb_ep_set_wait_limit) and end with
 * FB_STATUS_PIPELINE_TIMEOUT in the workspace status word. The rank count must be 1, 2, 4 or 8.
 * x_local is fp32.
 * Set-up (not part of a step): fb_ep_exchange_create allocates and zero-fills this rank's two
 * buffers on the current device (fb_ep_exchange_bytes(0 / 1) bytes) and writes their CUDA IPC
 * handles (2 x 64 bytes) to `handles`; the ranks trade the handle bytes through any channel and
 * fb_ep_exchange_open maps a peer's buffers into the context of the current device (lazy peer
 * access). fb_ep_exchange_close unmaps a peer's buffers (own = 0) or frees this rank's (own = 1). */
#define FB_EP_HANDLE_BYTES 64
#define FB_EP_MAX_RANKS 8
typedef struct fb_ep_peers {
  int32_t rank;
  int32_t n_ranks;
  void* x_all[FB_EP_MAX_RANKS];
  void* y_parts[FB_EP_MAX_RANKS];
} fb_ep_peers;
size_t fb_ep_exchange_bytes(int32_t which);
/* Polls a reader spends on one awaited exchange line before it gives up, records
 * FB_STATUS_PIPELINE_TIMEOUT and lets the step drain (0 restores the default of 2^20, about a second).
 * A host setting read at launch time; the reference's counterpart is the timeout_cycles argument of
 * its exchange waits (src/kernels/moe/moe.h:154-158, src/core/exchange.h:46-57). */
void fb_ep_set_wait_limit(uint32_t polls);
int32_t fb_ep_exchange_create(void** x_all, void** y_parts, uint8_t* handles);
int32_t fb_ep_exchange_open(const uint8_t* handles, void** x_all, void** y_parts);
int32_t fb_ep_exchange_close(void* x_all, void* y_parts, int32_t own);
int32_t fb_moe_layer_decode_ep_p2p(const void* router_w_bf16, const fb_moe_expert_layout* layout,
                                   const int32_t* slot_of, const float* x_local, int32_t tokens,
                                   const fb_ep_peers* peers, uint32_t step, const fb_moe_decode_workspace* ws,
                                   float* logits_scratch, float* y_local, void* stream);
/* Combine on the owning rank: y[r] = parts[0][r] + parts[1][r] + ... (rank order), rows x 2560 fp32. */
int32_t fb_ep_sum_ranks(const float* parts, int32_t n_ranks, int32_t rows, float* y, void* stream);
/* One expert-parallel prefill layer with the dense exchange, the whole step behind one call (no reference
 * counterpart: the reference is single-GPU). Every rank owns `tokens_local` consecutive tokens (the same count
 * on every rank) and a shard of the experts. The call enqueues on `stream`: fb_moe_topk of the rank's tokens;
 * an all-gather of the bf16 rows and of the (expert, weight) lists; fb_moe_route_placed (share != NULL: the
 * rank's [512] share table) or fb_moe_route_ep over [expert_lo, expert_hi) on all tokens_local * n_ranks rows;
 * the grouped gate/up and down GEMMs and the per-row sums over this rank's experts; then the combine:
 * FB_EP_COMBINE_ALL_TO_ALL returns each owner the n_ranks partial rows of its tokens and adds them in rank
 * order (fb_ep_sum_ranks; results are those of the single-GPU layer up to the parentheses of the fp32 sum),
 * FB_EP_COMBINE_REDUCE_SCATTER lets the collective library add them on the way (one summed row per token
 * arrives; the order of the additions is the library's). y_local: fp32 [tokens_local][2560].
 * `comm` is an ncclComm_t of exactly n_ranks ranks whose rank r owns tokens [r * tokens_local, (r + 1) *
 * tokens_local); the collective library is looked up in the process at the first call, not linked; with
 * n_ranks == 1 nothing of it is touched and comm may be NULL. `expert_blob` is the device table of blob
 * addresses by GLOBAL expert id (fb_moe_grouped_gate_up). `ws` must hold tokens_local * n_ranks rows;
 * `scratch` is caller-owned device memory of fb_ep_prefill_scratch_bytes() bytes, 256-byte aligned. Nothing is
 * allocated and nothing is read back on the host: the call may sit inside a longer stream of work. */
enum { FB_EP_COMBINE_ALL_TO_ALL = 0, FB_EP_COMBINE_REDUCE_SCATTER = 1 };
size_t fb_ep_prefill_scratch_bytes(int32_t tokens_local, int32_t n_ranks, int32_t combine);
int32_t fb_ep_prefill_layer(const fb_moe_expert_layout* layout, const uint8_t* const* expert_blob, const int32_t* share,
                            int32_t expert_lo, int32_t expert_hi, const float* router_logits, int32_t logits_stride,
                            const void* x_bf16, int32_t tokens_local, int32_t n_ranks, int32_t combine,
                            const fb_moe_prefill_workspace* ws, void* scratch, float* y_local, void* comm,
                            void* stream);

/* The decode layer for callers that may not allocate: no workspace, no logits scratch. This entry
 * point has no counterpart in the reference (whose kernels always take a caller workspace). It is
 * for hosts that cannot call cudaMalloc where they run a layer - a frozen memory plan, a plug-in
 * handed only tensor pointers - so the scratch sits in a static device array inside the library
 * (about 2.3 MB held by every GPU that loads it, until the process exits). Limit: tokens <= 16 and
 * the layouts fb_moe_layer_decode accepts; larger requests are refused with an error. The first
 * call on a device looks up the array's device address, so issue it before any stream capture.
 * All calls on a GPU share the array: calls that overlap on that GPU race, keep them in one
 * stream (or otherwise ordered). x and y_out are the caller's device buffers as above. */
int32_t fb_moe_layer_decode_static(const void* router_w_bf16, const fb_moe_expert_layout* layout, const void* x,
                                   int32_t x_dtype, int32_t tokens, float* y_out, void* stream);
/* The device status word (FB_STATUS_*) the last fb_moe_layer_decode_static call on the current GPU
 * left in the static array, copied to *status_host: the workspace of that entry point is hidden, so
 * this is how its caller learns that a bounded wait ran out (FB_STATUS_PIPELINE_TIMEOUT) or that
 * the work list was unusable (FB_STATUS_BAD_WORK). It enqueues one 4-byte copy on `stream` and waits
 * for that stream; it allocates nothing. No counterpart in the reference. */
int32_t fb_moe_layer_decode_static_status(uint32_t* status_host, void* stream);

/* ---------------------------------------------------------------- FP8-row dense projection
 * Fp8RowWeight + linear_fp8, src/kernels/linear/linear.h:57-62, :116-139:
 *   out = epilogue((x[t] . W[n]) * scale[n]), W = E4M3FN codes [n][k] (16-byte aligned) with one scale
 * per row, fp32 (FB_DT_F32) or bf16 (FB_DT_BF16, the reference's pack format). x is bf16 [tokens][k].
 * Epilogues (LinearEpilogue / LinearEpilogueParams, linear.h:64-103):
 *   FB_EPI_STORE_BF16    out bf16 [T][n]
 *   FB_EPI_STORE_F32     out fp32 [T][n]
 *   FB_EPI_GR_WRITE      out = X fp32 [T][4][n], X[t][s][r] += inj[t][s] * acc[t][r]   (inj fp32 [T][4])
 *   FB_EPI_SWIGLU        out = h bf16 [T][n/2], h[t][j] = silu(acc[t][j]) * acc[t][n/2 + j]
 *   FB_EPI_SHARED_SCALE  out = y fp32 [T][n], y[t][r] = sigmoid(gate_logit[t * gate_stride]) * acc[t][r]
 * (SiluQuarter and GrMix belong to the residual-stream mixer and are not provided.)
 * Paths (Fp8LinearPath, linear.h:116-120):
 *   FB_FP8_PATH_AUTO / FB_FP8_PATH_A16  exact activations, the reference's default at every T
 *     (src/kernels/linear/fp8/fp8_shapes.h:39-43). T <= 16 runs fb_linear_fp8_decode. Above, each token
 *     is scaled by a power of two and written into the workspace as the sum of two E4M3 numbers
 *     (hi = rne(x), lo = x - hi: a bf16 value has eight significant bits, four fit each piece), and the
 *     tcgen05 E4M3 x E4M3 GEMM adds both products into one fp32 accumulator in tensor memory: the
 *     numerics of the reference's bf16-activation GEMM (elements below 2^-9 of their row's maximum
 *     lose bits under 2^-17 of that maximum) without widening the weights.
 *   FB_FP8_PATH_A8  one E4M3 code per activation with a per-token fp32 scale max|x|/448
 *     (linear.h:32-37): half the tensor-core work, 1-4 % rms output noise; only on request.
 * Shapes: T > 16 needs n % 64 == 0 (n % 128 for SwiGlu), k % 128 == 0; T <= 16 as fb_linear_fp8_decode.
 * The reference's closed registry (linear_fp8.cpp:19-24) is not enforced. Every output element is written
 * once, by one thread, after the complete K reduction, in an order fixed by the shape: repeated calls
 * are bitwise identical (linear.h:39-44). Bad arguments return cudaErrorInvalidValue where the
 * reference throws std::invalid_argument (linear_fp8.cpp:83-95). */
enum { FB_EPI_STORE_BF16 = 0, FB_EPI_STORE_F32 = 1, FB_EPI_GR_WRITE = 2, FB_EPI_SWIGLU = 3, FB_EPI_SHARED_SCALE = 4 };
enum { FB_FP8_PATH_AUTO = 0, FB_FP8_PATH_A16 = 1, FB_FP8_PATH_A8 = 2 };
typedef struct fb_linear_epilogue {
  int32_t kind;            /* FB_EPI_* */
  int32_t gate_stride;     /* SharedScale */
  void* out;
  const float* inj;        /* GrWrite */
  const float* gate_logit; /* SharedScale */
} fb_linear_epilogue;
/* linear_fp8_workspace_bytes, src/kernels/linear/linear.h:132: enough for any T in [1, max_tokens] on
 * any path (two activation pieces [2][T][k] + token scales, or the decode-width scratch). */
size_t fb_linear_fp8_workspace_bytes(int32_t n, int32_t k, int32_t max_tokens);
/* linear_fp8, src/kernels/linear/linear.h:137-139. `workspace` is 256-byte aligned. */
int32_t fb_linear_fp8(const void* x_bf16, int32_t tokens, const uint8_t* w_codes, const void* w_scales,
                      int32_t w_scales_dtype, int32_t n, int32_t k, const fb_linear_epilogue* epilogue,
                      void* workspace, size_t workspace_bytes, void* stream, int32_t path);
/* The A8 activation quantizer alone (fp8_a8_quantize_kernel, src/kernels/linear/fp8/fp8_a8.cu:22-69):
 * codes [tokens][k], scales [tokens]; bit-identical to the host statement in
 * tests/kernels/linear/linear_ref.h:99-107 of the reference. */
int32_t fb_fp8_quantize_tokens(const void* x_bf16, int32_t tokens, int32_t k, uint8_t* codes, float* scales,
                               void* stream);
/* The two-piece split of the exact route alone (no reference counterpart; a parity probe):
 * scales[t] = 2^(floor(log2 max|x[t]|) - 7), codes_hi = rne_e4m3(x / scale),
 * codes_lo = rne_e4m3(x / scale - hi). */
int32_t fb_fp8_split_tokens(const void* x_bf16, int32_t tokens, int32_t k, uint8_t* codes_hi, uint8_t* codes_lo,
                            float* scales, void* stream);

/* linear_fp8 at decode width, the reference's "A16" path for T <= 16 (src/kernels/linear/linear.h:27-31,
 * :137-139; fp8/fp8_gemv.cuh, fp8/fp8_a16_ksplit_mma.cuh): bf16 activations are kept exactly (three
 * E5M2 pieces per value), E4M3 weights are used exactly, fp32 accumulation, one multiplication by the
 * row scale, then the epilogue. tokens 1..16, k % 128 == 0, n % 8 == 0 (n % 16 for SwiGlu). */
size_t fb_linear_fp8_decode_workspace_bytes(int32_t n, int32_t k);
int32_t fb_linear_fp8_decode(const void* x_bf16, int32_t tokens, const uint8_t* w_codes, const void* w_scales,
                             int32_t w_scales_dtype, int32_t n, int32_t k, const fb_linear_epilogue* epilogue,
                             void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------- parity probes (no reference counterpart)
 * The same device routines the GEMV kernels use, exposed so that dequantized weights and int8
 * activations can be compared bit for bit with the CPU reference. */
/* out[r][0..k) = exact fp32 dequantization of row r (dequantize_row_iq3_s / _iq4_nl,
 * third_party/ggml-iq/ggml-iq.c:231-288). */
int32_t fb_dequant_rows(int32_t format, const uint8_t* rows, int64_t row_bytes, int32_t nrows, int32_t k,
                        float* out, void* stream);
/* ggml activation blocks of `rows` rows of k values (quantize_row_q8_K_ref / quantize_row_q8_0_ref,
 * third_party/ggml-iq/ggml-iq.c:313-350, :75-98; all-zero Q8_K blocks get zero bsums as in
 * src/cpu/q8_cpu.h:7-8). */
int32_t fb_quantize_act(int32_t act_format, const void* x, int32_t x_dtype, int32_t rows, int32_t k, uint8_t* out,
                        void* stream);

/* Seeded synthetic expert bytes, generated on the device and reproducible on the host with
 * integer arithmetic only (see fngine_b200/synth.py): block b of the tensor takes its free bytes
 * from splitmix64(seed, counter) and its fp16 scale from `d_table[65536]` (device). */
int32_t fb_synth_fill_blocks(int32_t format, uint8_t* dst, int64_t n_blocks, int64_t first_block, uint64_t seed,
                             const uint16_t* d_table, void* stream);
/* The same stream written for `n_experts` consecutive experts in ONE launch: expert first_expert + s
 * takes blocks [(first_expert + s) * blocks_per_expert, ...) and lands at dst + s * expert_stride
 * (dst = the slot array base plus the matrix offset inside a blob). */
int32_t fb_synth_fill_experts(int32_t format, uint8_t* dst, int64_t expert_stride, int32_t n_experts,
                              int32_t first_expert, int64_t blocks_per_expert, uint64_t seed, const uint16_t* d_table,
                              void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FNGINE_B200_H */
