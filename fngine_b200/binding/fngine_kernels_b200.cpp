// Binding of the reference engine's kernel interface to libfngine_b200.so.
//
// One translation unit for the reference's build: it DEFINES the functions that
// src/kernels/moe/moe.h and src/kernels/linear/linear.h of the reference declare for the
// routed-expert path and the FP8-row projection, on top of the C ABI in include/fngine_b200.h, so that
// model::Forward::moe / Forward::dense (src/model/forward.cpp:316-379, :166-176) compile unchanged.
// It replaces src/kernels/moe/{moe_format.cpp, moe_decode.cu, moe_prefill.cu, moe_grouped_gemm.cu} and
// the definitions of linear_fp8 / linear_fp8_workspace_bytes in src/kernels/linear/linear_fp8.cpp.
// The reference's headers are used as they are; nothing in them changes.
//
// Compile: g++ -std=c++20 -I <reference>/src -I <cuda>/include -I <this repository>/include ...
// Link:    libfngine_b200.so
//
// What differs from the stock kernels (all stated in include/fngine_b200.h):
//  * there is no CPU expert tier behind these kernels (a 180 GB part keeps every expert resident):
//    exchange / control must be null and view.header must be null, cold pairs are not allowed;
//  * supported expert formats: IQ3_S and IQ4_NL gate/up, IQ4_NL down (and IQ3_S down at inter 512);
//  * decode activations follow the reference's CPU tier (Q8_K / Q8_0 blocks, src/cpu/iq_cpu.h:12-21);
//  * the workspace structs keep their reference fields, but the bytes behind them are laid out by this
//    library: sizes come from moe_decode_workspace_bytes() / moe_prefill_workspace_bytes() below and the
//    library's own view of a workspace is re-derived from its first pointer on every call (host
//    arithmetic only).
#include "kernels/linear/linear.h"
#include "kernels/moe/moe.h"

#include <fngine_b200.h>

#include <stdexcept>
#include <string>

namespace fngine::kernels {

namespace {

fb_moe_expert_layout to_fb(const MoeExpertLayout& l) {
  fb_moe_expert_layout f{};
  f.slots = l.slots;
  f.blob_stride = l.blob_stride;
  f.gate_offset = l.gate_offset;
  f.up_offset = l.up_offset;
  f.down_offset = l.down_offset;
  f.gate_up_format = static_cast<int32_t>(l.gate_up_format);
  f.down_format = static_cast<int32_t>(l.down_format);
  f.inter = dims::kExpertInter;
  return f;
}

// The library's view of a decode workspace made by make_moe_decode_workspace: `work` is the first
// region, i.e. the base address. A null layout leaves the formats open (the selection then
// quantizes x for both activation formats).
fb_moe_decode_workspace to_fb(const MoeDecodeWorkspace& ws, const fb_moe_expert_layout* layout) {
  fb_moe_decode_workspace f{};
  fb_moe_decode_workspace_make(ws.work, layout, &f);
  return f;
}

fb_moe_prefill_workspace to_fb(const MoePrefillWorkspace& ws) {
  fb_moe_prefill_workspace f{};
  fb_moe_prefill_workspace_make(ws.meta, ws.capacity, dims::kExpertInter, &f);  // `meta` is the first region
  return f;
}

cudaError_t status(int32_t st) { return static_cast<cudaError_t>(st); }

fb_linear_epilogue to_fb(const LinearEpilogueParams& e) {
  fb_linear_epilogue f{};
  f.kind = static_cast<int32_t>(e.kind);  // StoreBf16 .. SharedScale have the values of FB_EPI_*
  f.gate_stride = e.gate_stride;
  f.out = e.out;
  f.inj = e.inj;
  f.gate_logit = e.gate_logit;
  return f;
}

}  // namespace

// ---------------------------------------------------------------------------------- formats
int64_t moe_row_bytes(MoeFormat f, int32_t k) { return fb_moe_row_bytes(static_cast<int32_t>(f), k); }

// (decode width: all of the reference's formats; the prefill kernels exist for IQ3_S and IQ4_NL only and return
// cudaErrorInvalidValue for a layer in another format)
bool moe_gate_up_format_supported(MoeFormat f) {
  return f == MoeFormat::IQ2_S || f == MoeFormat::IQ3_XXS || f == MoeFormat::IQ3_S || f == MoeFormat::IQ4_XS ||
         f == MoeFormat::IQ4_NL;
}
bool moe_down_format_supported(MoeFormat f) { return f == MoeFormat::IQ4_NL || f == MoeFormat::Q2_0; }

MoeExpertLayout make_moe_expert_layout(const uint8_t* slots, int64_t blob_stride, MoeFormat gate_up_format,
                                       MoeFormat down_format) {
  fb_moe_expert_layout f{};
  if (fb_moe_expert_layout_make(slots, blob_stride, static_cast<int32_t>(gate_up_format),
                                static_cast<int32_t>(down_format), dims::kExpertInter, &f))
    throw std::invalid_argument(std::string("make_moe_expert_layout: ") + fb_last_error_string());
  MoeExpertLayout l;
  l.slots = f.slots;
  l.blob_stride = f.blob_stride;
  l.gate_offset = f.gate_offset;
  l.up_offset = f.up_offset;
  l.down_offset = f.down_offset;
  l.gate_up_format = gate_up_format;
  l.down_format = down_format;
  return l;
}

// ---------------------------------------------------------------------------------- decode
static_assert(sizeof(MoeDecodeWork) == sizeof(fb_moe_decode_work), "the work list has the reference's fields");

std::size_t moe_decode_workspace_bytes() { return fb_moe_decode_workspace_bytes(dims::kExpertInter); }

MoeDecodeWorkspace make_moe_decode_workspace(void* base) {
  fb_moe_decode_workspace f{};
  if (fb_moe_decode_workspace_make(base, nullptr, &f))
    throw std::invalid_argument(std::string("make_moe_decode_workspace: ") + fb_last_error_string());
  MoeDecodeWorkspace ws;
  ws.work = reinterpret_cast<MoeDecodeWork*>(f.work);
  ws.xq = reinterpret_cast<int8_t*>(f.xq);
  ws.xd = nullptr;  // block scales live inside the planar activation rows
  ws.h = f.h;
  ws.partial = f.partial;
  ws.relay = f.status;  // no CPU-tier relay exists; this is the device status word (FB_STATUS_*)
  return ws;
}

cudaError_t moe_select_publish(const float* router_logits, const __nv_bfloat16* x, const int32_t* slot_of,
                               int32_t layer, const uint32_t* seq, DecodeExchange* exchange, int32_t tokens,
                               const MoeDecodeWorkspace& ws, cudaStream_t stream, uint32_t* routing_counts) {
  const fb_moe_decode_workspace f = to_fb(ws, nullptr);
  return status(fb_moe_select_publish(router_logits, dims::kRouterRows, x, FB_DT_BF16, slot_of, layer, seq, exchange,
                                      tokens, &f, stream, routing_counts));
}

cudaError_t moe_hot_gate_up(const MoeExpertLayout& layout, int32_t tokens, const MoeDecodeWorkspace& ws,
                            cudaStream_t stream) {
  const fb_moe_expert_layout l = to_fb(layout);
  const fb_moe_decode_workspace f = to_fb(ws, nullptr);
  return status(fb_moe_hot_gate_up(&l, tokens, &f, stream));
}

cudaError_t moe_hot_down(const MoeExpertLayout& layout, int32_t tokens, const MoeDecodeWorkspace& ws,
                         cudaStream_t stream) {
  const fb_moe_expert_layout l = to_fb(layout);
  const fb_moe_decode_workspace f = to_fb(ws, nullptr);
  return status(fb_moe_hot_down(&l, tokens, &f, stream));
}

cudaError_t moe_combine(const MoeDecodeWorkspace& ws, const float* y_shared, DecodeExchange* exchange, int32_t layer,
                        const uint32_t* seq, const float* inj, float* X, float* y_out, int32_t tokens,
                        long long timeout_cycles, const float* ablate_direction, float ablate_scale,
                        cudaStream_t stream) {
  const fb_moe_decode_workspace f = to_fb(ws, nullptr);
  return status(fb_moe_combine(&f, y_shared, exchange, layer, seq, inj, X, y_out, tokens, timeout_cycles,
                               ablate_direction, ablate_scale, stream));
}

// ---------------------------------------------------------------------------------- prefill
std::size_t moe_prefill_workspace_bytes(int32_t capacity) {
  return fb_moe_prefill_workspace_bytes(capacity, dims::kExpertInter);
}

MoePrefillWorkspace make_moe_prefill_workspace(void* base, int32_t capacity) {
  fb_moe_prefill_workspace f{};
  if (fb_moe_prefill_workspace_make(base, capacity, dims::kExpertInter, &f))
    throw std::invalid_argument(std::string("make_moe_prefill_workspace: ") + fb_last_error_string());
  MoePrefillWorkspace ws;
  ws.capacity = capacity;
  ws.max_tiles = f.max_units_gate_up;
  ws.meta = f.meta;
  ws.expert_count = f.expert_count;
  ws.expert_offset = f.expert_offset;
  ws.expert_cursor = f.expert_cursor;
  ws.topk_expert = f.topk_expert;
  ws.topk_weight = f.topk_weight;
  ws.pair_token = f.pair_token;
  ws.pair_weight = f.pair_weight;
  ws.h = static_cast<__nv_bfloat16*>(f.h);
  ws.relay = f.status;
  // token_cold, row_of_token, tiles and y_fixed have no counterpart: every expert is resident, the work
  // list is the library's unit list and the per-token sum is formed in a fixed order without atomics
  return ws;
}

cudaError_t moe_route(const float* router_logits, const __nv_bfloat16* x, const uint8_t* const* expert_blob,
                      int32_t layer, const uint32_t* seq, ExchangeControl* control, const PrefillExchangeView& view,
                      int32_t tokens, const MoePrefillWorkspace& ws, cudaStream_t stream) {
  if (control || view.header) return cudaErrorInvalidValue;  // no CPU tier to publish cold rows to
  const fb_moe_prefill_workspace f = to_fb(ws);
  return status(fb_moe_route(router_logits, dims::kRouterRows, x, expert_blob, layer, seq, nullptr, tokens, &f, stream));
}

cudaError_t moe_grouped_gate_up(const MoeExpertLayout& layout, const uint8_t* const* expert_blob,
                                const __nv_bfloat16* x, int32_t tokens, const MoePrefillWorkspace& ws,
                                cudaStream_t stream) {
  const fb_moe_expert_layout l = to_fb(layout);
  const fb_moe_prefill_workspace f = to_fb(ws);
  return status(fb_moe_grouped_gate_up(&l, expert_blob, x, tokens, &f, stream));
}

cudaError_t moe_grouped_down(const MoeExpertLayout& layout, const uint8_t* const* expert_blob, int32_t tokens,
                             const MoePrefillWorkspace& ws, cudaStream_t stream) {
  const fb_moe_expert_layout l = to_fb(layout);
  const fb_moe_prefill_workspace f = to_fb(ws);
  return status(fb_moe_grouped_down(&l, expert_blob, tokens, &f, stream));
}

cudaError_t moe_prefill_combine(const MoePrefillWorkspace& ws, const float* y_shared, ExchangeControl* control,
                                const PrefillExchangeView& view, int32_t layer, const uint32_t* seq, const float* inj,
                                float* X, float* y_out, int32_t tokens, long long timeout_cycles,
                                const float* ablate_direction, float ablate_scale, cudaStream_t stream) {
  if (control || view.header) return cudaErrorInvalidValue;
  const fb_moe_prefill_workspace f = to_fb(ws);
  return status(fb_moe_prefill_combine(&f, y_shared, nullptr, layer, seq, inj, X, y_out, tokens, timeout_cycles,
                                       ablate_direction, ablate_scale, stream));
}

// ---------------------------------------------------------------------------------- FP8-row projection
std::size_t linear_fp8_workspace_bytes(std::int32_t n, std::int32_t k, std::int32_t max_tokens) {
  return fb_linear_fp8_workspace_bytes(n, k, max_tokens);
}

void linear_fp8(const __nv_bfloat16* x, std::int32_t tokens, const Fp8RowWeight& weight,
                const LinearEpilogueParams& epilogue, void* workspace, std::size_t workspace_bytes,
                cudaStream_t stream, Fp8LinearPath path) {
  if (epilogue.kind == LinearEpilogue::SiluQuarter || epilogue.kind == LinearEpilogue::GrMix)
    throw std::invalid_argument("linear_fp8: the residual-mixer epilogues (SiluQuarter, GrMix) are not part of "
                                "fngine_b200; keep the stock kernel for them");
  static_assert(int(LinearEpilogue::StoreBf16) == FB_EPI_STORE_BF16 && int(LinearEpilogue::StoreF32) == FB_EPI_STORE_F32 &&
                    int(LinearEpilogue::GrWrite) == FB_EPI_GR_WRITE && int(LinearEpilogue::SwiGlu) == FB_EPI_SWIGLU &&
                    int(LinearEpilogue::SharedScale) == FB_EPI_SHARED_SCALE,
                "epilogue ids");
  static_assert(int(Fp8LinearPath::Auto) == FB_FP8_PATH_AUTO && int(Fp8LinearPath::A16) == FB_FP8_PATH_A16 &&
                    int(Fp8LinearPath::A8) == FB_FP8_PATH_A8,
                "path ids");
  const fb_linear_epilogue e = to_fb(epilogue);
  // Auto keeps the bf16 activations exact at every T, as the reference's Auto does (fp8/fp8_shapes.h:39-43)
  if (fb_linear_fp8(x, tokens, weight.codes, weight.scales, FB_DT_BF16, weight.n, weight.k, &e, workspace,
                    workspace_bytes, stream, static_cast<int32_t>(path)))
    throw std::invalid_argument(fb_last_error_string());  // the reference's error behaviour (linear_fp8.cpp:83-95)
}

}  // namespace fngine::kernels
