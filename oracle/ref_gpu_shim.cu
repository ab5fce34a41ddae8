// TEST INFRASTRUCTURE ONLY: C-linkage entry into the reference's own GPU decode kernels
// (src/kernels/moe/moe_decode.cu of the reference, compiled unchanged for sm_100a by
// oracle/build_ref_gpu.py into oracle/_ref_gpu/). It exists so that the benchmark can time the
// reference's kernels on the same GPU, at the reference's native shape (intermediate 640), beside this
// library's; nothing in the product path links or loads it.
#include "kernels/moe/moe.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

using namespace fngine::kernels;

extern "C" {

size_t refgpu_decode_workspace_bytes() { return moe_decode_workspace_bytes(); }

// One decode layer as Forward::moe's decode branch issues it without the shared expert and without a
// CPU tier (src/model/forward.cpp:356-376): select -> hot gate/up -> hot down -> combine.
// router_logits: fp32 [tokens][513]; x: bf16 [tokens][2560]; slots: the layer's slot array (slot == expert);
// ws_base: 256-byte aligned device memory of refgpu_decode_workspace_bytes(), zero-filled once;
// y_out: fp32 [tokens][2560]; y_shared fp32 [tokens][2560], X fp32 [tokens][4][2560] and inj fp32 [tokens][4]:
// the combine reads and writes them unconditionally. Returns a cudaError_t.
int refgpu_layer_decode(const float* router_logits, const void* x_bf16, const unsigned char* slots, long long blob_stride,
                        int gate_up_format, int down_format, int tokens, void* ws_base, const float* y_shared,
                        const float* inj, float* X, float* y_out, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const MoeDecodeWorkspace ws = make_moe_decode_workspace(ws_base);
  const MoeExpertLayout layout = make_moe_expert_layout(slots, blob_stride, static_cast<MoeFormat>(gate_up_format),
                                                        static_cast<MoeFormat>(down_format));
  cudaError_t e = moe_select_publish(router_logits, static_cast<const __nv_bfloat16*>(x_bf16), nullptr, 0, nullptr, nullptr,
                                     tokens, ws, s, nullptr);
  if (e != cudaSuccess) return int(e);
  e = moe_hot_gate_up(layout, tokens, ws, s);
  if (e != cudaSuccess) return int(e);
  e = moe_hot_down(layout, tokens, ws, s);
  if (e != cudaSuccess) return int(e);
  e = moe_combine(ws, y_shared, nullptr, 0, nullptr, inj, X, y_out, tokens, kMoeExchangeTimeoutCycles, nullptr, 1.0f, s);
  return int(e);
}

}  // extern "C"
