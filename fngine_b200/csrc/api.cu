// Host-side pieces of the C ABI that launch nothing: error text, format tables, layout helpers.
#include "common.cuh"

#include <cstdarg>
#include <cstring>

namespace fb {
namespace {
thread_local char g_err[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int32_t invalid(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return int32_t(cudaErrorInvalidValue);
}

int32_t check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return 0;
  set_error("%s: %s", what, cudaGetErrorString(e));
  return int32_t(e);
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace fb

extern "C" {

const char* fb_last_error_string(void) { return fb::g_err; }
int32_t fb_abi_version(void) { return 1; }
int32_t fb_compiled_sm(void) { return 100; }

int64_t fb_moe_row_bytes(int32_t format, int32_t k) {
  if (k <= 0) return 0;
  if (format == FB_FMT_IQ3_S) return k % 256 ? 0 : int64_t(k) / 256 * 110;
  if (format == FB_FMT_IQ4_NL) return k % 32 ? 0 : int64_t(k) / 32 * 18;
  if (format == FB_FMT_IQ3_XXS) return k % 256 ? 0 : int64_t(k) / 256 * 98;
  if (format == FB_FMT_IQ2_S) return k % 256 ? 0 : int64_t(k) / 256 * 82;
  if (format == FB_FMT_IQ4_XS) return k % 256 ? 0 : int64_t(k) / 256 * 136;
  if (format == FB_FMT_Q2_0) return k % 64 ? 0 : int64_t(k) / 64 * 18;
  return 0;
}

int32_t fb_moe_act_format(int32_t format) {
  if (format == FB_FMT_IQ3_S || format == FB_FMT_IQ3_XXS || format == FB_FMT_IQ2_S || format == FB_FMT_IQ4_XS)
    return FB_ACT_Q8_K;
  if (format == FB_FMT_IQ4_NL || format == FB_FMT_Q2_0) return FB_ACT_Q8_0;
  return -1;
}

int64_t fb_act_row_bytes(int32_t act_format, int32_t k) {
  if (k <= 0) return 0;
  if (act_format == FB_ACT_Q8_K) return k % 256 ? 0 : int64_t(k) / 256 * 292;
  if (act_format == FB_ACT_Q8_0) return k % 32 ? 0 : int64_t(k) / 32 * 34;
  return 0;
}

int64_t fb_moe_blob_bytes(int32_t gate_up_format, int32_t down_format, int32_t inter) {
  const int64_t gu = fb_moe_row_bytes(gate_up_format, FB_HIDDEN), dn = fb_moe_row_bytes(down_format, inter);
  if (!gu || !dn || inter <= 0) return 0;
  return 2 * int64_t(inter) * gu + int64_t(FB_HIDDEN) * dn;
}

int32_t fb_moe_expert_layout_make(const uint8_t* slots, int64_t blob_stride, int32_t gate_up_format,
                                  int32_t down_format, int32_t inter, fb_moe_expert_layout* out) {
  if (!out) return fb::invalid("expert_layout_make: out is NULL");
  const int64_t gate_bytes = int64_t(inter) * fb_moe_row_bytes(gate_up_format, FB_HIDDEN);
  if (gate_bytes <= 0 || !fb_moe_row_bytes(down_format, inter))
    return fb::invalid("expert_layout_make: unsupported format/inter (ggml type ids 18, 20, 21, 22, 23, 42)");
  if (blob_stride < fb_moe_blob_bytes(gate_up_format, down_format, inter) || (blob_stride & 15))
    return fb::invalid("expert_layout_make: blob_stride too small or not a multiple of 16");
  out->slots = slots;
  out->blob_stride = blob_stride;
  out->gate_offset = 0;
  out->up_offset = gate_bytes;
  out->down_offset = 2 * gate_bytes;
  out->gate_up_format = gate_up_format;
  out->down_format = down_format;
  out->inter = inter;
  out->reserved = 0;
  return 0;
}

}  // extern "C"
