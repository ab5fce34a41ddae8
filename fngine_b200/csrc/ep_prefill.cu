// Expert-parallel prefill layer behind one C entry point: the rank's kernels (top-10, pair lists, grouped
// gate/up, grouped down, per-row sums) with the two exchanges done by the collective library the caller
// already has a communicator of. The library is not linked: its handful of functions is looked up in the
// process at the first call (the image a host framework already loaded, else libnccl.so.2 by name), so the
// shared object loads and every other entry point works where that library is absent.
#include <dlfcn.h>

#include <mutex>

#include "common.cuh"

namespace fb {
namespace {

// The part of the collective library's public C interface used here (nccl.h): an opaque communicator,
// result 0 = success, the data type and reduction codes below, and these seven functions.
using Comm = void*;
constexpr int kNcclInt8 = 0, kNcclInt32 = 2, kNcclFloat32 = 7, kNcclSum = 0;

struct Nccl {
  int (*all_gather)(const void*, void*, size_t, int, Comm, cudaStream_t) = nullptr;
  int (*reduce_scatter)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*send)(const void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*recv)(void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*group_start)() = nullptr;
  int (*group_end)() = nullptr;
  int (*comm_count)(Comm, int*) = nullptr;
  int (*comm_user_rank)(Comm, int*) = nullptr;
  const char* (*error_string)(int) = nullptr;
  bool ok = false;
};

const Nccl& nccl() {
  static Nccl n;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy the host process already uses
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    auto sym = [&](const char* name) { return dlsym(h, name); };
    n.all_gather = reinterpret_cast<decltype(n.all_gather)>(sym("ncclAllGather"));
    n.reduce_scatter = reinterpret_cast<decltype(n.reduce_scatter)>(sym("ncclReduceScatter"));
    n.send = reinterpret_cast<decltype(n.send)>(sym("ncclSend"));
    n.recv = reinterpret_cast<decltype(n.recv)>(sym("ncclRecv"));
    n.group_start = reinterpret_cast<decltype(n.group_start)>(sym("ncclGroupStart"));
    n.group_end = reinterpret_cast<decltype(n.group_end)>(sym("ncclGroupEnd"));
    n.comm_count = reinterpret_cast<decltype(n.comm_count)>(sym("ncclCommCount"));
    n.comm_user_rank = reinterpret_cast<decltype(n.comm_user_rank)>(sym("ncclCommUserRank"));
    n.error_string = reinterpret_cast<decltype(n.error_string)>(sym("ncclGetErrorString"));
    n.ok = n.all_gather && n.reduce_scatter && n.send && n.recv && n.group_start && n.group_end && n.comm_count &&
           n.comm_user_rank;
  });
  return n;
}

int32_t nccl_failed(const char* what, int rc) {
  const Nccl& n = nccl();
  set_error("ep_prefill_layer: %s failed: %s", what, n.error_string ? n.error_string(rc) : "collective library error");
  return int32_t(cudaErrorUnknown);
}

constexpr int kHidden = 2560, kTopK = 10;
constexpr size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

// Scratch layout: [e_local][w_local][x_all][e_all][w_all][y_part][recv (all-to-all combine only)]
struct Scratch {
  int32_t* e_local;
  float* w_local;
  uint8_t* x_all;
  int32_t* e_all;
  float* w_all;
  float* y_part;
  float* recv;
  size_t bytes;
};
Scratch carve(void* base, int tokens_local, int n_ranks, int combine) {
  const size_t tl = size_t(tokens_local), rows = tl * size_t(n_ranks);
  uint8_t* p = static_cast<uint8_t*>(base);
  size_t off = 0;
  auto take = [&](size_t n) {
    uint8_t* q = p + off;
    off += align256(n);
    return q;
  };
  Scratch s;
  s.e_local = reinterpret_cast<int32_t*>(take(tl * kTopK * 4));
  s.w_local = reinterpret_cast<float*>(take(tl * kTopK * 4));
  s.x_all = take(rows * kHidden * 2);
  s.e_all = reinterpret_cast<int32_t*>(take(rows * kTopK * 4));
  s.w_all = reinterpret_cast<float*>(take(rows * kTopK * 4));
  s.y_part = reinterpret_cast<float*>(take(rows * kHidden * 4));
  s.recv = reinterpret_cast<float*>(take(combine == FB_EP_COMBINE_ALL_TO_ALL && n_ranks > 1 ? rows * kHidden * 4 : 0));
  s.bytes = off;
  return s;
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" {

size_t fb_ep_prefill_scratch_bytes(int32_t tokens_local, int32_t n_ranks, int32_t combine) {
  if (tokens_local < 1 || n_ranks < 1 || n_ranks > FB_EP_MAX_RANKS) return 0;
  return carve(nullptr, tokens_local, n_ranks, combine).bytes;
}

int32_t fb_ep_prefill_layer(const fb_moe_expert_layout* layout, const uint8_t* const* expert_blob, const int32_t* share,
                            int32_t expert_lo, int32_t expert_hi, const float* router_logits, int32_t logits_stride,
                            const void* x_bf16, int32_t tokens_local, int32_t n_ranks, int32_t combine,
                            const fb_moe_prefill_workspace* ws, void* scratch, float* y_local, void* comm,
                            void* stream) {
  if (!layout || !expert_blob || !router_logits || !x_bf16 || !ws || !scratch || !y_local)
    return invalid("ep_prefill_layer: null argument");
  if (tokens_local < 1 || n_ranks < 1 || n_ranks > FB_EP_MAX_RANKS)
    return invalid("ep_prefill_layer: tokens_local %d, n_ranks %d", tokens_local, n_ranks);
  if (combine != FB_EP_COMBINE_ALL_TO_ALL && combine != FB_EP_COMBINE_REDUCE_SCATTER)
    return invalid("ep_prefill_layer: combine %d", combine);
  if ((reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) return invalid("ep_prefill_layer: scratch must be 256-byte aligned");
  const int64_t rows64 = int64_t(tokens_local) * n_ranks;
  if (rows64 > ws->capacity)
    return invalid("ep_prefill_layer: %lld rows exceed the workspace capacity %d", (long long)rows64, ws->capacity);
  if (!share && (expert_lo < 0 || expert_hi > 512 || expert_lo >= expert_hi))
    return invalid("ep_prefill_layer: expert range [%d, %d)", expert_lo, expert_hi);
  const int rows = int(rows64);
  const Nccl& n = nccl();
  if (n_ranks > 1) {
    if (!comm) return invalid("ep_prefill_layer: no communicator for %d ranks", n_ranks);
    if (!n.ok) {
      set_error("ep_prefill_layer: the collective library (libnccl.so.2) is not available in this process");
      return int32_t(cudaErrorNotSupported);
    }
    int count = 0;
    int rc = n.comm_count(comm, &count);
    if (rc != 0) return nccl_failed("ncclCommCount", rc);
    if (count != n_ranks) return invalid("ep_prefill_layer: communicator has %d ranks, call says %d", count, n_ranks);
  }
  cudaStream_t st = as_stream(stream);
  const Scratch s = carve(scratch, tokens_local, n_ranks, combine);
  const size_t tl = size_t(tokens_local);

  // 1. the owner's top-10 lists
  int32_t e = fb_moe_topk(router_logits, logits_stride, tokens_local, n_ranks > 1 ? s.e_local : s.e_all,
                          n_ranks > 1 ? s.w_local : s.w_all, stream);
  if (e != 0) return e;
  // 2. every rank gets every row and list (fixed sizes: nothing is read back on the host)
  const void* x_rows = x_bf16;
  if (n_ranks > 1) {
    int rc = n.group_start();
    if (rc != 0) return nccl_failed("ncclGroupStart", rc);
    rc = n.all_gather(x_bf16, s.x_all, tl * kHidden * 2, kNcclInt8, comm, st);
    if (rc == 0) rc = n.all_gather(s.e_local, s.e_all, tl * kTopK, kNcclInt32, comm, st);
    if (rc == 0) rc = n.all_gather(s.w_local, s.w_all, tl * kTopK, kNcclFloat32, comm, st);
    const int rc_end = n.group_end();
    if (rc != 0) return nccl_failed("ncclAllGather", rc);
    if (rc_end != 0) return nccl_failed("ncclGroupEnd", rc_end);
    x_rows = s.x_all;
  }
  // 3. this rank's experts over all rows: one partial row per row
  e = share ? fb_moe_route_placed(s.e_all, s.w_all, share, rows, ws, stream)
            : fb_moe_route_ep(s.e_all, s.w_all, expert_lo, expert_hi, rows, ws, stream);
  if (e != 0) return e;
  e = fb_moe_grouped_gate_up(layout, expert_blob, x_rows, rows, ws, stream);
  if (e != 0) return e;
  e = fb_moe_grouped_down(layout, expert_blob, rows, ws, stream);
  if (e != 0) return e;
  float* y_part = n_ranks > 1 ? s.y_part : y_local;
  e = fb_moe_prefill_combine(ws, nullptr, nullptr, 0, nullptr, nullptr, nullptr, y_part, rows, 0, nullptr, 0.0f, stream);
  if (e != 0 || n_ranks == 1) return e;
  // 4. the partial rows go back to their owners
  const size_t chunk = tl * kHidden;
  if (combine == FB_EP_COMBINE_REDUCE_SCATTER) {
    const int rc = n.reduce_scatter(s.y_part, y_local, chunk, kNcclFloat32, kNcclSum, comm, st);
    if (rc != 0) return nccl_failed("ncclReduceScatter", rc);
    return 0;
  }
  int rc = n.group_start();
  if (rc != 0) return nccl_failed("ncclGroupStart", rc);
  for (int d = 0; d < n_ranks && rc == 0; ++d) {
    rc = n.send(s.y_part + size_t(d) * chunk, chunk, kNcclFloat32, d, comm, st);
    if (rc == 0) rc = n.recv(s.recv + size_t(d) * chunk, chunk, kNcclFloat32, d, comm, st);
  }
  const int rc_end = n.group_end();
  if (rc != 0) return nccl_failed("ncclSend/ncclRecv", rc);
  if (rc_end != 0) return nccl_failed("ncclGroupEnd", rc_end);
  return fb_ep_sum_ranks(s.recv, n_ranks, tokens_local, y_local, stream);
}

}  // extern "C"
