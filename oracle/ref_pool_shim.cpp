// TEST INFRASTRUCTURE ONLY: C-linkage entry into the reference's own cpu::ExpertPool.
//
// The pool is the reference's production CPU expert tier (src/cpu/expert_pool.h:76-102); its shape is
// fixed at compile time (hidden 2560, intermediate 640, a Q8_0-family down projection). This shim runs
// one decode step of ONE layer through the pool's host exchange, the way the reference's own harness
// does (tests/cpu/pool_bench.h:42-140, tests/cpu/cpu_test_util.h:155-180): fill the layer's publish
// block, release ready[l] for every layer, wait for done[layer], read the result block. It is built
// into oracle/_ref by oracle/build_ref.py together with the reference sources it calls.
#include "core/exchange.h"
#include "core/model_dims.h"
#include "cpu/expert_pool.h"

#include <immintrin.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <vector>

using namespace fngine;

namespace {
void store_release(uint32_t& cell, uint32_t v) {
  std::atomic_ref<uint32_t>(cell).store(v, std::memory_order_release);
}
uint32_t load_acquire(const uint32_t& cell) {
  return std::atomic_ref<uint32_t>(const_cast<uint32_t&>(cell)).load(std::memory_order_acquire);
}
}  // namespace

extern "C" {

// y[T][2560] = the pool's result rows for one decode step of `tokens` tokens whose ten experts are all
// "cold" (computed by the pool). blobs: n_experts expert blobs `blob_stride` bytes apart with gate / up /
// down at the given offsets. ids / weights: [tokens][10]. Returns 0, or 1 with a message in err.
int ref_pool_decode_step(int gu_format, int down_format, const unsigned char* blobs, long long blob_stride,
                         int n_experts, long long gate_offset, long long up_offset, long long down_offset,
                         const unsigned short* x_bf16, int tokens, const int* ids, const float* weights, int workers,
                         float* y, char* err, int err_len) {
  try {
    if (tokens < 1 || tokens > kDecodeExchangeTokens || n_experts < 1 || n_experts > dims::kExperts || workers < 1)
      throw std::invalid_argument("bad tokens / experts / workers");
    void* mem = nullptr;
    if (posix_memalign(&mem, 4096, sizeof(DecodeExchange)) != 0) throw std::bad_alloc();
    std::memset(mem, 0, sizeof(DecodeExchange));
    auto* dec = static_cast<DecodeExchange*>(mem);
    const int layer = 0;
    std::vector<const void*> slots(std::size_t(kExchangeLayers) * dims::kExperts, nullptr);
    for (int e = 0; e < n_experts; ++e) slots[std::size_t(layer) * dims::kExperts + e] = blobs + std::size_t(e) * blob_stride;
    int rc = 0;
    {
      cpu::PoolConfig cfg;
      cfg.worker_cpus.assign(std::size_t(workers), -1);  // unpinned
      cfg.layers[layer] = cpu::ExpertLayerDesc{static_cast<cpu::WeightFormat>(gu_format),
                                               static_cast<cpu::WeightFormat>(down_format), std::size_t(gate_offset),
                                               std::size_t(up_offset), std::size_t(down_offset)};
      cfg.host_slot_of = slots.data();
      cfg.decode = dec;
      cpu::ExpertPool pool(cfg);
      const uint32_t seq = 1;
      pool.begin(seq, cpu::PoolMode::Decode);
      MoeDecodePublish& p = dec->publish[layer];
      p.tokens = tokens;
      p.n_cold = tokens * dims::kTopK;
      for (int t = 0; t < tokens; ++t) {
        p.cold_count[t] = dims::kTopK;
        for (int j = 0; j < dims::kTopK; ++j) {
          p.cold_expert[t][j] = ids[t * dims::kTopK + j];
          p.cold_weight[t][j] = weights[t * dims::kTopK + j];
        }
        std::memcpy(&p.x[t][0], x_bf16 + std::size_t(t) * dims::kHidden, dims::kHidden * 2);
      }
      for (int l = 0; l < kExchangeLayers; ++l) {
        if (l != layer) dec->publish[l].tokens = tokens;  // n_cold stays 0: the pool skips the layer
        store_release(dec->control.ready[l].value, seq);
      }
      const auto t0 = std::chrono::steady_clock::now();
      while (load_acquire(dec->control.done[layer].value) != seq) {
        _mm_pause();
        if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(60)) {
          store_release(dec->control.abort.value, 1);
          std::snprintf(err, std::size_t(err_len), "the pool did not finish the layer within 60 s");
          rc = 1;
          break;
        }
      }
      pool.wait_idle();
      if (!rc && pool.failed()) {
        std::snprintf(err, std::size_t(err_len), "%s", pool.failure().c_str());
        rc = 1;
      }
      if (!rc)
        for (int t = 0; t < tokens; ++t)
          std::memcpy(y + std::size_t(t) * dims::kHidden, &dec->result[layer].y[t][0], dims::kHidden * sizeof(float));
    }
    std::free(mem);
    return rc;
  } catch (const std::exception& e) {
    std::snprintf(err, std::size_t(err_len), "%s", e.what());
    return 1;
  }
}

}  // extern "C"
