// Block-sparse attention for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a region
// whose memory is owned by another allocator (an inference server's arena, a
// framework's caching allocator that must see every byte), in a latency-critical
// thread where an implicit device synchronisation is unacceptable, or under a
// memory budget fixed at start-up.  The regular entry point, rt_sparse_attention,
// needs an rt_attn_plan whose work list lives in memory obtained with cudaMalloc,
// and it reports a kernel that gave up waiting through a lazily allocated word.
// The entry point in this file keeps all of that - work items, list entries,
// per-CTA offsets and the status word - in ONE file-scope device array of fixed
// size that every GPU loading the library holds until the process exits.
//
// Limits and rules (also in include/raptor_b200.h):
//   * at most kMaxItems work items and kMaxEntries list entries per call
//     (25 sequences of 4096 tokens with 12 heads fit); larger batches are
//     rejected with RT_ERR_UNSUPPORTED and nothing is launched;
//   * the array is shared by every call on the device and keeps the previous
//     call's contents: each call overwrites the parts it uses and clears the
//     status word.  Two calls whose GPU work overlaps (different streams, or
//     different host threads) would race on it - issue them on one stream;
//   * the first call on a device looks up the array's device address
//     (cudaGetSymbolAddress) and sets the kernel's shared-memory attributes; make
//     that first call before any stream capture;
//   * each call starts by reading back the status word of the previous call (a 4-byte
//     copy queued on the caller's stream, which the host waits for), so a kernel that
//     gave up is reported one call late - and, because of that wait and of the copies
//     from temporary host memory, a call on a stream that is being captured is refused
//     with RT_ERR_UNSUPPORTED.
#include <cuda_runtime.h>

#include <mutex>
#include <vector>

#include "attention.h"
#include "common.h"
#include "metadata.h"

namespace rt {
namespace {

constexpr int kMaxItems = 10240;
constexpr int kMaxEntries = 131072;
constexpr int kMaxCtas = 1024;

struct StaticScratch {
  AttnItem items[kMaxItems];
  int32_t entries[kMaxEntries];
  int32_t cta_ptr[kMaxCtas + 1];
  int32_t status;  // 0 = ok, otherwise the wait site at which the last kernel gave up
};

// ~0.84 MB per GPU.  In host code this name is only a handle for the runtime's symbol
// calls; the device address is obtained once per device below.
static __device__ __align__(256) unsigned char g_static_scratch[sizeof(StaticScratch)];

std::mutex g_mu;
StaticScratch* g_scratch_addr[64] = {nullptr};  // per device
int g_sm_count[64] = {0};

rt_status scratch_for_current_device(StaticScratch** out, int* sm_count) {
  int dev = 0;
  RT_CHECK_CUDA(cudaGetDevice(&dev));
  RT_REQUIRE(dev >= 0 && dev < 64, RT_ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    RT_CHECK_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    RT_REQUIRE(p != nullptr, RT_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    RT_CHECK_CUDA(cudaMemset(p, 0, sizeof(StaticScratch)));
    int sms = 0;
    RT_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    g_sm_count[dev] = sms;
    g_scratch_addr[dev] = static_cast<StaticScratch*>(p);
  }
  *out = g_scratch_addr[dev];
  *sm_count = g_sm_count[dev];
  return RT_OK;
}

}  // namespace

// The status word of the static scratch on the current device (for the bounded-wait self-test).
int* static_scratch_status_word() {
  StaticScratch* sc = nullptr;
  int sms = 0;
  if (scratch_for_current_device(&sc, &sms) != RT_OK) return nullptr;
  return &sc->status;
}

}  // namespace rt

using namespace rt;

extern "C" rt_status rt_sparse_attention_static(void* ctx_dev, const void* q_dev, const void* k_dev,
                                                const void* v_dev, const rt_config* cfg,
                                                const int32_t* lens_tokens_host, int n_seq,
                                                const int32_t* kv_ptr_host, const int32_t* kv_idx_host, float scale,
                                                int dtype, void* stream) {
  RT_REQUIRE(ctx_dev && q_dev && k_dev && v_dev && cfg && lens_tokens_host && kv_ptr_host && kv_idx_host,
             RT_ERR_INVALID, "sparse_attention_static: null pointer");
  RT_TRY(check_config(cfg));
  RT_TRY(validate_lengths(*cfg, lens_tokens_host, n_seq));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Every call reads the status word back (the host blocks on it) and copies its work list from
  // host memory that is released on return: neither can be recorded into a CUDA graph.
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone)
    return fail(RT_ERR_UNSUPPORTED, "sparse_attention_static: the stream is being captured; this entry point "
                                    "blocks on a status read-back and cannot be recorded into a CUDA graph");
  StaticScratch* sc = nullptr;
  int sms = 0;
  RT_TRY(scratch_for_current_device(&sc, &sms));
  const int n_ctas = 2 * sms;
  RT_REQUIRE(n_ctas <= kMaxCtas, RT_ERR_UNSUPPORTED, "sparse_attention_static: %d SMs exceed the static CTA table", sms);

  // Status of the previous call, then clear it for this one.  The read is queued on `st` itself, so it
  // is ordered behind the previous call's kernel whatever kind of stream `st` is (a copy on the legacy
  // default stream would not wait for a non-blocking stream), and the host waits for it.
  int32_t prev = 0;
  RT_CHECK_CUDA(cudaMemcpyAsync(&prev, &sc->status, sizeof(prev), cudaMemcpyDeviceToHost, st));
  RT_CHECK_CUDA(cudaStreamSynchronize(st));
  RT_CHECK_CUDA(cudaMemsetAsync(&sc->status, 0, sizeof(int32_t), st));
  if (prev != 0)
    return fail(RT_ERR_DEVICE_WAIT, "sparse_attention_static: the previous call's kernel gave up at wait site %d", prev);

  int n_blocks = 0;
  for (int s = 0; s < n_seq; ++s) n_blocks += lens_tokens_host[s] / cfg->block;
  AttnPlanHost plan;  // host memory only
  RT_TRY(build_attn_plan(*cfg, lens_tokens_host, n_seq, kv_ptr_host, kv_idx_host, kv_ptr_host[n_blocks], n_ctas, plan,
                         /*split_entries=*/0));  // partial results would need more scratch: lists stay whole
  RT_REQUIRE(static_cast<int>(plan.items.size()) <= kMaxItems && static_cast<int>(plan.entries.size()) <= kMaxEntries,
             RT_ERR_UNSUPPORTED,
             "sparse_attention_static: batch needs %zu work items / %zu list entries, the static scratch holds %d / %d "
             "(use rt_sparse_attention with an rt_attn_plan for larger batches)",
             plan.items.size(), plan.entries.size(), kMaxItems, kMaxEntries);
  // pageable host -> device copies return once the source has been staged, so the
  // host-side plan may be released when this function returns
  RT_CHECK_CUDA(cudaMemcpyAsync(sc->items, plan.items.data(), plan.items.size() * sizeof(AttnItem),
                                cudaMemcpyHostToDevice, st));
  RT_CHECK_CUDA(cudaMemcpyAsync(sc->entries, plan.entries.data(), plan.entries.size() * sizeof(int32_t),
                                cudaMemcpyHostToDevice, st));
  RT_CHECK_CUDA(cudaMemcpyAsync(sc->cta_ptr, plan.cta_ptr.data(), plan.cta_ptr.size() * sizeof(int32_t),
                                cudaMemcpyHostToDevice, st));
  return launch_sparse_attention(ctx_dev, q_dev, k_dev, v_dev, sc->items, sc->entries, sc->cta_ptr, n_ctas,
                                 plan.total_tokens, plan.heads, scale, dtype, st, &sc->status);
}
