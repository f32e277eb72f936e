// Encoder object behind the C ABI: owns the weights (re-laid-out once to
// [out][in]), the scratch buffers (the reference's TensorSet), the per-batch
// metadata pipeline and the launch order of one layer.
//
// Metadata pipeline (rebuild of layers/metadata.cpp + layers/semaphore.cpp +
// the per-layer std::async workers of layers/multi_headed_attention.h:72-110 on
// CUDA streams and events): the encoder owns ONE persistent host worker.
// prepare_batch() hands it the batch; it builds, layer by layer, the attention work
// list into pinned memory, enqueues one upload per layer on a side stream and records
// an event per layer.  Query-block pairs, cuts of long lists and the assignment of
// work items to CTAs are computed once per batch (layer 0); the other layers only
// refill the list entries from their own block tables.  The forward pass issues the
// QKV GEMM of layer i first, then makes the compute stream wait on layer i's event
// (after a host-side check that the event has been recorded), so table construction
// and upload overlap the GEMMs.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <chrono>
#include <condition_variable>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "attention.h"
#include "common.h"
#include "device_error.h"
#include "launch_count.h"
#include "metadata.h"

namespace rt {
namespace {

__global__ void transpose16_kernel(uint16_t* __restrict__ dst, const uint16_t* __restrict__ src, int rows, int cols) {
  // dst[c][r] = src[r][c]; 32x32 tiles through shared memory
  __shared__ uint16_t tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[i][threadIdx.x] = src[static_cast<size_t>(r) * cols + c];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[static_cast<size_t>(c) * rows + r] = tile[threadIdx.x][i];
  }
}

__global__ void position_ids_kernel(int32_t* __restrict__ pos, const int32_t* __restrict__ seq_prefix, int n_seq,
                                    int tokens) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const int blk = t >> 6;
  int lo = 0, hi = n_seq;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (seq_prefix[mid] <= blk) lo = mid; else hi = mid;
  }
  pos[t] = t - seq_prefix[lo] * 64;
}

struct DevBuf {
  void* p = nullptr;
  size_t bytes = 0;
  rt_status ensure(size_t need) {
    if (need <= bytes) return RT_OK;
    if (p) cudaFree(p);
    p = nullptr;
    bytes = 0;
    RT_CHECK_CUDA(cudaMalloc(&p, need));
    bytes = need;
    return RT_OK;
  }
  void release() {
    if (p) cudaFree(p);
    p = nullptr;
    bytes = 0;
  }
};

struct LayerWeights {
  DevBuf qkv_w, qkv_b, ao_w, ao_b, aln_g, aln_b, up_w, up_b, down_w, down_b, oln_g, oln_b;
  uint32_t seed = 0;
  bool set = false;
};

struct StageTimer {
  std::vector<std::pair<std::string, std::pair<cudaEvent_t, cudaEvent_t>>> spans;
  std::vector<cudaEvent_t> pool;
  size_t used = 0;
  cudaEvent_t get() {
    if (used == pool.size()) {
      cudaEvent_t e;
      cudaEventCreate(&e);
      pool.push_back(e);
    }
    return pool[used++];
  }
  void reset() {
    spans.clear();
    used = 0;
  }
};

}  // namespace
}  // namespace rt

using namespace rt;

struct rt_encoder {
  rt_config cfg{};
  int sm_count = 148;
  int attn_ctas = 296;  // two resident attention CTAs per SM
  std::vector<LayerWeights> layers;
  DevBuf emb_word, emb_pos, emb_type, emb_g, emb_b;
  bool emb_set = false;
  bool fuse_gelu = true;
  bool fuse_qkv = true;
  // LayerNorm in the epilogue of the hidden-wide projections (rt_gemm_bias_residual_layernorm):
  // 0 never, 1 where it measured faster (FFN-down of a 768-wide model: long K, three column tiles), 2 wherever
  // the kernel exists (hidden 768 / 1024, both projections)
  int fuse_layernorm = 1;
  bool fuse_residual = false;  // measured slower on B200 (GEMM epilogue cost > LayerNorm saving); kept as an option

  // scratch ("TensorSet")
  std::map<std::string, DevBuf> scratch;
  int capacity_tokens = 0;

  // batch state
  std::vector<int32_t> lens;
  int n_seq = 0, tokens = 0, n_blocks = 0;
  bool prepared = false;
  int device = 0;
  DevBuf ids_dev, pos_dev;

  // Per-batch metadata lives in one of kSlots slots (round robin), so the worker can fill
  // the next batches' tables while earlier batches' kernels still read theirs.
  static constexpr int kSlots = 3;
  // A slot holds, for every layer, one region with the same layout in pinned host
  // memory and on the device: work items | list entries | per-CTA offsets.
  struct Slot {
    uint8_t* meta_pinned = nullptr;
    size_t meta_cap = 0;
    DevBuf meta_dev;
    int32_t* prefix_pinned = nullptr;  // [n_seq+1] block prefix sums, then [n_blocks][2] {first token, length}
    int prefix_cap = 0;
    DevBuf prefix_dev;
    size_t block_seq_off = 0;          // offset (int32 units) of the per-block table
    cudaEvent_t prefix_ready = nullptr;
    cudaEvent_t forward_done = nullptr;
    cudaEvent_t uploads_done = nullptr;  // behind the last layer's upload: the pinned region may be rewritten
    bool forward_recorded = false;
    bool uploads_recorded = false;
    bool used = false;
    std::vector<cudaEvent_t> table_ready;
  } slots[kSlots];
  uint64_t batch_counter = 0;
  Slot* cur = nullptr;
  size_t region_bytes = 0, items_off = 0, entries_off = 0, cta_off = 0, groups_off = 0;
  std::vector<int> plan_groups;        // per layer: split lists to merge
  DevBuf part_o, part_ml;              // partial results of split lists (shared by all layers)
  std::vector<BlockCsr> csr;           // per layer, host copy (tests / accessors)
  std::vector<int64_t> plan_entries;   // per layer
  int64_t plan_visits = 0;
  int plan_items = 0;
  TableCache table_cache;
  TemplateCache template_cache;
  std::vector<bool> csr_valid;         // host CSR copies are built on demand

  cudaStream_t meta_stream = nullptr;

  // Host-buffer pipeline (rt_encoder_submit_host / rt_encoder_wait_host): batches run back
  // to back on pipe_stream, each with its own device id and output buffers; in_stream brings a
  // batch's ids over while the previous batch computes, and copy_stream carries a finished
  // batch to the caller's memory while the next batch computes.
  struct HostJob {
    DevBuf ids, out;
    cudaEvent_t ids_ready = nullptr, computed = nullptr, copied = nullptr;
    int* err_host = nullptr;  // pinned copy of the device error word, taken behind the output copy
    bool busy = false;
    uint64_t ticket = 0;
  } jobs[2];
  cudaStream_t pipe_stream = nullptr, copy_stream = nullptr, in_stream = nullptr;
  uint64_t next_ticket = 1;
  // persistent metadata worker: sleeps on `cv` until prepare_batch posts a job
  std::thread worker;
  std::mutex mu;
  std::condition_variable cv;
  bool job_posted = false, worker_busy = false, worker_exit = false;
  int layers_recorded = 0;
  rt_status worker_status = RT_OK;
  std::string worker_error;
  PlanSkeleton skeleton;       // of the current batch (layer 0's assembly)
  AttnPlanHost base_plan;

  // timing
  bool timing = false;
  StageTimer timer;
  double pre_process_ms = 0.0;
  double host_blocked_ms = 0.0;  // cumulative: time the calling thread spent waiting for the GPU to free a slot / buffer
  std::map<std::string, float> last_ms;

  // returns once the worker has finished the batch it was given (it keeps running)
  void join_worker() {
    std::unique_lock<std::mutex> lk(mu);
    cv.wait(lk, [&] { return !job_posted && !worker_busy; });
  }
};

namespace {

size_t align256(size_t x) { return (x + 255) & ~size_t(255); }
size_t elt() { return 2; }

rt_status copy_or_transpose(DevBuf& dst, const void* src, int rows_in, int cols_in, bool transpose) {
  const size_t bytes = static_cast<size_t>(rows_in) * cols_in * 2;
  RT_TRY(dst.ensure(bytes));
  if (!transpose) {
    RT_CHECK_CUDA(cudaMemcpy(dst.p, src, bytes, cudaMemcpyDeviceToDevice));
  } else {
    dim3 grid((cols_in + 31) / 32, (rows_in + 31) / 32), block(32, 8);
    transpose16_kernel<<<grid, block>>>((uint16_t*)dst.p, (const uint16_t*)src, rows_in, cols_in);
    RT_CHECK_CUDA(cudaGetLastError());
    RT_CHECK_CUDA(cudaDeviceSynchronize());
  }
  return RT_OK;
}

rt_status copy_vec(DevBuf& dst, const void* src, size_t bytes) {
  RT_TRY(dst.ensure(bytes));
  RT_CHECK_CUDA(cudaMemcpy(dst.p, src, bytes, cudaMemcpyDeviceToDevice));
  return RT_OK;
}

struct Span {
  rt_encoder* e;
  cudaStream_t st;
  cudaEvent_t stop = nullptr;
  Span(rt_encoder* enc, cudaStream_t s, const char* key) : e(enc), st(s) {
    if (!e->timing) return;
    cudaEvent_t a = e->timer.get();
    stop = e->timer.get();
    cudaEventRecord(a, st);
    e->timer.spans.push_back({key, {a, stop}});
  }
  ~Span() {
    if (stop) cudaEventRecord(stop, st);
  }
};

// One batch: per layer, per-sequence templates (cached across batches) -> work list -> pinned
// region -> one asynchronous upload -> event.
void build_batch_metadata(rt_encoder* e) {
  rt_encoder::Slot& slot = *e->cur;
  std::vector<const SeqTemplate*> tmpl(e->n_seq);
  AttnPlanHost refill;
  for (int l = 0; l < e->cfg.layers; ++l) {
    rt_status s = RT_OK;
    for (int q = 0; q < e->n_seq && s == RT_OK; ++q) {
      const int L = e->lens[q] / e->cfg.block;
      // lists that do not depend on a random table are shared by all layers
      const uint32_t seed = uses_random_table(e->cfg, L) ? e->layers[l].seed : 0xffffffffu;
      auto key = std::make_pair(seed, L);
      auto it = e->template_cache.find(key);
      if (it == e->template_cache.end()) {
        SeqTemplate t;
        s = build_seq_template(e->cfg, seed, L, &e->table_cache, t);
        if (s == RT_OK) it = e->template_cache.emplace(key, std::move(t)).first;
      }
      if (s == RT_OK) tmpl[q] = &it->second;
    }
    const AttnPlanHost* plan = nullptr;
    if (s == RT_OK) {
      if (l == 0) {
        s = assemble_attn_plan(e->cfg, e->lens.data(), e->n_seq, tmpl.data(), e->attn_ctas, e->base_plan,
                               kDefaultSplitEntries, &e->skeleton);
        plan = &e->base_plan;
      } else {
        s = refill_attn_plan(e->skeleton, e->base_plan, tmpl.data(), refill);
        if (s == RT_ERR_STATE)  // a list that is cut changed its length: assemble this layer on its own
          s = assemble_attn_plan(e->cfg, e->lens.data(), e->n_seq, tmpl.data(), e->attn_ctas, refill);
        plan = &refill;
      }
    }
    if (s == RT_OK) {
      uint8_t* host = slot.meta_pinned + static_cast<size_t>(l) * e->region_bytes;
      uint8_t* dev = static_cast<uint8_t*>(slot.meta_dev.p) + static_cast<size_t>(l) * e->region_bytes;
      const size_t items_b = plan->items.size() * sizeof(AttnItem);
      const size_t entries_b = plan->entries.size() * sizeof(int32_t);
      const size_t cta_b = plan->cta_ptr.size() * sizeof(int32_t);
      const size_t groups_b = plan->groups.size() * sizeof(int32_t);
      if (e->items_off + items_b > e->entries_off || e->entries_off + entries_b > e->cta_off ||
          e->cta_off + cta_b > e->groups_off || e->groups_off + groups_b > e->region_bytes ||
          static_cast<size_t>(plan->n_slots) * 128 * 64 * sizeof(float) > e->part_o.bytes) {
        s = RT_ERR_STATE;
        last_error_ref() = "metadata region overflow";
      } else {
        std::memcpy(host + e->items_off, plan->items.data(), items_b);
        std::memcpy(host + e->entries_off, plan->entries.data(), entries_b);
        std::memcpy(host + e->cta_off, plan->cta_ptr.data(), cta_b);
        std::memcpy(host + e->groups_off, plan->groups.data(), groups_b);
        e->plan_groups[l] = static_cast<int>(plan->groups.size() / 6);
        // one copy for the whole region of the layer (items | entries | per-CTA offsets | groups)
        cudaError_t ce = cudaMemcpyAsync(dev, host, e->groups_off + groups_b, cudaMemcpyHostToDevice, e->meta_stream);
        if (ce == cudaSuccess) ce = cudaEventRecord(slot.table_ready[l], e->meta_stream);
        if (ce == cudaSuccess && l + 1 == e->cfg.layers) {
          ce = cudaEventRecord(slot.uploads_done, e->meta_stream);
          slot.uploads_recorded = ce == cudaSuccess;
        }
        if (ce != cudaSuccess) {
          s = RT_ERR_CUDA;
          last_error_ref() = cudaGetErrorString(ce);
        }
        e->plan_entries[l] = static_cast<int64_t>(plan->entries.size());
        if (l == 0) {
          e->plan_visits = plan->visits;
          e->plan_items = static_cast<int>(plan->items.size());
        }
      }
    }
    {
      std::lock_guard<std::mutex> lk(e->mu);
      if (s != RT_OK) {
        e->worker_status = s;
        e->worker_error = last_error_ref();
        e->layers_recorded = e->cfg.layers;  // release every waiter; they will see the status
      } else {
        e->layers_recorded = l + 1;
      }
    }
    e->cv.notify_all();
    if (s != RT_OK) return;
  }
}

void worker_main(rt_encoder* e) {
  cudaSetDevice(e->device);
  std::unique_lock<std::mutex> lk(e->mu);
  while (true) {
    e->cv.wait(lk, [&] { return e->job_posted || e->worker_exit; });
    if (e->worker_exit) return;
    e->job_posted = false;
    e->worker_busy = true;
    lk.unlock();
    build_batch_metadata(e);
    lk.lock();
    e->worker_busy = false;
    e->cv.notify_all();
  }
}

rt_status wait_layer_table(rt_encoder* e, int layer, cudaStream_t st) {
  auto t0 = std::chrono::steady_clock::now();
  {
    std::unique_lock<std::mutex> lk(e->mu);
    e->cv.wait(lk, [&] { return e->layers_recorded > layer; });
    if (e->worker_status != RT_OK) return fail(e->worker_status, "metadata worker: %s", e->worker_error.c_str());
  }
  e->pre_process_ms += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  RT_CHECK_CUDA(cudaStreamWaitEvent(st, e->cur->table_ready[layer], 0));
  return RT_OK;
}

rt_status ensure_scratch(rt_encoder* e, int tokens) {
  if (tokens <= e->capacity_tokens) return RT_OK;
  const size_t T = tokens, H = e->cfg.hidden, F = e->cfg.ffn;
  RT_CHECK_CUDA(cudaDeviceSynchronize());
  RT_TRY(e->scratch["tmp_qkv_out1"].ensure(T * 3 * H * 2));
  RT_TRY(e->scratch["q_out"].ensure(T * H * 2));
  RT_TRY(e->scratch["k_out"].ensure(T * H * 2));
  RT_TRY(e->scratch["v_out"].ensure(T * H * 2));
  RT_TRY(e->scratch["attention_out"].ensure(T * H * 2));
  RT_TRY(e->scratch["dense_out"].ensure(T * H * 2));
  RT_TRY(e->scratch["attention_output"].ensure(T * H * 2));
  RT_TRY(e->scratch["intermediate"].ensure(T * F * 2));
  e->capacity_tokens = tokens;
  return RT_OK;
}

// attention sub-layer: out = LN(ctx W_o + b_o + input)
rt_status run_attention(rt_encoder* e, int l, const void* input, void* output, cudaStream_t st) {
  const rt_config& c = e->cfg;
  LayerWeights& w = e->layers[l];
  RT_REQUIRE(w.set, RT_ERR_STATE, "layer %d has no weights", l);
  const int T = e->tokens, H = c.hidden, dt = c.dtype;
  void* qkv = e->scratch["tmp_qkv_out1"].p;
  void* q = e->scratch["q_out"].p;
  void* k = e->scratch["k_out"].p;
  void* v = e->scratch["v_out"].p;
  void* ctx = e->scratch["attention_out"].p;
  void* dense = e->scratch["dense_out"].p;
  RT_CHECK_CUDA(cudaStreamWaitEvent(st, e->cur->prefix_ready, 0));
  if (e->fuse_qkv) {
    Span s(e, st, "gemm.qkv");
    const int32_t* block_seq = static_cast<const int32_t*>(e->cur->prefix_dev.p) + e->cur->block_seq_off;
    RT_TRY(rt_gemm_qkv(q, k, v, input, w.qkv_w.p, w.qkv_b.p, block_seq, T, c.heads, H, 0.125f, dt, st));
  } else {
    {
      Span s(e, st, "gemm.qkv");
      RT_TRY(rt_gemm(qkv, input, w.qkv_w.p, nullptr, T, 3 * H, H, RT_EPI_NONE, dt, st));
    }
    Span s(e, st, "add_bias_and_transpose_kernel");
    RT_TRY(rt_qkv_bias_transpose(qkv, w.qkv_b.p, q, k, v, (const int32_t*)e->cur->prefix_dev.p, e->n_seq, e->n_blocks,
                                 c.heads, 0.125f, dt, st));
  }
  RT_TRY(wait_layer_table(e, l, st));
  {
    Span s(e, st, "attention");
    const uint8_t* dev = static_cast<const uint8_t*>(e->cur->meta_dev.p) + static_cast<size_t>(l) * e->region_bytes;
    RT_TRY(launch_sparse_attention(ctx, q, k, v, reinterpret_cast<const AttnItem*>(dev + e->items_off),
                                   reinterpret_cast<const int32_t*>(dev + e->entries_off),
                                   reinterpret_cast<const int32_t*>(dev + e->cta_off), e->attn_ctas, T, c.heads, 1.0f, dt,
                                   st, nullptr,
                                   AttnSplit{reinterpret_cast<const int32_t*>(dev + e->groups_off), e->plan_groups[l],
                                             static_cast<float*>(e->part_o.p), static_cast<float*>(e->part_ml.p)}));
  }
  if (e->fuse_layernorm == 2 && (H == 768 || H == 1024)) {
    Span s(e, st, "gemm.attention_output");
    RT_TRY(rt_gemm_bias_residual_layernorm(output, ctx, w.ao_w.p, w.ao_b.p, input, w.aln_g.p, w.aln_b.p, T, H, H, c.eps,
                                           dt, st));
  } else if (e->fuse_residual) {
    {
      Span s(e, st, "gemm.attention_output");
      RT_TRY(rt_gemm_residual(dense, ctx, w.ao_w.p, w.ao_b.p, input, T, H, H, dt, st));
    }
    Span s(e, st, "add_bias_and_layernorm_kernel");
    RT_TRY(rt_bias_residual_layernorm(output, dense, nullptr, nullptr, w.aln_g.p, w.aln_b.p, T, H, c.eps, dt, st));
  } else {
    {
      Span s(e, st, "gemm.attention_output");
      RT_TRY(rt_gemm(dense, ctx, w.ao_w.p, nullptr, T, H, H, RT_EPI_NONE, dt, st));
    }
    Span s(e, st, "add_bias_and_layernorm_kernel");
    RT_TRY(rt_bias_residual_layernorm(output, dense, w.ao_b.p, input, w.aln_g.p, w.aln_b.p, T, H, c.eps, dt, st));
  }
  return RT_OK;
}

rt_status run_intermediate(rt_encoder* e, int l, const void* input, void* output, cudaStream_t st) {
  const rt_config& c = e->cfg;
  LayerWeights& w = e->layers[l];
  RT_REQUIRE(w.set, RT_ERR_STATE, "layer %d has no weights", l);
  if (e->fuse_gelu) {
    Span s(e, st, "gemm.ffn_up");
    RT_TRY(rt_gemm(output, input, w.up_w.p, w.up_b.p, e->tokens, c.ffn, c.hidden, RT_EPI_BIAS_GELU, c.dtype, st));
  } else {
    {
      Span s(e, st, "gemm.ffn_up");
      RT_TRY(rt_gemm(output, input, w.up_w.p, nullptr, e->tokens, c.ffn, c.hidden, RT_EPI_NONE, c.dtype, st));
    }
    Span s(e, st, "add_bias_act_kernel");
    RT_TRY(rt_bias_gelu(output, w.up_b.p, e->tokens, c.ffn, c.dtype, st));
  }
  return RT_OK;
}

rt_status run_output(rt_encoder* e, int l, const void* ffn, const void* residual, void* out, cudaStream_t st) {
  const rt_config& c = e->cfg;
  LayerWeights& w = e->layers[l];
  RT_REQUIRE(w.set, RT_ERR_STATE, "layer %d has no weights", l);
  void* dense = e->scratch["dense_out"].p;
  if ((e->fuse_layernorm == 2 && (c.hidden == 768 || c.hidden == 1024)) ||
      (e->fuse_layernorm == 1 && c.hidden == 768 && c.ffn >= 2048)) {
    Span s(e, st, "gemm.ffn_down");
    return rt_gemm_bias_residual_layernorm(out, ffn, w.down_w.p, w.down_b.p, residual, w.oln_g.p, w.oln_b.p, e->tokens,
                                           c.hidden, c.ffn, c.eps, c.dtype, st);
  }
  if (e->fuse_residual) {
    {
      Span s(e, st, "gemm.ffn_down");
      RT_TRY(rt_gemm_residual(dense, ffn, w.down_w.p, w.down_b.p, residual, e->tokens, c.hidden, c.ffn, c.dtype, st));
    }
    Span s(e, st, "add_bias_and_layernorm_kernel");
    RT_TRY(rt_bias_residual_layernorm(out, dense, nullptr, nullptr, w.oln_g.p, w.oln_b.p, e->tokens, c.hidden, c.eps,
                                      c.dtype, st));
    return RT_OK;
  }
  {
    Span s(e, st, "gemm.ffn_down");
    RT_TRY(rt_gemm(dense, ffn, w.down_w.p, nullptr, e->tokens, c.hidden, c.ffn, RT_EPI_NONE, c.dtype, st));
  }
  Span s(e, st, "add_bias_and_layernorm_kernel");
  RT_TRY(rt_bias_residual_layernorm(out, dense, w.down_b.p, residual, w.oln_g.p, w.oln_b.p, e->tokens, c.hidden, c.eps,
                                    c.dtype, st));
  return RT_OK;
}

// varlen offsets [n_seq+1] and, behind them, {first token of its sequence, sequence length} of every packed
// block (the fused QKV epilogue's map), written to the slot's pinned buffer and uploaded
rt_status fill_prefix_impl(rt_encoder* e, rt_encoder::Slot& slot, const int32_t* lens, int n_seq, int prefix_ints,
                           int need_ints) {
  RT_TRY(rt_seq_block_prefix(lens, n_seq, e->cfg.block, slot.prefix_pinned));
  slot.block_seq_off = prefix_ints;
  int32_t* bs = slot.prefix_pinned + prefix_ints;
  int t0 = 0, b = 0;
  for (int q = 0; q < n_seq; ++q) {
    for (int i = 0; i < lens[q] / e->cfg.block; ++i, ++b) {
      bs[2 * b] = t0;
      bs[2 * b + 1] = lens[q];
    }
    t0 += lens[q];
  }
  RT_CHECK_CUDA(cudaMemcpyAsync(slot.prefix_dev.p, slot.prefix_pinned, need_ints * sizeof(int32_t),
                                cudaMemcpyHostToDevice, e->meta_stream));
  RT_CHECK_CUDA(cudaEventRecord(slot.prefix_ready, e->meta_stream));
  return RT_OK;
}
#define fill_prefix(e, slot, lens, n_seq, a, b) RT_TRY(fill_prefix_impl(e, slot, lens, n_seq, a, b))

}  // namespace

extern "C" rt_status rt_encoder_create(const rt_config* cfg, rt_encoder** out) {
  RT_REQUIRE(out != nullptr, RT_ERR_INVALID, "encoder_create: null output");
  RT_TRY(check_config(cfg));
  RT_REQUIRE(cfg->layers > 0 && cfg->ffn > 0 && cfg->ffn % 64 == 0, RT_ERR_INVALID,
             "encoder_create: layers > 0 and ffn %% 64 == 0 required");
  RT_REQUIRE(cfg->hidden <= 1024, RT_ERR_UNSUPPORTED, "encoder_create: hidden up to 1024 supported");
  RT_REQUIRE(cfg->dtype == RT_F16 || cfg->dtype == RT_BF16, RT_ERR_INVALID, "encoder_create: unknown dtype");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
    return fail(RT_ERR_CUDA, "encoder_create: no CUDA device (this library has no CPU path)");
  auto* e = new rt_encoder();
  e->cfg = *cfg;
  e->layers.resize(cfg->layers);
  for (int l = 0; l < cfg->layers; ++l) e->layers[l].seed = static_cast<uint32_t>(l);
  e->csr.resize(cfg->layers);
  e->csr_valid.assign(cfg->layers, false);
  e->plan_entries.assign(cfg->layers, 0);
  e->plan_groups.assign(cfg->layers, 0);
  cudaGetDevice(&e->device);
  cudaDeviceGetAttribute(&e->sm_count, cudaDevAttrMultiProcessorCount, e->device);
  e->attn_ctas = 2 * e->sm_count;
  if (cudaStreamCreateWithFlags(&e->meta_stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete e;
    return fail(RT_ERR_CUDA, "encoder_create: cannot create the metadata stream");
  }
  for (auto& slot : e->slots) {
    cudaEventCreateWithFlags(&slot.prefix_ready, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&slot.forward_done, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&slot.uploads_done, cudaEventDisableTiming);
    slot.table_ready.resize(cfg->layers);
    for (auto& ev : slot.table_ready) cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
  }
  e->worker = std::thread(worker_main, e);
  *out = e;
  return RT_OK;
}

extern "C" rt_status rt_encoder_destroy(rt_encoder* e) {
  if (!e) return RT_OK;
  e->join_worker();
  {
    std::lock_guard<std::mutex> lk(e->mu);
    e->worker_exit = true;
  }
  e->cv.notify_all();
  if (e->worker.joinable()) e->worker.join();
  cudaDeviceSynchronize();
  for (auto& l : e->layers)
    for (DevBuf* b : {&l.qkv_w, &l.qkv_b, &l.ao_w, &l.ao_b, &l.aln_g, &l.aln_b, &l.up_w, &l.up_b, &l.down_w, &l.down_b,
                      &l.oln_g, &l.oln_b})
      b->release();
  for (DevBuf* b : {&e->emb_word, &e->emb_pos, &e->emb_type, &e->emb_g, &e->emb_b, &e->ids_dev, &e->pos_dev, &e->part_o,
                    &e->part_ml})
    b->release();
  for (auto& kv : e->scratch) kv.second.release();
  for (auto& slot : e->slots) {
    slot.meta_dev.release();
    slot.prefix_dev.release();
    if (slot.meta_pinned) cudaFreeHost(slot.meta_pinned);
    if (slot.prefix_pinned) cudaFreeHost(slot.prefix_pinned);
    cudaEventDestroy(slot.prefix_ready);
    cudaEventDestroy(slot.forward_done);
    cudaEventDestroy(slot.uploads_done);
    for (auto& ev : slot.table_ready) cudaEventDestroy(ev);
  }
  for (auto& ev : e->timer.pool) cudaEventDestroy(ev);
  for (auto& job : e->jobs) {
    job.ids.release();
    job.out.release();
    if (job.ids_ready) cudaEventDestroy(job.ids_ready);
    if (job.computed) cudaEventDestroy(job.computed);
    if (job.copied) cudaEventDestroy(job.copied);
    if (job.err_host) cudaFreeHost(job.err_host);
  }
  if (e->pipe_stream) cudaStreamDestroy(e->pipe_stream);
  if (e->copy_stream) cudaStreamDestroy(e->copy_stream);
  if (e->in_stream) cudaStreamDestroy(e->in_stream);
  if (e->meta_stream) cudaStreamDestroy(e->meta_stream);
  delete e;
  return RT_OK;
}

extern "C" rt_status rt_encoder_set_layer(rt_encoder* e, int layer, uint32_t table_seed, int in_out_layout,
                                          const void* qkv_w, const void* qkv_b, const void* ao_w, const void* ao_b,
                                          const void* aln_g, const void* aln_b, const void* up_w, const void* up_b,
                                          const void* down_w, const void* down_b, const void* oln_g,
                                          const void* oln_b) {
  RT_REQUIRE(e != nullptr, RT_ERR_INVALID, "set_layer: null encoder");
  RT_REQUIRE(layer >= 0 && layer < e->cfg.layers, RT_ERR_INVALID, "set_layer: layer %d out of range", layer);
  RT_REQUIRE(qkv_w && qkv_b && ao_w && ao_b && aln_g && aln_b && up_w && up_b && down_w && down_b && oln_g && oln_b,
             RT_ERR_INVALID, "set_layer: null weight pointer");
  e->join_worker();
  const int H = e->cfg.hidden, F = e->cfg.ffn;
  LayerWeights& w = e->layers[layer];
  const bool tr = in_out_layout != 0;
  // stored layout is always [out][in]; an [in][out] source (rows_in = in) is transposed
  RT_TRY(copy_or_transpose(w.qkv_w, qkv_w, tr ? H : 3 * H, tr ? 3 * H : H, tr));
  RT_TRY(copy_or_transpose(w.ao_w, ao_w, H, H, tr));
  RT_TRY(copy_or_transpose(w.up_w, up_w, tr ? H : F, tr ? F : H, tr));
  RT_TRY(copy_or_transpose(w.down_w, down_w, tr ? F : H, tr ? H : F, tr));
  RT_TRY(copy_vec(w.qkv_b, qkv_b, 3 * H * elt()));
  RT_TRY(copy_vec(w.ao_b, ao_b, H * elt()));
  RT_TRY(copy_vec(w.aln_g, aln_g, H * elt()));
  RT_TRY(copy_vec(w.aln_b, aln_b, H * elt()));
  RT_TRY(copy_vec(w.up_b, up_b, F * elt()));
  RT_TRY(copy_vec(w.down_b, down_b, H * elt()));
  RT_TRY(copy_vec(w.oln_g, oln_g, H * elt()));
  RT_TRY(copy_vec(w.oln_b, oln_b, H * elt()));
  w.seed = table_seed;
  w.set = true;
  return RT_OK;
}

extern "C" rt_status rt_encoder_set_embeddings(rt_encoder* e, const void* word, const void* pos, const void* type,
                                               const void* ln_g, const void* ln_b) {
  RT_REQUIRE(e && word && pos && type && ln_g && ln_b, RT_ERR_INVALID, "set_embeddings: null pointer");
  const size_t H = e->cfg.hidden;
  RT_TRY(copy_vec(e->emb_word, word, static_cast<size_t>(e->cfg.vocab) * H * 4));
  RT_TRY(copy_vec(e->emb_pos, pos, static_cast<size_t>(e->cfg.max_pos) * H * 4));
  RT_TRY(copy_vec(e->emb_type, type, static_cast<size_t>(e->cfg.type_vocab) * H * 4));
  RT_TRY(copy_vec(e->emb_g, ln_g, H * 4));
  RT_TRY(copy_vec(e->emb_b, ln_b, H * 4));
  e->emb_set = true;
  return RT_OK;
}

extern "C" rt_status rt_encoder_set_option(rt_encoder* e, const char* name, int value) {
  RT_REQUIRE(e && name, RT_ERR_INVALID, "set_option: null pointer");
  if (std::strcmp(name, "fuse_gelu") == 0) {
    e->fuse_gelu = value != 0;
    return RT_OK;
  }
  if (std::strcmp(name, "fuse_qkv") == 0) {
    e->fuse_qkv = value != 0;
    return RT_OK;
  }
  if (std::strcmp(name, "fuse_layernorm") == 0) {
    RT_REQUIRE(value >= 0 && value <= 2, RT_ERR_INVALID, "set_option: fuse_layernorm takes 0, 1 or 2");
    e->fuse_layernorm = value;
    return RT_OK;
  }
  if (std::strcmp(name, "fuse_residual") == 0) {
    e->fuse_residual = value != 0;
    return RT_OK;
  }
  return fail(RT_ERR_INVALID, "set_option: unknown option '%s'", name);
}

extern "C" rt_status rt_encoder_get_option(rt_encoder* e, const char* name, int* value_out) {
  RT_REQUIRE(e && name && value_out, RT_ERR_INVALID, "get_option: null pointer");
  if (std::strcmp(name, "fuse_gelu") == 0) *value_out = e->fuse_gelu;
  else if (std::strcmp(name, "fuse_qkv") == 0) *value_out = e->fuse_qkv;
  else if (std::strcmp(name, "fuse_layernorm") == 0) *value_out = e->fuse_layernorm;
  else if (std::strcmp(name, "fuse_residual") == 0) *value_out = e->fuse_residual;
  else return fail(RT_ERR_INVALID, "get_option: unknown option '%s'", name);
  return RT_OK;
}

extern "C" rt_status rt_encoder_prepare_batch(rt_encoder* e, const int32_t* lens, int n_seq) {
  RT_REQUIRE(e != nullptr, RT_ERR_INVALID, "prepare_batch: null encoder");
  RT_TRY(validate_lengths(e->cfg, lens, n_seq));
  e->join_worker();
  e->prepared = false;
  e->lens.assign(lens, lens + n_seq);
  e->n_seq = n_seq;
  int T = 0;
  for (int s = 0; s < n_seq; ++s) T += lens[s];
  e->tokens = T;
  e->n_blocks = T / e->cfg.block;
  RT_TRY(ensure_scratch(e, T));

  // this batch's slot; its previous user (two batches ago) must have finished on the device
  rt_encoder::Slot& slot = e->slots[e->batch_counter % rt_encoder::kSlots];
  ++e->batch_counter;
  const auto blocked_t0 = std::chrono::steady_clock::now();
  if (slot.forward_recorded) RT_CHECK_CUDA(cudaEventSynchronize(slot.forward_done));
  else if (slot.used) RT_CHECK_CUDA(cudaDeviceSynchronize());  // driven through the per-operator calls
  // this slot's earlier uploads read the pinned memory that is about to be rewritten
  if (slot.uploads_recorded) RT_CHECK_CUDA(cudaEventSynchronize(slot.uploads_done));
  else if (slot.used) RT_CHECK_CUDA(cudaStreamSynchronize(e->meta_stream));
  e->host_blocked_ms += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - blocked_t0).count();
  slot.used = true;
  slot.forward_recorded = false;
  slot.uploads_recorded = false;
  e->cur = &slot;

  // varlen offsets + per-block {first token of the sequence, sequence length}
  const int prefix_ints = ((n_seq + 1 + 7) / 8) * 8;  // keeps the block table 32-byte aligned
  const int need_ints = prefix_ints + 2 * e->n_blocks;

  // per-layer regions, sized by bounds that hold for every table seed
  size_t n_items = 0, n_entries = 0, slots_bound = 0, groups_bound = 0;
  attn_plan_bounds(e->cfg, lens, n_seq, kDefaultSplitEntries, &n_items, &n_entries, &slots_bound, &groups_bound);
  e->items_off = 0;
  e->entries_off = align256(n_items * sizeof(AttnItem));
  e->cta_off = e->entries_off + align256(n_entries * sizeof(int32_t));
  e->groups_off = e->cta_off + align256((e->attn_ctas + 1) * sizeof(int32_t));
  e->region_bytes = e->groups_off + align256(groups_bound * 6 * sizeof(int32_t));
  if (slots_bound * 128 * 64 * sizeof(float) > e->part_o.bytes) {
    RT_CHECK_CUDA(cudaDeviceSynchronize());
    RT_TRY(e->part_o.ensure(slots_bound * 128 * 64 * sizeof(float)));
    RT_TRY(e->part_ml.ensure(slots_bound * 128 * 2 * sizeof(float)));
  }
  // Metadata buffers of ALL slots grow together, at the first batch that needs more: a serving loop
  // that has seen its largest batch once never allocates again, whichever slot a batch lands in.
  const size_t need = e->region_bytes * e->cfg.layers;
  if (need > slot.meta_cap || need_ints > slot.prefix_cap) {
    RT_CHECK_CUDA(cudaDeviceSynchronize());  // the other slots may still be read by queued kernels and uploads
    const size_t meta_cap = std::max(slot.meta_cap, need + need / 4);
    const int prefix_cap = std::max(slot.prefix_cap, std::max(2 * need_ints, 1024));
    for (auto& sl : e->slots) {
      if (sl.meta_cap < meta_cap) {
        if (sl.meta_pinned) cudaFreeHost(sl.meta_pinned);
        sl.meta_pinned = nullptr;
        sl.meta_cap = 0;
        RT_CHECK_CUDA(cudaMallocHost(&sl.meta_pinned, meta_cap));
        RT_TRY(sl.meta_dev.ensure(meta_cap));
        sl.meta_cap = meta_cap;
      }
      if (sl.prefix_cap < prefix_cap) {
        if (sl.prefix_pinned) cudaFreeHost(sl.prefix_pinned);
        sl.prefix_pinned = nullptr;
        sl.prefix_cap = 0;
        RT_CHECK_CUDA(cudaMallocHost(&sl.prefix_pinned, prefix_cap * sizeof(int32_t)));
        RT_TRY(sl.prefix_dev.ensure(prefix_cap * sizeof(int32_t)));
        sl.prefix_cap = prefix_cap;
      }
    }
  }
  fill_prefix(e, slot, lens, n_seq, prefix_ints, need_ints);
  e->pre_process_ms = 0.0;
  e->csr_valid.assign(e->cfg.layers, false);
  {
    std::lock_guard<std::mutex> lk(e->mu);
    e->layers_recorded = 0;
    e->worker_status = RT_OK;
    e->worker_error.clear();
    e->job_posted = true;
  }
  e->cv.notify_all();
  e->prepared = true;
  return RT_OK;
}

extern "C" rt_status rt_encoder_attention(rt_encoder* e, int layer, const void* input, void* output, void* stream) {
  RT_REQUIRE(e && input && output, RT_ERR_INVALID, "attention: null pointer");
  RT_REQUIRE(e->prepared, RT_ERR_STATE, "attention: call rt_encoder_prepare_batch first");
  RT_REQUIRE(layer >= 0 && layer < e->cfg.layers, RT_ERR_INVALID, "attention: layer out of range");
  return run_attention(e, layer, input, output, static_cast<cudaStream_t>(stream));
}

extern "C" rt_status rt_encoder_intermediate(rt_encoder* e, int layer, const void* input, void* output, void* stream) {
  RT_REQUIRE(e && input && output, RT_ERR_INVALID, "intermediate: null pointer");
  RT_REQUIRE(e->prepared, RT_ERR_STATE, "intermediate: call rt_encoder_prepare_batch first");
  RT_REQUIRE(layer >= 0 && layer < e->cfg.layers, RT_ERR_INVALID, "intermediate: layer out of range");
  return run_intermediate(e, layer, input, output, static_cast<cudaStream_t>(stream));
}

extern "C" rt_status rt_encoder_output(rt_encoder* e, int layer, const void* ffn, const void* residual, void* out,
                                       void* stream) {
  RT_REQUIRE(e && ffn && residual && out, RT_ERR_INVALID, "output: null pointer");
  RT_REQUIRE(e->prepared, RT_ERR_STATE, "output: call rt_encoder_prepare_batch first");
  RT_REQUIRE(layer >= 0 && layer < e->cfg.layers, RT_ERR_INVALID, "output: layer out of range");
  return run_output(e, layer, ffn, residual, out, static_cast<cudaStream_t>(stream));
}

namespace {
rt_status begin_forward(rt_encoder* e, cudaStream_t st) {
  if (e->timing) e->timer.reset();
  RT_CHECK_CUDA(cudaStreamWaitEvent(st, e->cur->prefix_ready, 0));
  return RT_OK;
}
rt_status end_forward(rt_encoder* e, cudaStream_t st) {
  RT_CHECK_CUDA(cudaEventRecord(e->cur->forward_done, st));
  e->cur->forward_recorded = true;
  return RT_OK;
}
rt_status run_layers(rt_encoder* e, void* hidden, int l0, int l1, cudaStream_t st) {
  void* attn_out = e->scratch["attention_output"].p;
  void* ffn = e->scratch["intermediate"].p;
  for (int l = l0; l < l1; ++l) {
    RT_TRY(run_attention(e, l, hidden, attn_out, st));
    RT_TRY(run_intermediate(e, l, attn_out, ffn, st));
    RT_TRY(run_output(e, l, ffn, attn_out, hidden, st));
  }
  return RT_OK;
}
}  // namespace

extern "C" rt_status rt_encoder_forward_hidden(rt_encoder* e, void* hidden, int layer_begin, int layer_end,
                                               void* stream) {
  RT_REQUIRE(e && hidden, RT_ERR_INVALID, "forward_hidden: null pointer");
  RT_REQUIRE(e->prepared, RT_ERR_STATE, "forward_hidden: call rt_encoder_prepare_batch first");
  RT_REQUIRE(0 <= layer_begin && layer_begin <= layer_end && layer_end <= e->cfg.layers, RT_ERR_INVALID,
             "forward_hidden: bad layer range [%d, %d)", layer_begin, layer_end);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  RT_TRY(begin_forward(e, st));
  RT_TRY(run_layers(e, hidden, layer_begin, layer_end, st));
  return end_forward(e, st);
}

extern "C" rt_status rt_encoder_forward_ids(rt_encoder* e, const int32_t* ids, const int32_t* pos_ids,
                                            const int32_t* type_ids, void* out, void* stream) {
  RT_REQUIRE(e && ids && out, RT_ERR_INVALID, "forward_ids: null pointer");
  RT_REQUIRE(e->prepared, RT_ERR_STATE, "forward_ids: call rt_encoder_prepare_batch first");
  RT_REQUIRE(e->emb_set, RT_ERR_STATE, "forward_ids: embeddings not set");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  RT_TRY(begin_forward(e, st));
  if (!pos_ids) {
    RT_TRY(e->pos_dev.ensure(static_cast<size_t>(e->tokens) * sizeof(int32_t)));
    position_ids_kernel<<<(e->tokens + 255) / 256, 256, 0, st>>>((int32_t*)e->pos_dev.p,
                                                                 (const int32_t*)e->cur->prefix_dev.p, e->n_seq,
                                                                 e->tokens);
    count_launch();
    RT_CHECK_CUDA(cudaGetLastError());
    pos_ids = (const int32_t*)e->pos_dev.p;
  }
  {
    Span s(e, st, "embeddings");
    RT_TRY(rt_embeddings(out, ids, pos_ids, type_ids, e->emb_word.p, e->emb_pos.p, e->emb_type.p, e->emb_g.p,
                         e->emb_b.p, e->tokens, e->cfg.hidden, e->cfg.eps, e->cfg.dtype, st));
  }
  RT_TRY(run_layers(e, out, 0, e->cfg.layers, st));
  return end_forward(e, st);
}

extern "C" rt_status rt_encoder_submit_host(rt_encoder* e, const int32_t* lens, int n_seq, const int32_t* ids_host,
                                            void* out_host, uint64_t* ticket) {
  RT_REQUIRE(e && ids_host && out_host && ticket, RT_ERR_INVALID, "submit_host: null pointer");
  if (!e->pipe_stream) {
    RT_CHECK_CUDA(cudaStreamCreateWithFlags(&e->pipe_stream, cudaStreamNonBlocking));
    RT_CHECK_CUDA(cudaStreamCreateWithFlags(&e->copy_stream, cudaStreamNonBlocking));
    RT_CHECK_CUDA(cudaStreamCreateWithFlags(&e->in_stream, cudaStreamNonBlocking));
    for (auto& job : e->jobs) {
      RT_CHECK_CUDA(cudaEventCreateWithFlags(&job.ids_ready, cudaEventDisableTiming));
      RT_CHECK_CUDA(cudaEventCreateWithFlags(&job.computed, cudaEventDisableTiming));
      RT_CHECK_CUDA(cudaEventCreateWithFlags(&job.copied, cudaEventDisableTiming));
      RT_CHECK_CUDA(cudaMallocHost(&job.err_host, sizeof(int)));
      *job.err_host = 0;
    }
  }
  rt_encoder::HostJob& job = e->jobs[e->next_ticket & 1];
  if (job.busy) {  // at most two batches in flight: this buffer's previous batch must have reached the host
    const auto t0 = std::chrono::steady_clock::now();
    RT_CHECK_CUDA(cudaEventSynchronize(job.copied));
    e->host_blocked_ms += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    job.busy = false;
  }
  // a forward issued through the device-buffer entry points on another stream shares the scratch
  rt_encoder::Slot* prev = e->cur;
  RT_TRY(rt_encoder_prepare_batch(e, lens, n_seq));
  if (prev && prev->forward_recorded) RT_CHECK_CUDA(cudaStreamWaitEvent(e->pipe_stream, prev->forward_done, 0));
  const size_t T = e->tokens;
  RT_TRY(job.ids.ensure(T * sizeof(int32_t)));
  const size_t out_bytes = T * e->cfg.hidden * 2;
  RT_TRY(job.out.ensure(out_bytes));
  cudaStream_t st = e->pipe_stream;
  // this buffer's previous batch has reached the host (waited for above), so its ids are long consumed
  RT_CHECK_CUDA(cudaMemcpyAsync(job.ids.p, ids_host, T * sizeof(int32_t), cudaMemcpyHostToDevice, e->in_stream));
  RT_CHECK_CUDA(cudaEventRecord(job.ids_ready, e->in_stream));
  RT_CHECK_CUDA(cudaStreamWaitEvent(st, job.ids_ready, 0));
  RT_TRY(rt_encoder_forward_ids(e, (const int32_t*)job.ids.p, nullptr, nullptr, job.out.p, st));
  RT_CHECK_CUDA(cudaEventRecord(job.computed, st));
  RT_CHECK_CUDA(cudaStreamWaitEvent(e->copy_stream, job.computed, 0));
  RT_CHECK_CUDA(cudaMemcpyAsync(out_host, job.out.p, out_bytes, cudaMemcpyDeviceToHost, e->copy_stream));
  if (int* err = device_error_word())
    RT_CHECK_CUDA(cudaMemcpyAsync(job.err_host, err, sizeof(int), cudaMemcpyDeviceToHost, e->copy_stream));
  RT_CHECK_CUDA(cudaEventRecord(job.copied, e->copy_stream));
  job.busy = true;
  job.ticket = e->next_ticket;
  *ticket = e->next_ticket++;
  return RT_OK;
}

extern "C" rt_status rt_encoder_wait_host(rt_encoder* e, uint64_t ticket) {
  RT_REQUIRE(e != nullptr, RT_ERR_INVALID, "wait_host: null encoder");
  RT_REQUIRE(ticket >= 1 && ticket < e->next_ticket, RT_ERR_INVALID, "wait_host: unknown ticket %llu",
             static_cast<unsigned long long>(ticket));
  for (auto& job : e->jobs) {
    if (!job.busy || job.ticket != ticket) continue;
    RT_CHECK_CUDA(cudaEventSynchronize(job.copied));
    job.busy = false;
    if (*job.err_host != 0)  // rt_check_device() reports the site and clears the word
      return fail(RT_ERR_DEVICE_WAIT, "wait_host: a bounded device-side wait ran out at site %d", *job.err_host);
    return RT_OK;
  }
  return RT_OK;  // already waited for (by a later submit that needed its buffer)
}

extern "C" rt_status rt_encoder_forward_host(rt_encoder* e, const int32_t* lens, int n_seq, const int32_t* ids_host,
                                             void* out_host) {
  uint64_t ticket = 0;
  RT_TRY(rt_encoder_submit_host(e, lens, n_seq, ids_host, out_host, &ticket));
  return rt_encoder_wait_host(e, ticket);
}

extern "C" rt_status rt_encoder_get_table(rt_encoder* e, int layer, const int32_t** kv_ptr, const int32_t** kv_idx,
                                          int64_t* visits) {
  RT_REQUIRE(e != nullptr, RT_ERR_INVALID, "get_table: null encoder");
  RT_REQUIRE(e->prepared, RT_ERR_STATE, "get_table: call rt_encoder_prepare_batch first");
  RT_REQUIRE(layer >= 0 && layer < e->cfg.layers, RT_ERR_INVALID, "get_table: layer out of range");
  e->join_worker();
  if (e->worker_status != RT_OK) return fail(e->worker_status, "metadata worker: %s", e->worker_error.c_str());
  if (!e->csr_valid[layer]) {
    RT_TRY(build_block_csr(e->cfg, e->layers[layer].seed, e->lens.data(), e->n_seq, e->csr[layer], &e->table_cache));
    e->csr_valid[layer] = true;
  }
  if (kv_ptr) *kv_ptr = e->csr[layer].kv_ptr.data();
  if (kv_idx) *kv_idx = e->csr[layer].kv_idx.data();
  if (visits) *visits = e->csr[layer].visits;
  return RT_OK;
}

extern "C" rt_status rt_encoder_plan_stats(rt_encoder* e, int layer, int64_t* entries, int64_t* visits, int32_t* items) {
  RT_REQUIRE(e != nullptr && e->prepared, RT_ERR_STATE, "plan_stats: call rt_encoder_prepare_batch first");
  RT_REQUIRE(layer >= 0 && layer < e->cfg.layers, RT_ERR_INVALID, "plan_stats: layer out of range");
  e->join_worker();
  if (entries) *entries = e->plan_entries[layer];
  if (visits) *visits = e->plan_visits;
  if (items) *items = e->plan_items;
  return RT_OK;
}

extern "C" rt_status rt_encoder_get_scratch(rt_encoder* e, const char* name, void** ptr, size_t* bytes) {
  RT_REQUIRE(e && name, RT_ERR_INVALID, "get_scratch: null pointer");
  auto it = e->scratch.find(name);
  if (it == e->scratch.end() || !it->second.p) return fail(RT_ERR_INVALID, "no exists tensor '%s'", name);
  if (ptr) *ptr = it->second.p;
  if (bytes) *bytes = it->second.bytes;
  return RT_OK;
}

extern "C" rt_status rt_encoder_enable_timing(rt_encoder* e, int on) {
  RT_REQUIRE(e != nullptr, RT_ERR_INVALID, "enable_timing: null encoder");
  e->timing = on != 0;
  e->timer.reset();
  return RT_OK;
}

extern "C" rt_status rt_encoder_get_timing(rt_encoder* e, const char* key, float* ms_out) {
  RT_REQUIRE(e && key && ms_out, RT_ERR_INVALID, "get_timing: null pointer");
  if (std::strcmp(key, "pre_process") == 0) {
    *ms_out = static_cast<float>(e->pre_process_ms);
    return RT_OK;
  }
  if (std::strcmp(key, "host_blocked") == 0) {  // cumulative since the encoder was created
    *ms_out = static_cast<float>(e->host_blocked_ms);
    return RT_OK;
  }
  RT_CHECK_CUDA(cudaDeviceSynchronize());
  float total = 0.f;
  const size_t klen = std::strlen(key);
  for (auto& s : e->timer.spans) {
    // "gemm" also collects "gemm.qkv", "gemm.ffn_up", ...
    const bool sub = s.first.size() > klen && s.first.compare(0, klen, key) == 0 && s.first[klen] == '.';
    if (s.first != key && !sub) continue;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, s.second.first, s.second.second) == cudaSuccess) total += ms;
  }
  *ms_out = total;
  return RT_OK;
}

extern "C" rt_status rt_encoder_kernel_launches(rt_encoder* e, int64_t* launches_out) {
  RT_REQUIRE(launches_out != nullptr, RT_ERR_INVALID, "kernel_launches: null output");
  (void)e;
  *launches_out = launch_counter().load();
  return RT_OK;
}
