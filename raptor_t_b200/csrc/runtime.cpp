// Process-wide state of the library: last-error string, launch counter, the
// per-device error word, and the metadata entry points of the C ABI.
#include <cuda_runtime.h>

#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

#include <set>
#include <utility>

#include "device_error.h"
#include "launch.h"
#include "launch_count.h"
#include "metadata.h"

namespace rt {

std::string& last_error_ref() {
  static thread_local std::string e;
  return e;
}

std::atomic<int64_t>& launch_counter() {
  static std::atomic<int64_t> c{0};
  return c;
}

namespace {
std::mutex g_attr_mu;
std::set<std::pair<const void*, int>> g_attr_done;  // (kernel, device) pairs whose attributes are set
}  // namespace

rt_status ensure_kernel_smem(const void* func, int smem_bytes, bool max_carveout) {
  int dev = 0;
  RT_CHECK_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_attr_mu);
  if (g_attr_done.count({func, dev})) return RT_OK;
  RT_CHECK_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  if (max_carveout)
    RT_CHECK_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributePreferredSharedMemoryCarveout,
                                       cudaSharedmemCarveoutMaxShared));
  g_attr_done.insert({func, dev});
  return RT_OK;
}

namespace {
std::mutex g_err_mu;
int* g_err_words[64] = {nullptr};
}  // namespace

int* device_error_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_err_mu);
  if (!g_err_words[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    if (cudaMemset(p, 0, sizeof(int)) != cudaSuccess) return nullptr;
    g_err_words[dev] = p;
  }
  return g_err_words[dev];
}

rt_status check_device_error(const char* what) {
  RT_CHECK_CUDA(cudaDeviceSynchronize());
  int dev = 0;
  RT_CHECK_CUDA(cudaGetDevice(&dev));
  int* w = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_err_mu);
    if (dev >= 0 && dev < 64) w = g_err_words[dev];
  }
  if (!w) return RT_OK;
  int h = 0;
  RT_CHECK_CUDA(cudaMemcpy(&h, w, sizeof(int), cudaMemcpyDeviceToHost));
  if (h != 0) {
    cudaMemset(w, 0, sizeof(int));
    return fail(RT_ERR_DEVICE_WAIT, "%s: a bounded device-side wait ran out at site %d", what, h);
  }
  return RT_OK;
}

}  // namespace rt

using namespace rt;

extern "C" const char* rt_last_error(void) { return last_error_ref().c_str(); }
extern "C" int rt_version(void) { return 100; }

extern "C" rt_status rt_check_device(void) { return check_device_error("device check"); }
extern "C" int64_t rt_kernel_launches(void) { return launch_counter().load(); }

extern "C" rt_status rt_rand_block_table(uint32_t seed, int heads, int n_blocks, int num_rand, int max_pos, int block,
                                         int32_t* out_host) {
  RT_REQUIRE(out_host != nullptr, RT_ERR_INVALID, "rand_block_table: null output");
  std::vector<int32_t> t;
  RT_TRY(rand_block_table(seed, heads, n_blocks, num_rand, max_pos, block, t));
  std::memcpy(out_host, t.data(), t.size() * sizeof(int32_t));
  return RT_OK;
}

static rt_status check_cfg(const rt_config* cfg) {
  RT_REQUIRE(cfg != nullptr, RT_ERR_INVALID, "null config");
  RT_REQUIRE(cfg->block == 64, RT_ERR_UNSUPPORTED, "block size must be 64 (got %d)", cfg->block);
  RT_REQUIRE(cfg->heads > 0 && cfg->hidden == cfg->heads * 64, RT_ERR_UNSUPPORTED,
             "hidden must be heads*64 (got hidden=%d heads=%d)", cfg->hidden, cfg->heads);
  RT_REQUIRE(cfg->pattern == RT_PATTERN_BIGBIRD || cfg->pattern == RT_PATTERN_BAND, RT_ERR_INVALID,
             "unknown pattern %d", cfg->pattern);
  RT_REQUIRE(cfg->pattern != RT_PATTERN_BIGBIRD || (cfg->num_rand >= 1 && cfg->num_rand <= 8), RT_ERR_UNSUPPORTED,
             "num_rand must be in 1..8");
  RT_REQUIRE(cfg->pattern != RT_PATTERN_BAND || cfg->band_half >= 0, RT_ERR_INVALID, "band_half must be >= 0");
  RT_REQUIRE(cfg->max_pos > 0 && cfg->max_pos % 64 == 0, RT_ERR_INVALID, "max_pos must be a multiple of 64");
  return RT_OK;
}

namespace rt {
rt_status check_config(const rt_config* cfg) { return check_cfg(cfg); }
}

extern "C" rt_status rt_count_visits(const rt_config* cfg, const int32_t* lens, int n_seq, int64_t* visits_out) {
  RT_TRY(check_cfg(cfg));
  RT_REQUIRE(visits_out != nullptr, RT_ERR_INVALID, "count_visits: null output");
  RT_TRY(validate_lengths(*cfg, lens, n_seq));
  std::vector<std::vector<int32_t>> lists;
  std::vector<int32_t> zeros;
  int64_t v = 0;
  for (int s = 0; s < n_seq; ++s) {
    const int L = lens[s] / cfg->block;
    zeros.assign(static_cast<size_t>(L) * (cfg->num_rand > 0 ? cfg->num_rand : 1), 0);
    kv_block_lists(*cfg, L, zeros.data(), lists);
    for (auto& l : lists) v += static_cast<int64_t>(l.size());
  }
  *visits_out = v;
  return RT_OK;
}

extern "C" rt_status rt_build_block_csr(const rt_config* cfg, uint32_t layer_seed, const int32_t* lens, int n_seq,
                                        int32_t* kv_ptr_host, int32_t* kv_idx_host) {
  RT_TRY(check_cfg(cfg));
  RT_REQUIRE(kv_ptr_host && kv_idx_host, RT_ERR_INVALID, "build_block_csr: null output");
  BlockCsr csr;
  RT_TRY(build_block_csr(*cfg, layer_seed, lens, n_seq, csr, nullptr));
  std::memcpy(kv_ptr_host, csr.kv_ptr.data(), csr.kv_ptr.size() * sizeof(int32_t));
  std::memcpy(kv_idx_host, csr.kv_idx.data(), csr.kv_idx.size() * sizeof(int32_t));
  return RT_OK;
}

extern "C" rt_status rt_seq_block_prefix(const int32_t* lens, int n_seq, int block, int32_t* out_host) {
  RT_REQUIRE(lens && out_host && n_seq > 0 && block > 0, RT_ERR_INVALID, "seq_block_prefix: bad arguments");
  out_host[0] = 0;
  for (int s = 0; s < n_seq; ++s) {
    RT_REQUIRE(lens[s] > 0 && lens[s] % block == 0, RT_ERR_INVALID,
               "sequence %d: length %d is not a positive multiple of the block size %d", s, lens[s], block);
    out_host[s + 1] = out_host[s] + lens[s] / block;
  }
  return RT_OK;
}

extern "C" rt_status rt_lpt_partition(const int32_t* cost, int n_qblocks, const int32_t* seq_prefix, int n_seq,
                                      int n_parts, int heads, int32_t* offsets_host, int32_t* ids_host) {
  RT_REQUIRE(cost && seq_prefix && offsets_host && ids_host, RT_ERR_INVALID, "lpt_partition: null pointer");
  RT_REQUIRE(n_qblocks >= 0 && n_seq > 0 && n_parts > 0 && heads > 0, RT_ERR_INVALID, "lpt_partition: bad sizes");
  RT_REQUIRE(seq_prefix[n_seq] == n_qblocks, RT_ERR_INVALID, "lpt_partition: prefix does not cover the batch");
  std::vector<int32_t> off, ids;
  lpt_partition(cost, n_qblocks, seq_prefix, n_seq, n_parts, heads, off, ids);
  std::memcpy(offsets_host, off.data(), off.size() * sizeof(int32_t));
  std::memcpy(ids_host, ids.data(), ids.size() * sizeof(int32_t));
  return RT_OK;
}

extern "C" rt_status rt_binpack_sequences(const double* cost, int n_seq, int n_bins, int32_t* bin_of_seq_host) {
  RT_REQUIRE(cost && bin_of_seq_host && n_seq > 0 && n_bins > 0, RT_ERR_INVALID, "binpack: bad arguments");
  binpack_sequences(cost, n_seq, n_bins, bin_of_seq_host);
  return RT_OK;
}

extern "C" rt_status rt_attn_plan_bounds(const rt_config* cfg, const int32_t* lens, int n_seq, int split_entries,
                                         int64_t* items, int64_t* entries, int64_t* slots, int64_t* groups) {
  RT_TRY(check_cfg(cfg));
  RT_REQUIRE(items && entries && slots && groups, RT_ERR_INVALID, "attn_plan_bounds: null output");
  RT_TRY(validate_lengths(*cfg, lens, n_seq));
  size_t a = 0, b = 0, c = 0, d = 0;
  attn_plan_bounds(*cfg, lens, n_seq, split_entries < 0 ? kDefaultSplitEntries : split_entries, &a, &b, &c, &d);
  *items = static_cast<int64_t>(a);
  *entries = static_cast<int64_t>(b);
  *slots = static_cast<int64_t>(c);
  *groups = static_cast<int64_t>(d);
  return RT_OK;
}

// Host-only construction of the attention work list (no GPU): via the CSR table
// (use_templates = 0) or via the cached per-sequence templates the encoder uses
// (use_templates = 1).  items_out holds 8 int32 per item in AttnItem field order.
extern "C" rt_status rt_attn_plan_build_host(const rt_config* cfg, uint32_t layer_seed, const int32_t* lens, int n_seq,
                                             int n_ctas, int use_templates, int32_t* items_out, int64_t items_cap,
                                             int32_t* entries_out, int64_t entries_cap, int32_t* cta_ptr_out,
                                             int64_t* n_items, int64_t* n_entries, int64_t* visits) {
  RT_TRY(check_cfg(cfg));
  RT_REQUIRE(n_items && n_entries && visits, RT_ERR_INVALID, "attn_plan_build_host: null counters");
  RT_TRY(validate_lengths(*cfg, lens, n_seq));
  AttnPlanHost plan;
  TableCache tables;
  if (use_templates) {
    TemplateCache cache;
    auto templates_for = [&](uint32_t seed_of_layer, std::vector<const SeqTemplate*>& tmpl) -> rt_status {
      tmpl.resize(n_seq);
      for (int q = 0; q < n_seq; ++q) {
        const int L = lens[q] / cfg->block;
        const uint32_t seed = uses_random_table(*cfg, L) ? seed_of_layer : 0xffffffffu;
        auto key = std::make_pair(seed, L);
        auto it = cache.find(key);
        if (it == cache.end()) {
          SeqTemplate t;
          RT_TRY(build_seq_template(*cfg, seed, L, &tables, t));
          it = cache.emplace(key, std::move(t)).first;
        }
        tmpl[q] = &it->second;
      }
      return RT_OK;
    };
    std::vector<const SeqTemplate*> tmpl;
    if (use_templates == 2) {
      // the encoder's path for layers after the first: skeleton from another seed's lists, entries refilled
      PlanSkeleton skel;
      AttnPlanHost base;
      RT_TRY(templates_for(layer_seed + 1, tmpl));
      RT_TRY(assemble_attn_plan(*cfg, lens, n_seq, tmpl.data(), n_ctas, base, kDefaultSplitEntries, &skel));
      RT_TRY(templates_for(layer_seed, tmpl));
      RT_TRY(refill_attn_plan(skel, base, tmpl.data(), plan));
    } else {
      RT_TRY(templates_for(layer_seed, tmpl));
      RT_TRY(assemble_attn_plan(*cfg, lens, n_seq, tmpl.data(), n_ctas, plan));
    }
  } else {
    BlockCsr csr;
    RT_TRY(build_block_csr(*cfg, layer_seed, lens, n_seq, csr, &tables));
    RT_TRY(build_attn_plan(*cfg, lens, n_seq, csr.kv_ptr.data(), csr.kv_idx.data(), csr.visits, n_ctas, plan));
  }
  *n_items = static_cast<int64_t>(plan.items.size());
  *n_entries = static_cast<int64_t>(plan.entries.size());
  *visits = plan.visits;
  if (items_out) {
    RT_REQUIRE(items_cap >= *n_items && entries_cap >= *n_entries && entries_out && cta_ptr_out, RT_ERR_INVALID,
               "attn_plan_build_host: output buffers too small");
    static_assert(sizeof(AttnItem) == 8 * sizeof(int32_t), "AttnItem layout");
    std::memcpy(items_out, plan.items.data(), plan.items.size() * sizeof(AttnItem));
    std::memcpy(entries_out, plan.entries.data(), plan.entries.size() * sizeof(int32_t));
    std::memcpy(cta_ptr_out, plan.cta_ptr.data(), plan.cta_ptr.size() * sizeof(int32_t));
  }
  return RT_OK;
}
