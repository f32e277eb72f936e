// Host-side metadata of the block-sparse encoder: random-block tables (bit-exact
// with numpy's legacy RandomState, which the reference's validation model uses),
// CSR block lists, varlen offsets, work partitions and the attention work list.
#pragma once
#include <cstdint>
#include <map>
#include <utility>
#include <vector>

#include "common.h"

namespace rt {

// MT19937 with numpy's legacy seeding, masked-rejection bounded integers and
// Fisher-Yates shuffle (numpy.random.seed / numpy.random.permutation).
class NumpyLegacyRng {
 public:
  void seed(uint32_t s);
  uint32_t next_u32();
  uint32_t interval(uint32_t max_inclusive);
  void shuffle(int32_t* a, int n);

 private:
  uint32_t key_[624];
  int pos_ = 624;
};

// out: [heads][n_blocks-2][r].  Returns RT_ERR_UNSUPPORTED for lengths the
// validation model itself cannot run (ids beyond the sequence).
rt_status rand_block_table(uint32_t seed, int heads, int n_blocks, int r, int max_pos, int block,
                           std::vector<int32_t>& out);

// Key/value block lists of all query blocks of one (sequence, head); `rand`
// points at this head's [n_blocks-2][r] slice (or null for dense / band).
void kv_block_lists(const rt_config& cfg, int n_blocks, const int32_t* rand_head,
                    std::vector<std::vector<int32_t>>& lists);

inline bool uses_random_table(const rt_config& cfg, int n_blocks) {
  return cfg.pattern == RT_PATTERN_BIGBIRD && n_blocks > 5 + 2 * cfg.num_rand;
}

struct BlockCsr {
  std::vector<int32_t> kv_ptr;  // [N+1]
  std::vector<int32_t> kv_idx;  // [heads][visits]
  int64_t visits = 0;
};

// Tables are pure functions of (seed, n_blocks); the cache keeps them across batches.
using TableCache = std::map<std::pair<uint32_t, int>, std::vector<int32_t>>;

rt_status build_block_csr(const rt_config& cfg, uint32_t layer_seed, const int32_t* lens_tokens, int n_seq,
                          BlockCsr& out, TableCache* cache);

rt_status validate_lengths(const rt_config& cfg, const int32_t* lens_tokens, int n_seq);

void lpt_partition(const int32_t* cost, int n_qblocks, const int32_t* seq_prefix, int n_seq, int n_parts,
                   int heads, std::vector<int32_t>& offsets, std::vector<int32_t>& ids);

void binpack_sequences(const double* cost, int n_seq, int n_bins, int32_t* bin_of_seq);

// ---- attention work list ---------------------------------------------------
struct AttnItem {
  int32_t q_row0;     // row of query block A in the head-major [T*heads][64] view
  int32_t q_row1;     // row of query block B (== q_row0 when the item has one block)
  int32_t kv_row0;    // row of key/value block 0 of this (sequence, head)
  int32_t entry_off;  // first entry in the entry array
  int32_t n_entries;
  int32_t out_tok0;   // first token (packed) of query block A
  int32_t out_tok1;   // first token of query block B, or -1
  int32_t head;       // bits 0-7: head; bits 8-31: 1 + partial-result slot when the item is one part of a split list
};

struct AttnPlanHost {
  std::vector<AttnItem> items;     // ordered by CTA
  std::vector<int32_t> entries;    // (local block id << 2) | mask; mask bit0: block A uses it, bit1: block B
  std::vector<int32_t> cta_ptr;    // [n_ctas+1]
  // Long lists (the global query blocks attend to every block) are cut into parts of at most
  // `split` entries; every part is a work item that leaves an un-normalised partial result
  // (fp32 output tile + row max + row sum) in scratch slot, and a merge kernel combines the
  // parts of a group.  groups: 6 int32 each {first_slot, n_parts, out_tok0, out_tok1, head, 0}.
  std::vector<int32_t> groups;
  int n_slots = 0;
  int64_t visits = 0;              // useful (query block, key block) pairs, all heads
  int total_tokens = 0;
  int heads = 0;
};

// split_entries: lists longer than this are cut into parts (0 = never split).
constexpr int kDefaultSplitEntries = 24;
rt_status build_attn_plan(const rt_config& cfg, const int32_t* lens_tokens, int n_seq, const int32_t* kv_ptr,
                          const int32_t* kv_idx, int64_t visits_per_head, int n_ctas, AttnPlanHost& out,
                          int split_entries = kDefaultSplitEntries);

// Work-list template of ONE sequence of n_blocks blocks under one table seed, all heads:
// the query-block pairs and their merged, masked key/value lists with sequence-local
// block ids.  A pure function of (seed, n_blocks), so it is cached across batches; a
// batch's work list is assembled from the templates of its sequences.
struct SeqTemplate {
  int n_blocks = 0;
  int n_pairs = 0;                  // items per head
  std::vector<int32_t> qa, qb;      // [n_pairs] query blocks of a pair (qb = -1: single)
  std::vector<int32_t> item_off;    // [heads * n_pairs + 1] offsets into ent
  std::vector<int32_t> ent;         // (local block id << 2) | mask
  int64_t visits = 0;               // useful (query block, key block) pairs, all heads
};
using TemplateCache = std::map<std::pair<uint32_t, int>, SeqTemplate>;

rt_status build_seq_template(const rt_config& cfg, uint32_t seed, int n_blocks, TableCache* tables, SeqTemplate& out);

// Where every item of an assembled work list came from, so that the list of another layer of
// the same batch (same lengths, another table seed) is a refill instead of a new assembly: the
// query-block pairs, the cuts of long lists and the assignment of items to CTAs depend on the
// list lengths, which differ between layers only where two random blocks happen to coincide.
struct PlanSkeleton {
  struct Src {
    int32_t seq;        // sequence of the batch
    int32_t tmpl_item;  // item index inside that sequence's template (head * n_pairs + pair)
    int32_t part_off;   // offset inside the template item's list
    int32_t part_len;   // -1: the whole list, else the length of this part of a split list
  };
  std::vector<Src> src;  // one per emitted item, in emission (CTA) order
};

// Assemble the batch work list from per-sequence templates (templates[s] for sequence s)
// and assign items to CTAs (longest processing time first).  skel (optional) records the
// provenance of every item for refill_attn_plan.
rt_status assemble_attn_plan(const rt_config& cfg, const int32_t* lens_tokens, int n_seq,
                             const SeqTemplate* const* templates, int n_ctas, AttnPlanHost& out,
                             int split_entries = kDefaultSplitEntries, PlanSkeleton* skel = nullptr);

// The work list of another layer of the same batch: items, CTA assignment and cuts of `base`
// (assembled with `skel`), list entries from that layer's templates.
rt_status refill_attn_plan(const PlanSkeleton& skel, const AttnPlanHost& base, const SeqTemplate* const* templates,
                           AttnPlanHost& out);

// Upper bounds of a batch's work-list sizes for any table seed (buffers are sized before the
// tables exist): work items, list entries, partial-result slots and groups of split lists.
void attn_plan_bounds(const rt_config& cfg, const int32_t* lens_tokens, int n_seq, int split_entries, size_t* items,
                      size_t* entries, size_t* slots, size_t* groups);

}  // namespace rt
