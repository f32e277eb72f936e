// Host metadata: see metadata.h.  The random-block tables follow the reference's
// validation model python/modeling_big_bird.py (table branch :573-600, "old plan"
// :1072-1125, with-head plan :1127-1314) and reproduce numpy's legacy RNG stream.
#include "metadata.h"

#include <algorithm>
#include <numeric>
#include <queue>

namespace rt {

// ---------------------------------------------------------------------------
// numpy legacy RandomState
// ---------------------------------------------------------------------------
void NumpyLegacyRng::seed(uint32_t s) {
  for (int i = 0; i < 624; ++i) {
    key_[i] = s;
    s = 1812433253u * (s ^ (s >> 30)) + static_cast<uint32_t>(i) + 1u;
  }
  pos_ = 624;
}

uint32_t NumpyLegacyRng::next_u32() {
  constexpr int N = 624, M = 397;
  if (pos_ == N) {
    int i;
    uint32_t y;
    for (i = 0; i < N - M; ++i) {
      y = (key_[i] & 0x80000000u) | (key_[i + 1] & 0x7fffffffu);
      key_[i] = key_[i + M] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
    }
    for (; i < N - 1; ++i) {
      y = (key_[i] & 0x80000000u) | (key_[i + 1] & 0x7fffffffu);
      key_[i] = key_[i + (M - N)] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
    }
    y = (key_[N - 1] & 0x80000000u) | (key_[0] & 0x7fffffffu);
    key_[N - 1] = key_[M - 1] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
    pos_ = 0;
  }
  uint32_t y = key_[pos_++];
  y ^= (y >> 11);
  y ^= (y << 7) & 0x9d2c5680u;
  y ^= (y << 15) & 0xefc60000u;
  y ^= (y >> 18);
  return y;
}

uint32_t NumpyLegacyRng::interval(uint32_t max_inclusive) {
  if (max_inclusive == 0) return 0;
  uint32_t mask = max_inclusive;
  mask |= mask >> 1;
  mask |= mask >> 2;
  mask |= mask >> 4;
  mask |= mask >> 8;
  mask |= mask >> 16;
  uint32_t v;
  while ((v = (next_u32() & mask)) > max_inclusive) {
  }
  return v;
}

void NumpyLegacyRng::shuffle(int32_t* a, int n) {
  for (int i = n - 1; i >= 1; --i) {
    uint32_t j = interval(static_cast<uint32_t>(i));
    std::swap(a[i], a[j]);
  }
}

// ---------------------------------------------------------------------------
// random-block tables
// ---------------------------------------------------------------------------
namespace {

// Python slice a[lo:hi] of the array 1,2,...,n (middle_seq), appended to out.
void append_middle_slice(int n, int lo, int hi, std::vector<int32_t>& out) {
  lo = std::max(0, std::min(lo, n));
  hi = std::max(0, std::min(hi, n));
  for (int k = lo; k < hi; ++k) out.push_back(k + 1);
}

// One head of the "old plan": rows for ALL nb-2 middle blocks of a sequence of
// max_position_embeddings tokens are drawn (the RNG stream of the next head
// depends on it); only the first keep_rows are stored.
bool old_plan_head(NumpyLegacyRng& rng, int nb, int r, int block, int keep_rows, int32_t* out) {
  const int n_mid = nb - 2;
  int last = nb - 1;
  if (1024 > 2 * block) last = 1024 / block - 1;
  std::vector<int32_t> cand;
  for (int i = 1; i < nb - 1; ++i) {
    cand.clear();
    int start = i - 2, end = i;
    if (i == 1) {
      append_middle_slice(n_mid, 2, last, cand);
    } else if (i == 2) {
      append_middle_slice(n_mid, 3, last, cand);
    } else if (i == nb - 3 || i == nb - 2) {
      append_middle_slice(n_mid, 0, last, cand);
    } else if (start > last) {
      append_middle_slice(n_mid, 0, last, cand);
    } else if (end + 1 == last) {
      append_middle_slice(n_mid, 0, start, cand);
    } else {
      append_middle_slice(n_mid, 0, start, cand);
      append_middle_slice(n_mid, end + 1, last, cand);
    }
    rng.shuffle(cand.data(), static_cast<int>(cand.size()));
    if (static_cast<int>(cand.size()) < r) return false;
    if (i - 1 < keep_rows)
      for (int k = 0; k < r; ++k) out[(i - 1) * r + k] = cand[k];
  }
  return true;
}

}  // namespace

rt_status rand_block_table(uint32_t seed, int heads, int n_blocks, int r, int max_pos, int block,
                           std::vector<int32_t>& out) {
  RT_REQUIRE(block > 0 && heads > 0 && r > 0, RT_ERR_INVALID, "rand_block_table: bad arguments");
  RT_REQUIRE(n_blocks > 5 + 2 * r, RT_ERR_INVALID,
             "rand_block_table: %d blocks use full attention, no random table exists", n_blocks);
  const int rows = n_blocks - 2;
  out.assign(static_cast<size_t>(heads) * rows * r, 0);
  NumpyLegacyRng rng;
  rng.seed(seed);
  if ((static_cast<int64_t>(n_blocks) * block) % 256 == 0) {
    const int nb = max_pos / block;
    RT_REQUIRE(nb - 2 >= rows, RT_ERR_UNSUPPORTED, "%d blocks exceed max_position_embeddings=%d", n_blocks,
               max_pos);
    for (int h = 0; h < heads; ++h)
      if (!old_plan_head(rng, nb, r, block, rows, out.data() + static_cast<size_t>(h) * rows * r))
        return fail(RT_ERR_UNSUPPORTED, "random-block plan has fewer than %d candidates", r);
  } else {
    // plan = [(2r+5) blocks, n_blocks] with [r, 0] random blocks: every row draws
    // from to-blocks [0, 2r+5); rows outer, heads inner.
    const int P = 2 * r + 5;
    std::vector<int32_t> perm(P);
    for (int row = 1; row < n_blocks; ++row) {
      for (int h = 0; h < heads; ++h) {
        std::iota(perm.begin(), perm.end(), 0);
        rng.shuffle(perm.data(), P);
        int got = 0;
        int32_t picked[16];
        for (int i = 0; i < P && got < r; ++i) {
          const int b = perm[i];
          bool illegal = (b == row - 1 || b == row || b == row + 1 || b == 0 || b == P - 1);
          if (row == 1 && b == P - 2) illegal = true;
          if (row == P - 2 && b == 1) illegal = true;
          if (!illegal) picked[got++] = b;
        }
        if (got < r) return fail(RT_ERR_UNSUPPORTED, "random-block plan has fewer than %d candidates", r);
        if (row <= rows)
          for (int k = 0; k < r; ++k) out[(static_cast<size_t>(h) * rows + (row - 1)) * r + k] = picked[k];
      }
    }
  }
  int32_t mx = 0;
  for (int32_t v : out) mx = std::max(mx, v);
  RT_REQUIRE(mx < n_blocks, RT_ERR_UNSUPPORTED,
             "%d tokens: random block id %d lies beyond the sequence (the validation model fails here too)",
             n_blocks * block, mx);
  return RT_OK;
}

void kv_block_lists(const rt_config& cfg, int L, const int32_t* rand_head,
                    std::vector<std::vector<int32_t>>& lists) {
  lists.assign(L, {});
  auto all = [&](std::vector<int32_t>& v) {
    v.resize(L);
    std::iota(v.begin(), v.end(), 0);
  };
  if (cfg.pattern == RT_PATTERN_BAND) {
    all(lists[0]);
    for (int i = 1; i < L; ++i) {
      const int lo = std::max(0, i - cfg.band_half), hi = std::min(L - 1, i + cfg.band_half);
      if (lo > 0) lists[i].push_back(0);
      for (int b = lo; b <= hi; ++b) lists[i].push_back(b);
    }
    return;
  }
  if (!uses_random_table(cfg, L)) {
    for (int i = 0; i < L; ++i) all(lists[i]);
    return;
  }
  const int r = cfg.num_rand;
  auto rnd = [&](int row, std::vector<int32_t>& v) {
    for (int k = 0; k < r; ++k) v.push_back(rand_head[row * r + k]);
  };
  all(lists[0]);
  lists[1] = {0, 1, 2, L - 1};
  rnd(0, lists[1]);
  for (int i = 2; i < L - 2; ++i) {
    lists[i] = {0, i - 1, i, i + 1};
    rnd(i - 1, lists[i]);
    lists[i].push_back(L - 1);
  }
  lists[L - 2] = {0, L - 3, L - 2, L - 1};
  rnd(L - 3, lists[L - 2]);
  all(lists[L - 1]);
}

rt_status validate_lengths(const rt_config& cfg, const int32_t* lens, int n_seq) {
  RT_REQUIRE(lens != nullptr && n_seq > 0, RT_ERR_INVALID, "empty batch");
  for (int s = 0; s < n_seq; ++s) {
    RT_REQUIRE(lens[s] > 0 && lens[s] % cfg.block == 0, RT_ERR_INVALID,
               "sequence %d: length %d is not a positive multiple of the block size %d", s, lens[s], cfg.block);
    RT_REQUIRE(lens[s] <= cfg.max_pos, RT_ERR_UNSUPPORTED, "sequence %d: length %d exceeds max_pos %d", s,
               lens[s], cfg.max_pos);
  }
  return RT_OK;
}

rt_status build_block_csr(const rt_config& cfg, uint32_t layer_seed, const int32_t* lens, int n_seq,
                          BlockCsr& out, TableCache* cache) {
  RT_TRY(validate_lengths(cfg, lens, n_seq));
  TableCache local;
  TableCache& tc = cache ? *cache : local;
  // pass 1: offsets
  out.kv_ptr.clear();
  out.kv_ptr.push_back(0);
  std::vector<std::vector<int32_t>> lists;
  std::vector<int32_t> zero_rand;
  for (int s = 0; s < n_seq; ++s) {
    const int L = lens[s] / cfg.block;
    if (uses_random_table(cfg, L)) {
      auto key = std::make_pair(layer_seed, L);
      if (!tc.count(key)) {
        std::vector<int32_t> t;
        RT_TRY(rand_block_table(layer_seed, cfg.heads, L, cfg.num_rand, cfg.max_pos, cfg.block, t));
        tc.emplace(key, std::move(t));
      }
      zero_rand.assign(static_cast<size_t>(L) * cfg.num_rand, 0);
    }
    kv_block_lists(cfg, L, zero_rand.data(), lists);
    for (int q = 0; q < L; ++q) out.kv_ptr.push_back(out.kv_ptr.back() + static_cast<int32_t>(lists[q].size()));
  }
  out.visits = out.kv_ptr.back();
  out.kv_idx.assign(static_cast<size_t>(cfg.heads) * out.visits, 0);
  // pass 2: ids per head
  int qbase = 0;
  for (int s = 0; s < n_seq; ++s) {
    const int L = lens[s] / cfg.block;
    const int32_t* table = nullptr;
    if (uses_random_table(cfg, L)) table = tc[std::make_pair(layer_seed, L)].data();
    for (int h = 0; h < cfg.heads; ++h) {
      kv_block_lists(cfg, L, table ? table + static_cast<size_t>(h) * (L - 2) * cfg.num_rand : nullptr, lists);
      int32_t* dst = out.kv_idx.data() + static_cast<size_t>(h) * out.visits;
      for (int q = 0; q < L; ++q) std::copy(lists[q].begin(), lists[q].end(), dst + out.kv_ptr[qbase + q]);
    }
    qbase += L;
  }
  return RT_OK;
}

// ---------------------------------------------------------------------------
// partitions
// ---------------------------------------------------------------------------
void lpt_partition(const int32_t* cost, int n_q, const int32_t* seq_prefix, int n_seq, int n_parts, int heads,
                   std::vector<int32_t>& offsets, std::vector<int32_t>& ids) {
  std::vector<int32_t> order(n_q);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cost[a] > cost[b]; });
  using Entry = std::pair<int64_t, int32_t>;  // (load, part): smallest load first, then smallest part
  std::priority_queue<Entry, std::vector<Entry>, std::greater<Entry>> heap;
  for (int p = 0; p < n_parts; ++p) heap.emplace(0, p);
  std::vector<std::vector<int32_t>> parts(n_parts);
  for (int g : order) {
    int s = 0;
    while (s + 1 < n_seq && g >= seq_prefix[s + 1]) ++s;
    const int first = seq_prefix[s], nblk = seq_prefix[s + 1] - seq_prefix[s];
    for (int h = 0; h < heads; ++h) {
      Entry e = heap.top();
      heap.pop();
      parts[e.second].push_back(g - first + h * nblk + first * heads);
      heap.emplace(e.first + cost[g], e.second);
    }
  }
  offsets.assign(1, 0);
  ids.clear();
  for (auto& p : parts) {
    ids.insert(ids.end(), p.begin(), p.end());
    offsets.push_back(static_cast<int32_t>(ids.size()));
  }
}

void binpack_sequences(const double* cost, int n_seq, int n_bins, int32_t* bin_of_seq) {
  std::vector<int> order(n_seq);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cost[a] > cost[b]; });
  std::vector<double> load(n_bins, 0.0);
  for (int i : order) {
    int best = 0;
    for (int b = 1; b < n_bins; ++b)
      if (load[b] < load[best]) best = b;
    bin_of_seq[i] = best;
    load[best] += cost[i];
  }
}

// ---------------------------------------------------------------------------
// attention work list
// ---------------------------------------------------------------------------
namespace {

void query_block_pairs(const rt_config& cfg, int L, std::vector<std::pair<int, int>>& pairs) {
  pairs.clear();
  if (uses_random_table(cfg, L)) {
    pairs.emplace_back(0, L - 1);  // identical lists (every block)
    for (int q = 1; q <= L - 2; q += 2) pairs.emplace_back(q, q + 1 <= L - 2 ? q + 1 : -1);
  } else if (cfg.pattern == RT_PATTERN_BAND) {
    pairs.emplace_back(0, -1);
    for (int q = 1; q < L; q += 2) pairs.emplace_back(q, q + 1 < L ? q + 1 : -1);
  } else {
    for (int q = 0; q < L; q += 2) pairs.emplace_back(q, q + 1 < L ? q + 1 : -1);
  }
}

// Multiset union of two block lists: an id present in both (per occurrence) gets mask 3,
// otherwise mask 1 (first list only) or 2 (second list only).  Appends to ent.
//
// The kernel consumes a list two entries per step (one 128-column score tile), with the
// softmax of tile rows 0-63 done by two warps and of rows 64-127 by two others.  The merged
// list is therefore ordered so that both halves get equal work in every step: shared entries
// (mask 3) first, then entries of the first and of the second block alternating.
rt_status merge_lists(const int32_t* la, int na, const int32_t* lb, int nb, int L, std::vector<char>& used,
                      std::vector<int32_t>& ent) {
  for (int i = 0; i < na; ++i)
    RT_REQUIRE(la[i] >= 0 && la[i] < L, RT_ERR_INVALID, "block id %d outside sequence of %d blocks", la[i], L);
  for (int j = 0; j < nb; ++j)
    RT_REQUIRE(lb[j] >= 0 && lb[j] < L, RT_ERR_INVALID, "block id %d outside sequence of %d blocks", lb[j], L);
  if (nb == 0 || (na == nb && std::equal(la, la + na, lb))) {
    for (int i = 0; i < na; ++i) ent.push_back((la[i] << 2) | (nb == 0 ? 1 : 3));
    return RT_OK;
  }
  used.assign(nb, 0);
  static thread_local std::vector<int32_t> only_a, only_b;
  only_a.clear();
  only_b.clear();
  for (int i = 0; i < na; ++i) {
    bool both = false;
    for (int j = 0; j < nb; ++j)
      if (!used[j] && lb[j] == la[i]) {
        used[j] = 1;
        both = true;
        break;
      }
    if (both) ent.push_back((la[i] << 2) | 3);
    else only_a.push_back((la[i] << 2) | 1);
  }
  for (int j = 0; j < nb; ++j)
    if (!used[j]) only_b.push_back((lb[j] << 2) | 2);
  // alternate; when the shared part is odd its last step is completed by the first single-block entry
  size_t ia = 0, ib = 0;
  while (ia < only_a.size() || ib < only_b.size()) {
    if (ia < only_a.size()) ent.push_back(only_a[ia++]);
    if (ib < only_b.size()) ent.push_back(only_b[ib++]);
  }
  return RT_OK;
}

struct ItemRef {
  int32_t n_entries;
  const int32_t* ent;
  AttnItem it;
  int32_t seq = -1;      // source of the list for PlanSkeleton: sequence, item index inside its template,
  int32_t tmpl_item = 0; // offset of this part inside the template item's list, and whether it is a part
  int32_t part_off = 0;
  int32_t is_part = 0;
};

// Cuts long lists into near-equal parts; each part becomes an item of its own that writes a
// partial result to a scratch slot.  A list is cut only when it is longer than both `split`
// and one CTA's fair share of the whole batch: on a large batch the longest list already fits
// inside a CTA's share, and parts would only add partial-result traffic and a merge.
void split_long_items(std::vector<ItemRef>& refs, int split, int n_ctas, AttnPlanHost& out) {
  out.groups.clear();
  out.n_slots = 0;
  if (split <= 0) return;
  int64_t cost = 0;
  for (const ItemRef& r : refs) cost += r.n_entries + 2;
  split = std::max<int64_t>(split, (cost + n_ctas - 1) / n_ctas);
  std::vector<ItemRef> res;
  res.reserve(refs.size());
  for (const ItemRef& r : refs) {
    if (r.n_entries <= split) {
      res.push_back(r);
      continue;
    }
    // parts are whole steps (two entries each); only the last part may end on a single entry
    const int steps = (r.n_entries + 1) / 2;
    const int split_steps = std::max(1, split / 2);
    const int parts = (steps + split_steps - 1) / split_steps;
    const int base = steps / parts, extra = steps % parts;
    const int32_t g[6] = {out.n_slots, parts, r.it.out_tok0, r.it.out_tok1, r.it.head, 0};
    out.groups.insert(out.groups.end(), g, g + 6);
    int off = 0;
    for (int p = 0; p < parts; ++p) {
      ItemRef part = r;
      part.n_entries = std::min(2 * (base + (p < extra ? 1 : 0)), r.n_entries - off);
      part.ent = r.ent + off;
      part.it.n_entries = part.n_entries;
      part.it.head = r.it.head | ((out.n_slots + 1) << 8);
      part.part_off = off;
      part.is_part = 1;
      off += part.n_entries;
      ++out.n_slots;
      res.push_back(part);
    }
  }
  refs.swap(res);
}

void assign_and_emit(std::vector<ItemRef>& refs, int n_ctas, AttnPlanHost& out, PlanSkeleton* skel = nullptr) {
  // longest-processing-time assignment of items to CTAs; cost = steps of two entries + 1 (per-item
  // prologue / epilogue)
  std::vector<int> order(refs.size());
  std::iota(order.begin(), order.end(), 0);
  auto cost_of = [&](int i) { return (refs[i].n_entries + 1) / 2 + 1; };
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cost_of(a) > cost_of(b); });
  using Entry = std::pair<int64_t, int32_t>;
  std::priority_queue<Entry, std::vector<Entry>, std::greater<Entry>> heap;
  for (int c = 0; c < n_ctas; ++c) heap.emplace(0, c);
  std::vector<int32_t> cta_of(refs.size());
  std::vector<int32_t> count(n_ctas + 1, 0);
  size_t total_entries = 0;
  for (int i : order) {
    Entry e = heap.top();
    heap.pop();
    cta_of[i] = e.second;
    ++count[e.second + 1];
    heap.emplace(e.first + cost_of(i), e.second);
    total_entries += refs[i].n_entries;
  }
  out.cta_ptr.assign(n_ctas + 1, 0);
  for (int c = 0; c < n_ctas; ++c) out.cta_ptr[c + 1] = out.cta_ptr[c] + count[c + 1];
  std::vector<int32_t> cursor(out.cta_ptr.begin(), out.cta_ptr.end() - 1);
  out.items.resize(refs.size());
  std::vector<int32_t> slot_of(refs.size());
  for (int i : order) slot_of[i] = cursor[cta_of[i]]++;  // descending cost inside each CTA
  std::vector<int32_t> pos_item(refs.size());
  for (size_t i = 0; i < refs.size(); ++i) pos_item[slot_of[i]] = static_cast<int32_t>(i);
  out.entries.resize(total_entries);
  size_t off = 0;
  for (size_t sidx = 0; sidx < refs.size(); ++sidx) {
    const ItemRef& r = refs[pos_item[sidx]];
    AttnItem it = r.it;
    it.entry_off = static_cast<int32_t>(off);
    it.n_entries = r.n_entries;
    std::copy(r.ent, r.ent + r.n_entries, out.entries.begin() + off);
    off += r.n_entries;
    out.items[sidx] = it;
  }
  if (skel) {
    skel->src.resize(refs.size());
    for (size_t sidx = 0; sidx < refs.size(); ++sidx) {
      const ItemRef& r = refs[pos_item[sidx]];
      skel->src[sidx] = PlanSkeleton::Src{r.seq, r.tmpl_item, r.part_off, r.is_part ? r.n_entries : -1};
    }
  }
}

}  // namespace

rt_status build_attn_plan(const rt_config& cfg, const int32_t* lens, int n_seq, const int32_t* kv_ptr,
                          const int32_t* kv_idx, int64_t visits_per_head, int n_ctas, AttnPlanHost& out,
                          int split_entries) {
  RT_REQUIRE(n_ctas > 0, RT_ERR_INVALID, "attention plan needs at least one CTA");
  const int nh = cfg.heads, B = cfg.block;
  std::vector<int32_t> pool;  // all merged lists, back to back
  struct Pending {
    AttnItem it;
    size_t off;
    int32_t n;
  };
  std::vector<Pending> pend;
  int tok0 = 0, qbase = 0;
  std::vector<std::pair<int, int>> pairs;
  std::vector<char> used;
  out = AttnPlanHost();
  for (int s = 0; s < n_seq; ++s) {
    const int L = lens[s] / B;
    query_block_pairs(cfg, L, pairs);
    for (int h = 0; h < nh; ++h) {
      const int32_t* idx = kv_idx + static_cast<size_t>(h) * visits_per_head;
      for (auto& pr : pairs) {
        const int qa = pr.first, qb = pr.second;
        const int32_t* la = idx + kv_ptr[qbase + qa];
        const int na = kv_ptr[qbase + qa + 1] - kv_ptr[qbase + qa];
        const int32_t* lb = qb >= 0 ? idx + kv_ptr[qbase + qb] : nullptr;
        const int nb = qb >= 0 ? kv_ptr[qbase + qb + 1] - kv_ptr[qbase + qb] : 0;
        Pending p;
        p.off = pool.size();
        RT_TRY(merge_lists(la, na, lb, nb, L, used, pool));
        p.n = static_cast<int32_t>(pool.size() - p.off);
        const int base_row = tok0 * nh + h * lens[s];
        p.it.kv_row0 = base_row;
        p.it.q_row0 = base_row + qa * B;
        p.it.q_row1 = qb >= 0 ? base_row + qb * B : p.it.q_row0;
        p.it.out_tok0 = tok0 + qa * B;
        p.it.out_tok1 = qb >= 0 ? tok0 + qb * B : -1;
        p.it.head = h;
        p.it.n_entries = p.n;
        p.it.entry_off = 0;
        out.visits += na + nb;
        pend.push_back(p);
      }
    }
    tok0 += lens[s];
    qbase += L;
  }
  std::vector<ItemRef> refs(pend.size());
  for (size_t i = 0; i < pend.size(); ++i) refs[i] = ItemRef{pend[i].n, pool.data() + pend[i].off, pend[i].it};
  split_long_items(refs, split_entries, n_ctas, out);
  assign_and_emit(refs, n_ctas, out);
  out.total_tokens = tok0;
  out.heads = nh;
  return RT_OK;
}

rt_status build_seq_template(const rt_config& cfg, uint32_t seed, int L, TableCache* tables, SeqTemplate& out) {
  out = SeqTemplate();
  out.n_blocks = L;
  const int32_t* table = nullptr;
  std::vector<int32_t> local;
  if (uses_random_table(cfg, L)) {
    auto key = std::make_pair(seed, L);
    if (tables && tables->count(key)) {
      table = (*tables)[key].data();
    } else {
      RT_TRY(rand_block_table(seed, cfg.heads, L, cfg.num_rand, cfg.max_pos, cfg.block, local));
      if (tables) {
        auto it = tables->emplace(key, std::move(local)).first;
        table = it->second.data();
      } else {
        table = local.data();
      }
    }
  }
  std::vector<std::pair<int, int>> pairs;
  query_block_pairs(cfg, L, pairs);
  out.n_pairs = static_cast<int>(pairs.size());
  for (auto& pr : pairs) {
    out.qa.push_back(pr.first);
    out.qb.push_back(pr.second);
  }
  std::vector<std::vector<int32_t>> lists;
  std::vector<char> used;
  out.item_off.push_back(0);
  for (int h = 0; h < cfg.heads; ++h) {
    kv_block_lists(cfg, L, table ? table + static_cast<size_t>(h) * (L - 2) * cfg.num_rand : nullptr, lists);
    for (auto& pr : pairs) {
      const auto& la = lists[pr.first];
      static const std::vector<int32_t> kEmpty;
      const auto& lb = pr.second >= 0 ? lists[pr.second] : kEmpty;
      RT_TRY(merge_lists(la.data(), static_cast<int>(la.size()), lb.data(), static_cast<int>(lb.size()), L, used,
                         out.ent));
      out.item_off.push_back(static_cast<int32_t>(out.ent.size()));
      out.visits += static_cast<int64_t>(la.size() + lb.size());
    }
  }
  return RT_OK;
}

rt_status assemble_attn_plan(const rt_config& cfg, const int32_t* lens, int n_seq,
                             const SeqTemplate* const* templates, int n_ctas, AttnPlanHost& out,
                             int split_entries, PlanSkeleton* skel) {
  RT_REQUIRE(n_ctas > 0, RT_ERR_INVALID, "attention plan needs at least one CTA");
  const int nh = cfg.heads, B = cfg.block;
  out = AttnPlanHost();
  size_t n_items = 0;
  for (int s = 0; s < n_seq; ++s) n_items += static_cast<size_t>(templates[s]->n_pairs) * nh;
  std::vector<ItemRef> refs;
  refs.reserve(n_items);
  int tok0 = 0;
  for (int s = 0; s < n_seq; ++s) {
    const SeqTemplate& t = *templates[s];
    RT_REQUIRE(t.n_blocks * B == lens[s], RT_ERR_STATE, "template does not match sequence %d", s);
    for (int h = 0; h < nh; ++h) {
      const int base_row = tok0 * nh + h * lens[s];
      for (int p = 0; p < t.n_pairs; ++p) {
        const int idx = h * t.n_pairs + p;
        ItemRef r;
        r.n_entries = t.item_off[idx + 1] - t.item_off[idx];
        r.ent = t.ent.data() + t.item_off[idx];
        r.it.kv_row0 = base_row;
        r.it.q_row0 = base_row + t.qa[p] * B;
        r.it.q_row1 = t.qb[p] >= 0 ? base_row + t.qb[p] * B : r.it.q_row0;
        r.it.out_tok0 = tok0 + t.qa[p] * B;
        r.it.out_tok1 = t.qb[p] >= 0 ? tok0 + t.qb[p] * B : -1;
        r.it.head = h;
        r.it.entry_off = 0;
        r.it.n_entries = r.n_entries;
        r.seq = s;
        r.tmpl_item = idx;
        refs.push_back(r);
      }
    }
    out.visits += t.visits;
    tok0 += lens[s];
  }
  split_long_items(refs, split_entries, n_ctas, out);
  assign_and_emit(refs, n_ctas, out, skel);
  out.total_tokens = tok0;
  out.heads = nh;
  return RT_OK;
}

rt_status refill_attn_plan(const PlanSkeleton& skel, const AttnPlanHost& base, const SeqTemplate* const* templates,
                           AttnPlanHost& out) {
  RT_REQUIRE(skel.src.size() == base.items.size(), RT_ERR_STATE, "plan skeleton does not match its plan");
  out.items = base.items;
  out.cta_ptr = base.cta_ptr;
  out.groups = base.groups;
  out.n_slots = base.n_slots;
  out.total_tokens = base.total_tokens;
  out.heads = base.heads;
  out.visits = base.visits;
  out.entries.clear();
  out.entries.reserve(base.entries.size() + base.entries.size() / 8);
  for (size_t i = 0; i < skel.src.size(); ++i) {
    const PlanSkeleton::Src& sr = skel.src[i];
    const SeqTemplate& t = *templates[sr.seq];
    RT_REQUIRE(sr.tmpl_item + 1 < static_cast<int>(t.item_off.size()), RT_ERR_STATE, "template does not fit the skeleton");
    const int32_t* list = t.ent.data() + t.item_off[sr.tmpl_item];
    const int full = t.item_off[sr.tmpl_item + 1] - t.item_off[sr.tmpl_item];
    int n = full;
    if (sr.part_len >= 0) {  // one part of a split list: the same cut in every layer
      RT_REQUIRE(sr.part_off + sr.part_len <= full, RT_ERR_STATE, "split list changed its length between layers");
      list += sr.part_off;
      n = sr.part_len;
    }
    AttnItem& it = out.items[i];
    it.entry_off = static_cast<int32_t>(out.entries.size());
    it.n_entries = n;
    out.entries.insert(out.entries.end(), list, list + n);
  }
  return RT_OK;
}

void attn_plan_bounds(const rt_config& cfg, const int32_t* lens, int n_seq, int split_entries, size_t* items,
                      size_t* entries, size_t* slots, size_t* groups) {
  size_t n_items = 0, n_entries = 0, n_slots = 0, n_groups = 0;
  std::vector<std::pair<int, int>> pairs;
  const int split = split_entries > 0 ? split_entries : 0;
  for (int s = 0; s < n_seq; ++s) {
    const int L = lens[s] / cfg.block;
    query_block_pairs(cfg, L, pairs);
    auto len_of = [&](int q) -> int {  // list length of query block q (table-independent)
      if (q < 0) return 0;
      if (cfg.pattern == RT_PATTERN_BAND) {
        if (q == 0) return L;
        const int lo = std::max(0, q - cfg.band_half), hi = std::min(L - 1, q + cfg.band_half);
        return hi - lo + 1 + (lo > 0 ? 1 : 0);
      }
      if (!uses_random_table(cfg, L) || q == 0 || q == L - 1) return L;
      return (q == 1 || q == L - 2 ? 4 : 5) + cfg.num_rand;
    };
    for (auto& pr : pairs) {
      const size_t ub = static_cast<size_t>(len_of(pr.first)) + len_of(pr.second);  // merged list: at most the sum
      n_items += 1;
      n_entries += ub;
      if (split > 0 && ub > static_cast<size_t>(split)) {
        const size_t parts = ub / split + 2;
        n_slots += parts;
        n_items += parts;
        n_groups += 1;
      }
    }
  }
  *items = n_items * cfg.heads;
  *entries = n_entries * cfg.heads;
  *slots = n_slots * cfg.heads;
  *groups = n_groups * cfg.heads;
}

}  // namespace rt
