// Block-sparse attention for sm_100a (tcgen05 + TMEM + TMA), online softmax fused.
//
// A persistent CTA walks its list of work items.  An item is up to two 64-token
// query blocks of one (sequence, head) stacked into a 128-row tile, plus the
// merged list of 64-token key/value blocks they attend to (global, window and
// random blocks come from the same table; each entry carries a 2-bit mask that
// says which of the two query blocks uses it).
//
// Four warps contribute one thread each, with blocking (bounded) waits on their own
// barriers, so that their serial latencies run side by side:
//   warp 4   K / Q loader: TMA loads of the Q tile per item and of one K box (64 x 64,
//            128-byte swizzle) per list entry into a shared-memory ring.  The only role
//            that reads the work list in global memory (4-byte asynchronous copies, eight
//            entries ahead); it publishes one record per entry ({entry, first/last flags,
//            key/value row}) in a shared-memory ring for the other roles;
//   warp 6   V loader: one V box per entry into its own ring;
//   warp 7   issues S = Q K^T (M=128, N=64, K=64; both operands K-major in shared memory)
//            into one of two TMEM score buffers, as soon as the K block has landed and the
//            PV MMA two entries back has completed (which frees score buffer and
//            probability buffer of that parity at once);
//   warp 5   issues PV = P V (P read from TMEM, V MN-major in shared memory), accumulating
//            the output tile in TMEM;
//   warps 0-3  softmax: thread r owns tile row r.  It pulls its score row out of
//            TMEM, keeps the running max / sum in fp32 (base-2 exponentials) and
//            writes the 16-bit probabilities back to TMEM for the PV MMA.  The
//            output tile accumulates in TMEM across the whole list (the PV MMAs
//            add into it); it is rescaled only when a row's max has grown by more
//            than 2^8 since the last rescale ("lazy" rescaling: probabilities are
//            then at most 256, well inside 16-bit range), and read once per item
//            for the final division by the row sum.  One barrier wait (score tile
//            ready) and one arrival (probabilities stored) per entry.
// The kernel is launched with 128 registers per thread; the issue warps hand registers
// to the softmax warps (setmaxnreg 72 / 184), which hold a 64-column score row each.
//
// Two CTAs share an SM (256 TMEM columns and ~107 KB of shared memory each), so one
// CTA's softmax latency hides behind the other's.
//
// Lists that are longer than one CTA's share of the batch are cut into parts by the
// host; a part leaves its un-normalised fp32 output tile, row maxima and row sums in
// scratch and merge_partials_kernel combines the parts of a list.
//
// Output rows go token-major [T][heads*64].  Counterpart of
// layers/kernels/sparse_attention.cu:2953-3228; the math follows the reference's
// validation model (python/modeling_big_bird.py:626-851: softmax over the
// concatenated listed blocks, duplicates counted twice).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <vector>

#include "attention.h"
#include "common.h"
#include "device_error.h"
#include "launch.h"
#include "launch_count.h"
#include "sm100_ptx.cuh"
#include "tma_host.h"

namespace rt {
namespace {

using namespace ptx;

constexpr int kThreads = 256;  // warps 0-3 softmax; 4: K/Q loads, 5: PV issue, 6: V loads, 7: S issue (one thread each)
constexpr int kStagesK = 4;              // K ring depth (a slot is free again once the S MMA has read it)
constexpr int kStagesV = 5;              // V ring depth (a slot is held until the PV MMA, two softmax periods later)
constexpr int kEntRing = 32;             // per-entry records travel from the K cursor to the other roles through smem
constexpr int kEntStage = 16;            // landing slots of the asynchronous work-list reads
constexpr int kEntAhead = 8;             // how many list entries the producer reads ahead
constexpr int kEntFirst = 1 << 29;       // record flags: first / last entry of its item
constexpr int kEntLast = 1 << 30;
constexpr int kTileBytes = 64 * 64 * 2;  // one 64 x 64 16-bit block
constexpr int kQBytes = 2 * kTileBytes;
constexpr int kTmemCols = 256;
constexpr int kColS = 0;     // 2 x 64 fp32 score columns
constexpr int kColP = 128;   // 2 x 32 columns of packed 16-bit probabilities
constexpr int kColO = 192;   // 64 fp32 output columns, accumulated over the item's list
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct Smem {
  uint8_t q[2][kQBytes];
  uint8_t k[kStagesK][kTileBytes];
  uint8_t v[kStagesV][kTileBytes];
  uint64_t q_full[2], q_empty[2];
  uint64_t k_full[kStagesK], k_empty[kStagesK], v_full[kStagesV], v_empty[kStagesV];
  uint64_t s_full[2], p_full[2], pv_done[2], o_free;
  int2 ent_ring[kEntRing];      // {entry (block << 2 | mask) | flags, row of the key/value block}
  int32_t ent_stage[kEntStage];
  uint32_t tmem_slot;
  int abort_flag;
  uint32_t k_published;  // entry records written so far (K loader -> V loader)
};
constexpr int kSmemBytes = sizeof(Smem);

// 4-byte asynchronous global -> shared copies: the producer thread reads its work list
// ahead without ever stalling on a global load.
__device__ __forceinline__ void cp_async_4(void* dst_smem, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// A CTA's items are consecutive and so are their lists: [first, first + count) of `entries`.
__device__ __forceinline__ void cta_entry_range(const AttnItem* items, int item_begin, int item_end, int& first,
                                                uint32_t& count) {
  first = 0;
  count = 0;
  if (item_begin < item_end) {
    const int a = items[item_begin].entry_off;
    const AttnItem& z = items[item_end - 1];
    first = a;
    count = static_cast<uint32_t>(z.entry_off + z.n_entries - a);
  }
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed fp32x2 arithmetic and three-input max (sm_100): half the issue slots of the
// scalar forms in the softmax inner loops.
__device__ __forceinline__ unsigned long long f2_pack(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void f2_unpack(unsigned long long v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long f2_fma(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long f2_add(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}


// Register budget: the kernel is launched with 128 registers per thread (two CTAs of 256
// threads per SM); the four single-thread warps then give registers back and the softmax
// warps, which hold a 64-column score row per thread, take them.
constexpr int kRegsIssue = 72;
constexpr int kRegsSoftmax = 184;
template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

template <bool BF16>
__global__ void __launch_bounds__(kThreads, 2)
sparse_attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, uint16_t* __restrict__ ctx,
                        const AttnItem* __restrict__ items, const int32_t* __restrict__ entries,
                        const int32_t* __restrict__ cta_ptr, int hidden, float scale_log2, int* error_flag,
                        float* __restrict__ part_o, float* __restrict__ part_ml) {
  RT_PDL_LAUNCH_DEPENDENTS();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if ((smem_u32(smem_raw) & 1023u) != 0) {  // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(error_flag, 0, 299);
    return;
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.q_full[i], 1);
      mbar_init(&sm.q_empty[i], 1);
      mbar_init(&sm.s_full[i], 1);
      mbar_init(&sm.p_full[i], 4);  // one elected arrival per softmax warp
      mbar_init(&sm.pv_done[i], 1);
    }
    mbar_init(&sm.o_free, 4);
    for (int s = 0; s < kStagesK; ++s) {
      mbar_init(&sm.k_full[s], 1);
      mbar_init(&sm.k_empty[s], 1);
    }
    for (int s = 0; s < kStagesV; ++s) {
      mbar_init(&sm.v_full[s], 1);
      mbar_init(&sm.v_empty[s], 1);
    }
    sm.abort_flag = 0;
    sm.k_published = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(&sm.tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sm.tmem_slot;
  AbortCtx ab{&sm.abort_flag, error_flag};
  RT_PDL_WAIT();  // q/k/v, the work list and the output buffer belong to earlier work until here

  const int item_begin = cta_ptr[blockIdx.x];
  const int item_end = cta_ptr[blockIdx.x + 1];

  // Four single-thread roles walk the CTA's flattened (item, entry) stream, each with blocking
  // (bounded) waits on its own barriers, so that their serial latencies (barrier round trips,
  // descriptor set-up, TMA / MMA issue, commits: several hundred clocks per entry each) run
  // side by side instead of adding up in one thread.
  if (warp >= 4) {
  reg_dealloc<kRegsIssue>();  // executed by all four warps of the upper warpgroup at this one place
  if (warp == 4) {
    // ------------------------------------------------------------------ K / Q loader
    // The only role that reads the work list in global memory: entries arrive through 4-byte
    // asynchronous copies issued kEntAhead entries early, the next item is prefetched in
    // registers.  It publishes one record per entry for the other roles.
    if (lane == 0) {
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_k);
      int ent_first;
      uint32_t total;
      cta_entry_range(items, item_begin, item_end, ent_first, total);
      const int32_t* ent = entries + ent_first;
      auto fetch = [&](uint32_t i) {
        if (i < total) cp_async_4(&sm.ent_stage[i % kEntStage], ent + i);
        cp_async_commit();  // one group per entry, empty past the end: the wait below counts groups
      };
      for (uint32_t i = 0; i < kEntAhead; ++i) fetch(i);
      int k_item = item_begin, k_j = 0;
      uint32_t k_itn = 0;
      AttnItem ki{}, kn{};
      auto settle_item = [&]() {  // k_item -> first item with a non-empty list; prefetch the one after it
        while (k_item < item_end && ki.n_entries == 0) {
          ++k_item;
          if (k_item < item_end) ki = items[k_item];
        }
        if (k_item + 1 < item_end) kn = items[k_item + 1];
      };
      if (k_item < item_end) ki = items[k_item];
      settle_item();
      bool ok = true;
      for (uint32_t k_g = 0; ok && k_g < total; ++k_g) {
        if (k_j == 0) {
          const int qb = k_itn & 1;
          if (!mbar_wait(&sm.q_empty[qb], ((k_itn >> 1) & 1) ^ 1, ab, 211)) break;
          mbar_arrive_expect_tx(&sm.q_full[qb], kQBytes);
          tma_load_2d(sm.q[qb], &map_q, 0, ki.q_row0, &sm.q_full[qb]);
          tma_load_2d(sm.q[qb] + kTileBytes, &map_q, 0, ki.q_row1, &sm.q_full[qb]);
        }
        const int st = k_g % kStagesK;
        if (!mbar_wait(&sm.k_empty[st], ((k_g / kStagesK) & 1) ^ 1, ab, 212)) break;
        cp_async_wait<kEntAhead - 1>();  // the copy of entry k_g has landed
        const int e = *reinterpret_cast<volatile int32_t*>(&sm.ent_stage[k_g % kEntStage]);
        fetch(k_g + kEntAhead);
        const int row = ki.kv_row0 + (e >> 2) * 64;
        const bool last = k_j + 1 == ki.n_entries;
        sm.ent_ring[k_g % kEntRing] = make_int2(e | (k_j == 0 ? kEntFirst : 0) | (last ? kEntLast : 0), row);
        __threadfence_block();
        *reinterpret_cast<volatile uint32_t*>(&sm.k_published) = k_g + 1;
        mbar_arrive_expect_tx(&sm.k_full[st], kTileBytes);
        tma_load_2d(sm.k[st], &map_k, 0, row, &sm.k_full[st]);
        ++k_j;
        if (last) {
          ++k_item;
          ++k_itn;
          k_j = 0;
          ki = kn;
          settle_item();
        }
      }
      cp_async_wait<0>();
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------------ V loader
    if (lane == 0) {
      prefetch_tensormap(&map_v);
      int ent_first;
      uint32_t total;
      cta_entry_range(items, item_begin, item_end, ent_first, total);
      volatile uint32_t* published = &sm.k_published;
      volatile int* abort_flag = &sm.abort_flag;
      bool ok = true;
      for (uint32_t v_g = 0; ok && v_g < total; ++v_g) {
        const int st = v_g % kStagesV;
        if (!mbar_wait(&sm.v_empty[st], ((v_g / kStagesV) & 1) ^ 1, ab, 213)) break;
        if (*published <= v_g) {  // the record of this entry is not written yet (rare: V runs behind K)
          const long long t0 = clock64();
          while (*published <= v_g && !*abort_flag) {
            __nanosleep(40);
            if (clock64() - t0 > kWaitCycles) {
              *abort_flag = 1;
              atomicCAS(error_flag, 0, 217);
            }
          }
          if (*abort_flag) break;
        }
        __threadfence_block();
        const int row = sm.ent_ring[v_g % kEntRing].y;
        mbar_arrive_expect_tx(&sm.v_full[st], kTileBytes);
        tma_load_2d(sm.v[st], &map_v, 0, row, &sm.v_full[st]);
      }
    }
  } else if (warp == 7) {
    // ------------------------------------------------------------------ S = Q K^T issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(128, 64, BF16 ? 1 : 0, false);
      int ent_first;
      uint32_t total;
      cta_entry_range(items, item_begin, item_end, ent_first, total);
      uint32_t s_itn = 0;
      for (uint32_t s_g = 0; s_g < total; ++s_g) {
        const int b = s_g & 1;
        const int st = s_g % kStagesK;
        if (!mbar_wait(&sm.k_full[st], (s_g / kStagesK) & 1, ab, 218)) break;
        // the K loader wrote this entry's record before it armed the barrier just waited for
        const int rec = *reinterpret_cast<volatile int*>(&sm.ent_ring[s_g % kEntRing].x);
        const int qb = s_itn & 1;
        if (rec & kEntFirst) {
          if (!mbar_wait(&sm.q_full[qb], (s_itn >> 1) & 1, ab, 219)) break;
        }
        // buffer b (scores and probabilities) is free once the PV MMA of entry s_g-2 has completed:
        // the softmax warps finished that entry before its PV MMA was issued
        if (s_g >= 2) {
          if (!mbar_wait(&sm.pv_done[b], ((s_g - 2) >> 1) & 1, ab, 220)) break;
        }
        tc_fence_after_sync();
        const uint64_t dq = make_smem_desc_sw128(smem_u32(sm.q[qb]));
        const uint64_t dk = make_smem_desc_sw128(smem_u32(sm.k[st]));
        const uint32_t d = tmem_base + kColS + b * 64;
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ss(d, dq + (k * 32 >> 4), dk + (k * 32 >> 4), idesc_s, k ? 1u : 0u);
        tc_commit(&sm.k_empty[st]);
        tc_commit(&sm.s_full[b]);
        if (rec & kEntLast) {
          tc_commit(&sm.q_empty[qb]);
          ++s_itn;
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_pv = make_idesc_f16(128, 64, BF16 ? 1 : 0, true);
      // this thread issues the PV MMAs; the S MMAs are issued by the producer thread, so the
      // two serial issue chains (waits, four MMAs, commits per entry) run side by side
      int ent_first;
      uint32_t total;
      cta_entry_range(items, item_begin, item_end, ent_first, total);
      uint32_t pv_itn = 0;
      bool ok = true;
      for (uint32_t pv_g = 0; ok && pv_g < total; ++pv_g) {
        const int b = pv_g & 1;
        const uint32_t u = pv_g >> 1;
        const int st = pv_g % kStagesV;
        const uint32_t ph = (pv_g / kStagesV) & 1;
        if (!mbar_wait(&sm.v_full[st], ph, ab, 214)) { ok = false; break; }
        // the producer wrote this entry's record before it issued the V copy just waited for
        const int rec = *reinterpret_cast<volatile int*>(&sm.ent_ring[pv_g % kEntRing].x);
        const bool first = (rec & kEntFirst) != 0;
        if (first) {
          // the output tile is overwritten: the softmax warps must have read the previous item's result
          if (!mbar_wait(&sm.o_free, (pv_itn & 1) ^ 1, ab, 215)) { ok = false; break; }
        }
        if (!mbar_wait(&sm.p_full[b], u & 1, ab, 216)) { ok = false; break; }
        tc_fence_after_sync();
        const uint64_t dv = make_smem_desc_sw128(smem_u32(sm.v[st]));
        const uint32_t d = tmem_base + kColO;
        const uint32_t a = tmem_base + kColP + b * 32;
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ts(d, a + k * 8, dv + (k * 2048 >> 4), idesc_pv, (!first || k) ? 1u : 0u);
        tc_commit(&sm.v_empty[st]);
        tc_commit(&sm.pv_done[b]);
        if (rec & kEntLast) ++pv_itn;
      }
    }
  }
  } else {
    reg_alloc<kRegsSoftmax>();
    // ------------------------------------------------------------------ softmax warps 0..3
    const int row = warp * 32 + lane;  // tile row == TMEM lane
    const int half = row >> 6;         // 0: query block A, 1: query block B
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    uint32_t g = 0, itn = 0;
    bool ok = true;
    AttnItem next_item = item_begin < item_end ? items[item_begin] : AttnItem{};
    for (int it = item_begin; it < item_end && ok; ++it) {
      const AttnItem item = next_item;
      if (it + 1 < item_end) next_item = items[it + 1];  // in flight while this item is processed
      const int n = item.n_entries;
      if (n == 0) continue;
      float m_ref = -INFINITY;  // max the stored probabilities / output are relative to (log2 units)
      float l = 0.f;
      for (int j = 0; j < n; ++j) {
        const uint32_t gj = g + j;
        const int b = gj & 1;
        const uint32_t u = gj >> 1;
        // The S MMA of this entry was issued after the PV MMA of entry gj-2 had completed, so this one
        // wait also says that the probability buffer b and the score buffer b are free again.
        if (!mbar_wait(&sm.s_full[b], u & 1, ab, 221)) { ok = false; break; }
        tc_fence_after_sync();
        // the K loader published this entry's record before it loaded the K block of the S tile just waited for
        const bool active = ((sm.ent_ring[gj % kEntRing].x >> half) & 1) != 0;
        uint32_t s[64];
        if (active) {
          tmem_ld32(lane_base + kColS + b * 64, s);
          tmem_ld32(lane_base + kColS + b * 64 + 32, s + 32);
          tc_wait_ld();
        }
        float alpha = 1.f;
        bool fix = false;
        if (active) {
          float mx0 = __uint_as_float(s[0]), mx1 = __uint_as_float(s[1]);
          float mx2 = __uint_as_float(s[2]), mx3 = __uint_as_float(s[3]);
#pragma unroll
          for (int i = 4; i < 60; i += 8) {
            mx0 = max3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
            mx1 = max3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
            mx2 = max3(mx2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
            mx3 = max3(mx3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
          }
          mx0 = max3(mx0, __uint_as_float(s[60]), __uint_as_float(s[61]));
          mx1 = max3(mx1, __uint_as_float(s[62]), __uint_as_float(s[63]));
          const float m_new = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;
          if (m_ref == -INFINITY) {
            m_ref = m_new;  // nothing accumulated for this row yet (its output columns are still zero)
          } else if (m_new > m_ref + kRescaleThreshold) {
            alpha = ex2(m_ref - m_new);
            m_ref = m_new;
            fix = true;
          }
        }
        // the probability buffer was last read by the PV MMA two entries back

        if (__any_sync(0xffffffffu, fix)) {
          // rescale this warp's rows of the output tile; every PV MMA issued so far must be done
          if (j > 0) {
            if (!mbar_wait(&sm.pv_done[b ^ 1], ((gj - 1) >> 1) & 1, ab, 223)) { ok = false; break; }
            tc_fence_after_sync();
#pragma unroll 1
            for (int hc = 0; hc < 2; ++hc) {
              uint32_t o[32];
              tmem_ld32(lane_base + kColO + hc * 32, o);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(lane_base + kColO + hc * 32, o);
            }
          }
          l *= alpha;
        }
        if (active) {
          const unsigned long long c2 = f2_pack(scale_log2, scale_log2);
          const unsigned long long nm2 = f2_pack(-m_ref, -m_ref);
          unsigned long long acc0 = 0ull, acc1 = 0ull;  // two packed partial sums (+0.0f, +0.0f)
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            uint32_t p[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const unsigned long long t =
                  f2_fma(f2_pack(__uint_as_float(s[32 * hc + 2 * i]), __uint_as_float(s[32 * hc + 2 * i + 1])), c2, nm2);
              float t0, t1;
              f2_unpack(t, t0, t1);
              const float p0 = ex2(t0), p1 = ex2(t1);
              if (i & 1) acc1 = f2_add(acc1, f2_pack(p0, p1));
              else acc0 = f2_add(acc0, f2_pack(p0, p1));
              p[i] = pack2<BF16>(p0, p1);
            }
            tmem_st16(lane_base + kColP + b * 32 + hc * 16, p);
          }
          float s0, s1;
          f2_unpack(f2_add(acc0, acc1), s0, s1);
          l += s0 + s1;
        } else {
          uint32_t p[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) p[i] = 0u;
          tmem_st16(lane_base + kColP + b * 32, p);
          tmem_st16(lane_base + kColP + b * 32 + 16, p);
        }
        tc_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.p_full[b]);
      }
      if (!ok) break;
      g += n;
      // final: the last PV MMA of the item completes the output tile
      {
        const uint32_t gl = g - 1;
        if (!mbar_wait(&sm.pv_done[gl & 1], (gl >> 1) & 1, ab, 224)) { ok = false; break; }
        tc_fence_after_sync();
      }
      const int tok0 = half == 0 ? item.out_tok0 : item.out_tok1;
      const int slot = (item.head >> 8) - 1;  // >= 0: this item is one part of a split list
      const float inv = slot >= 0 ? 1.0f : 1.0f / l;
      uint16_t* dst = ctx + static_cast<size_t>((tok0 >= 0 ? tok0 : 0) + (row & 63)) * hidden + (item.head & 255) * 64;
      float* pdst = part_o + (static_cast<size_t>(slot >= 0 ? slot : 0) * 128 + row) * 64;
      if (slot >= 0 && tok0 >= 0) {
        float2 ml = make_float2(m_ref, l);
        *reinterpret_cast<float2*>(part_ml + (static_cast<size_t>(slot) * 128 + row) * 2) = ml;
      }
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {
        uint32_t o[32];
        if (tok0 >= 0) {
          tmem_ld32(lane_base + kColO + hc * 32, o);
          tc_wait_ld();
        }
        if (hc == 1) {
          // both halves are in registers: the MMA warp may overwrite the output tile
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.o_free);
        }
        if (tok0 >= 0) {
          if (slot >= 0) {
            // un-normalised fp32 partial result (relative to m_ref) for the merge kernel
#pragma unroll
            for (int q = 0; q < 4; ++q) st_global_v8(pdst + hc * 32 + 8 * q, o + 8 * q);
          } else {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              uint32_t w[8];
#pragma unroll
              for (int e = 0; e < 8; ++e)
                w[e] = pack2<BF16>(__uint_as_float(o[16 * q + 2 * e]) * inv, __uint_as_float(o[16 * q + 2 * e + 1]) * inv);
              st_global_v8(dst + hc * 32 + 16 * q, w);
            }
          }
        }
      }
      ++itn;
    }
    (void)itn;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Merges the partial results of split lists: one CTA per group, one thread per tile row.
//   out = sum_i O_i 2^(m_i - M) / sum_i l_i 2^(m_i - M),  M = max_i m_i
template <bool BF16>
__global__ void __launch_bounds__(128) merge_partials_kernel(uint16_t* __restrict__ ctx,
                                                             const int32_t* __restrict__ groups,
                                                             const float* __restrict__ part_o,
                                                             const float* __restrict__ part_ml, int hidden) {
  RT_PDL_LAUNCH_DEPENDENTS();
  RT_PDL_WAIT();
  const int32_t* g = groups + blockIdx.x * 6;
  const int first = g[0], parts = g[1], head = g[4] & 255;
  const int row = threadIdx.x;
  const int tok0 = row < 64 ? g[2] : g[3];
  if (tok0 < 0) return;
  float M = -INFINITY;
  for (int i = 0; i < parts; ++i) M = fmaxf(M, part_ml[(static_cast<size_t>(first + i) * 128 + row) * 2]);
  float L = 0.f;
  for (int i = 0; i < parts; ++i) {
    const float2 ml = *reinterpret_cast<const float2*>(part_ml + (static_cast<size_t>(first + i) * 128 + row) * 2);
    L += ml.y * ex2(ml.x - M);
  }
  const float inv = 1.0f / L;
  uint16_t* dst = ctx + static_cast<size_t>(tok0 + (row & 63)) * hidden + head * 64;
#pragma unroll 1
  for (int c = 0; c < 64; c += 16) {
    float acc[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) acc[k] = 0.f;
    for (int i = 0; i < parts; ++i) {
      const size_t base = static_cast<size_t>(first + i) * 128 + row;
      const float w = ex2(part_ml[base * 2] - M);
      const float4* src = reinterpret_cast<const float4*>(part_o + base * 64 + c);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 v = src[q];
        acc[4 * q] += w * v.x;
        acc[4 * q + 1] += w * v.y;
        acc[4 * q + 2] += w * v.z;
        acc[4 * q + 3] += w * v.w;
      }
    }
    uint32_t o[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = pack2<BF16>(acc[2 * k] * inv, acc[2 * k + 1] * inv);
    st_global_v8(dst + c, o);
  }
}

}  // namespace

rt_status launch_sparse_attention(void* ctx, const void* q, const void* k, const void* v, const AttnItem* items_dev,
                                  const int32_t* entries_dev, const int32_t* cta_ptr_dev, int n_ctas,
                                  int total_tokens, int heads, float scale, int dtype, cudaStream_t st, int* error_word_dev,
                                  const AttnSplit& split) {
  RT_REQUIRE(dtype == RT_F16 || dtype == RT_BF16, RT_ERR_INVALID, "sparse_attention: unknown dtype %d", dtype);
  RT_REQUIRE(n_ctas > 0 && total_tokens > 0 && heads > 0, RT_ERR_INVALID, "sparse_attention: empty plan");
  const uint64_t rows = static_cast<uint64_t>(total_tokens) * heads;
  CUtensorMap mq, mk, mv;
  RT_TRY(make_tensor_map_2d(&mq, q, rows, 64, 64, 64, 64, true));
  RT_TRY(make_tensor_map_2d(&mk, k, rows, 64, 64, 64, 64, true));
  RT_TRY(make_tensor_map_2d(&mv, v, rows, 64, 64, 64, 64, true));
  int* err = error_word_dev ? error_word_dev : device_error_word();
  RT_REQUIRE(err != nullptr, RT_ERR_CUDA, "sparse_attention: cannot allocate the device error word");
  const float scale_log2 = scale * 1.4426950408889634f;
  const int hidden = heads * 64;
  if (dtype == RT_BF16) {
    RT_TRY(ensure_kernel_smem(reinterpret_cast<const void*>(sparse_attention_kernel<true>), kSmemBytes, true));
    RT_CHECK_CUDA(launch_kernel(sparse_attention_kernel<true>, dim3(n_ctas), dim3(kThreads), kSmemBytes, st, mq, mk, mv,
                                (uint16_t*)ctx, items_dev, entries_dev, cta_ptr_dev, hidden, scale_log2, err,
                                split.part_o, split.part_ml));
  } else {
    RT_TRY(ensure_kernel_smem(reinterpret_cast<const void*>(sparse_attention_kernel<false>), kSmemBytes, true));
    RT_CHECK_CUDA(launch_kernel(sparse_attention_kernel<false>, dim3(n_ctas), dim3(kThreads), kSmemBytes, st, mq, mk, mv,
                                (uint16_t*)ctx, items_dev, entries_dev, cta_ptr_dev, hidden, scale_log2, err,
                                split.part_o, split.part_ml));
  }
  count_launch();
  RT_CHECK_CUDA(cudaGetLastError());
  if (split.n_groups > 0) {
    RT_REQUIRE(split.groups_dev && split.part_o && split.part_ml, RT_ERR_INVALID,
               "sparse_attention: split lists without partial-result scratch");
    if (dtype == RT_BF16)
      RT_CHECK_CUDA(launch_kernel(merge_partials_kernel<true>, dim3(split.n_groups), dim3(128), 0, st, (uint16_t*)ctx,
                                  split.groups_dev, (const float*)split.part_o, (const float*)split.part_ml, hidden));
    else
      RT_CHECK_CUDA(launch_kernel(merge_partials_kernel<false>, dim3(split.n_groups), dim3(128), 0, st, (uint16_t*)ctx,
                                  split.groups_dev, (const float*)split.part_o, (const float*)split.part_ml, hidden));
    count_launch();
    RT_CHECK_CUDA(cudaGetLastError());
  }
  return RT_OK;
}

}  // namespace rt

// ---------------------------------------------------------------------------------------------
// C ABI: stand-alone attention plan + launch
// ---------------------------------------------------------------------------------------------
using namespace rt;

struct rt_attn_plan {
  AttnPlanHost host;
  uint8_t* dev = nullptr;
  size_t items_off = 0, entries_off = 0, cta_off = 0, groups_off = 0, part_o_off = 0, part_ml_off = 0, bytes = 0;
  int n_ctas = 0;
  int dtype = 0;
};

extern "C" rt_status rt_attn_plan_create(const rt_config* cfg, const int32_t* lens, int n_seq, const int32_t* kv_ptr,
                                         const int32_t* kv_idx, int n_ctas, int split_entries, void* stream,
                                         rt_attn_plan** out) {
  RT_REQUIRE(cfg && lens && kv_ptr && kv_idx && out, RT_ERR_INVALID, "attn_plan_create: null pointer");
  RT_TRY(check_config(cfg));
  RT_TRY(validate_lengths(*cfg, lens, n_seq));
  if (n_ctas <= 0) {
    int dev = 0;
    RT_CHECK_CUDA(cudaGetDevice(&dev));
    RT_CHECK_CUDA(cudaDeviceGetAttribute(&n_ctas, cudaDevAttrMultiProcessorCount, dev));
    n_ctas *= 2;  // two CTAs of the attention kernel are resident per SM
  }
  int nblk = 0;
  for (int s = 0; s < n_seq; ++s) nblk += lens[s] / cfg->block;
  const int64_t visits = kv_ptr[nblk];
  auto* p = new rt_attn_plan();
  const int split = split_entries < 0 ? kDefaultSplitEntries : split_entries;
  rt_status s = build_attn_plan(*cfg, lens, n_seq, kv_ptr, kv_idx, visits, n_ctas, p->host, split);
  if (s != RT_OK) {
    delete p;
    return s;
  }
  p->n_ctas = n_ctas;
  auto align = [](size_t x) { return (x + 255) & ~size_t(255); };
  p->items_off = 0;
  p->entries_off = align(p->host.items.size() * sizeof(AttnItem));
  p->cta_off = p->entries_off + align(p->host.entries.size() * sizeof(int32_t));
  p->groups_off = p->cta_off + align(p->host.cta_ptr.size() * sizeof(int32_t));
  p->part_o_off = p->groups_off + align(p->host.groups.size() * sizeof(int32_t));
  p->part_ml_off = p->part_o_off + align(static_cast<size_t>(p->host.n_slots) * 128 * 64 * sizeof(float));
  p->bytes = p->part_ml_off + align(static_cast<size_t>(p->host.n_slots) * 128 * 2 * sizeof(float)) + 256;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMalloc(&p->dev, p->bytes);
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(p->dev + p->items_off, p->host.items.data(), p->host.items.size() * sizeof(AttnItem),
                        cudaMemcpyHostToDevice, st);
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(p->dev + p->entries_off, p->host.entries.data(), p->host.entries.size() * sizeof(int32_t),
                        cudaMemcpyHostToDevice, st);
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(p->dev + p->cta_off, p->host.cta_ptr.data(), p->host.cta_ptr.size() * sizeof(int32_t),
                        cudaMemcpyHostToDevice, st);
  if (e == cudaSuccess && !p->host.groups.empty())
    e = cudaMemcpyAsync(p->dev + p->groups_off, p->host.groups.data(), p->host.groups.size() * sizeof(int32_t),
                        cudaMemcpyHostToDevice, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    if (p->dev) cudaFree(p->dev);
    delete p;
    return fail(RT_ERR_CUDA, "attn_plan_create: %s", cudaGetErrorString(e));
  }
  *out = p;
  return RT_OK;
}

extern "C" rt_status rt_attn_plan_destroy(rt_attn_plan* p) {
  if (!p) return RT_OK;
  if (p->dev) cudaFree(p->dev);
  delete p;
  return RT_OK;
}

extern "C" rt_status rt_attn_plan_stats(const rt_attn_plan* p, int64_t* entries_out, int64_t* visits_out,
                                        int32_t* items_out) {
  RT_REQUIRE(p != nullptr, RT_ERR_INVALID, "attn_plan_stats: null plan");
  if (entries_out) *entries_out = static_cast<int64_t>(p->host.entries.size());
  if (visits_out) *visits_out = p->host.visits;
  if (items_out) *items_out = static_cast<int32_t>(p->host.items.size());
  return RT_OK;
}

extern "C" rt_status rt_sparse_attention(void* ctx, const void* q, const void* k, const void* v,
                                         const rt_attn_plan* plan, float scale, int dtype, void* stream) {
  RT_REQUIRE(ctx && q && k && v && plan, RT_ERR_INVALID, "sparse_attention: null pointer");
  return launch_sparse_attention(ctx, q, k, v, reinterpret_cast<const AttnItem*>(plan->dev + plan->items_off),
                                 reinterpret_cast<const int32_t*>(plan->dev + plan->entries_off),
                                 reinterpret_cast<const int32_t*>(plan->dev + plan->cta_off), plan->n_ctas,
                                 plan->host.total_tokens, plan->host.heads, scale, dtype,
                                 static_cast<cudaStream_t>(stream), nullptr,
                                 AttnSplit{reinterpret_cast<const int32_t*>(plan->dev + plan->groups_off),
                                           static_cast<int>(plan->host.groups.size() / 6),
                                           reinterpret_cast<float*>(plan->dev + plan->part_o_off),
                                           reinterpret_cast<float*>(plan->dev + plan->part_ml_off)});
}
