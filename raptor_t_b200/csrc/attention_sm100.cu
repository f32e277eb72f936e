// Block-sparse attention for sm_100a (tcgen05 + TMEM + TMA), online softmax fused.
//
// A persistent CTA walks its list of work items.  An item is up to two 64-token query blocks
// of one (sequence, head) stacked into a 128-row tile, plus the merged list of 64-token
// key/value blocks they attend to (global, window and random blocks come from the same
// table; each entry carries a 2-bit mask that says which of the two query blocks uses it).
// The list is consumed TWO entries per step: one 128 x 128 score tile, one hand-off.
//
//   warp 4   loader (one thread): TMA loads of the Q tile per item and, per step, of two K
//            boxes and two V boxes (64 x 64, 128-byte swizzle) into adjacent shared-memory
//            tiles, so that a step's keys are one 128-row operand and its values one 128-row
//            operand.  The only role that reads the work list in global memory (4-byte
//            asynchronous copies, eight entries ahead); it publishes one record per step
//            ({entries, first/last flags, key/value rows}) in a shared-memory ring.
//   warp 5   MMA issuer, scores: S = Q K^T as M=128 N=128 K=64 (both operands K-major in
//            shared memory) into the score columns of TMEM.  The scores of step g+1 are
//            issued as soon as the softmax warps have pulled step g's scores into registers,
//            i.e. under their exponentials.
//   warp 6   MMA issuer, outputs: O += P V (P read from TMEM, V MN-major in shared memory) into
//            the output columns, in two halves per step, each as soon as that half of the
//            probabilities has been stored.  (tcgen05.mma blocks its issuing thread while the
//            tensor pipe's queue is full: with one issuing warp the output MMAs of a step sat
//            behind the score MMAs of the next.)
//   warps 0-3  softmax: thread r owns tile row r (TMEM lane r).  It pulls its score row out of
//            TMEM, keeps the running max / sum in fp32 (base-2 exponentials) and writes the
//            16-bit probabilities to their own TMEM columns.  The output tile accumulates in
//            TMEM across the whole list; it is rescaled only when a row's max has grown by
//            more than 2^8 since the last rescale ("lazy" rescaling: probabilities are then at
//            most 256, well inside 16-bit range), and read once per item for the final
//            division by the row sum.  Warps whose query block does not use an entry skip its
//            exponentials and keep zeros in its probability columns.  Every fourth pair of
//            exponentials is a cubic on the FMA pipe instead of the exponential unit.
// The kernel is launched with 128 registers per thread; the upper warpgroup hands registers
// to the softmax warps (setmaxnreg), which hold a 128-column score row each.
//
// Two CTAs share an SM (256 TMEM columns and ~113 KB of shared memory each): the exponentials
// (16 per clock per SM) bound the kernel, and one CTA's exponentials run under the other's
// loads, maxima and stores.
//
// Lists that are longer than one CTA's share of the batch are cut into parts by the host; a
// part leaves its un-normalised fp32 output tile, row maxima and row sums in scratch and
// merge_partials_kernel combines the parts of a list.
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

constexpr int kThreads = 256;            // warps 0-3 softmax; 4: loader, 5: score MMAs, 6: output MMAs; 7 only lends registers
constexpr int kStagesK = 2;              // K ring depth in steps (a slot is free again once the S MMA has read it)
constexpr int kStagesV = 3;              // V ring depth in steps (a slot is held until the PV MMA, a softmax period later)
constexpr int kStepRing = 16;            // per-step records travel from the loader to the other roles through smem
constexpr int kEntStage = 16;            // landing slots of the asynchronous work-list reads
constexpr int kEntAhead = 8;             // how many list entries the loader reads ahead
constexpr int kRecFirst = 1 << 29;       // record flags (in .x): first / last step of its item
constexpr int kRecLast = 1 << 30;
constexpr int kTileBytes = 64 * 64 * 2;  // one 64 x 64 16-bit block
constexpr int kStepBytes = 2 * kTileBytes;
constexpr int kTmemCols = 256;
constexpr int kColS = 0;     // 128 fp32 score columns (two key blocks)
constexpr int kColO = 128;   // 64 fp32 output columns, accumulated over the item's list
constexpr int kColP = 192;   // 64 columns of packed 16-bit probabilities (2 x 32)
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct Smem {
  uint8_t q[2][kStepBytes];
  uint8_t k[kStagesK][kStepBytes];
  uint8_t v[kStagesV][kStepBytes];
  uint64_t q_full[2], q_empty[2];
  uint64_t k_full[kStagesK], k_empty[kStagesK], v_full[kStagesV], v_empty[kStagesV];
  uint64_t s_full, s_free, p_full[2], pv_done, o_free;
  int4 step_ring[kStepRing];    // {entry 0 | flags, entry 1 or -1, key/value row of entry 0, of entry 1}
  int32_t ent_stage[kEntStage];
  uint32_t tmem_slot;
  int abort_flag;
};
constexpr int kSmemBytes = sizeof(Smem);
static_assert(kSmemBytes <= 113 * 1024, "two CTAs must fit one SM's shared memory");

// 4-byte asynchronous global -> shared copies: the loader thread reads its work list
// ahead without ever stalling on a global load.
__device__ __forceinline__ void cp_async_4(void* dst_smem, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ int steps_of(int n_entries) { return (n_entries + 1) >> 1; }

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

// Row maximum of 64 scores held in registers.
__device__ __forceinline__ float max64(const uint32_t* s) {
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
  return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
}

// 2^x for a pair of arguments on the FMA pipe (the exponential unit is the kernel's bottleneck, a part of
// the columns goes here instead): clamp, split x = n + f with |f| <= 0.5 by adding 1.5 * 2^23 (the integer
// lands in the low mantissa bits), 2^f by a cubic (relative error 7.5e-5, below the 16-bit rounding of the
// probabilities), n added to the exponent field.
__device__ __forceinline__ void ex2_fma_pair(float x0, float x1, float& r0, float& r1) {
  x0 = fmaxf(x0, -126.f);
  x1 = fmaxf(x1, -126.f);
  const unsigned long long x = f2_pack(x0, x1);
  const unsigned long long xr = f2_add(x, f2_pack(12582912.f, 12582912.f));
  const unsigned long long n = f2_add(xr, f2_pack(-12582912.f, -12582912.f));
  const unsigned long long f = f2_fma(n, f2_pack(-1.f, -1.f), x);
  unsigned long long r = f2_fma(f, f2_pack(0.05517167f, 0.05517167f), f2_pack(0.24261112f, 0.24261112f));
  r = f2_fma(r, f, f2_pack(0.69326099f, 0.69326099f));
  r = f2_fma(r, f, f2_pack(0.99992807f, 0.99992807f));
  float a0, a1, b0, b1;
  f2_unpack(r, a0, a1);
  f2_unpack(xr, b0, b1);
  r0 = __int_as_float(__float_as_int(a0) + (__float_as_int(b0) << 23));
  r1 = __int_as_float(__float_as_int(a1) + (__float_as_int(b1) << 23));
}

// p[i] = 2^(s[2i] * c - m), 2^(s[2i+1] * c - m) packed to 16 bits, for 64 scores; returns their sum.
// Every kPolyEvery-th pair is computed on the FMA pipe.
constexpr int kPolyEvery = 4;  // measured: 3 and 4 are equal within noise, 2 is slower (issue slots)
template <bool BF16>
__device__ __forceinline__ float exp64(const uint32_t* s, uint32_t* p, float scale_log2, float m_ref) {
  const unsigned long long c2 = f2_pack(scale_log2, scale_log2);
  const unsigned long long nm2 = f2_pack(-m_ref, -m_ref);
  unsigned long long acc0 = 0ull, acc1 = 0ull;  // two packed partial sums (+0.0f, +0.0f)
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const unsigned long long t = f2_fma(f2_pack(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), c2, nm2);
    float t0, t1;
    f2_unpack(t, t0, t1);
    float p0, p1;
    if (kPolyEvery > 0 && i % kPolyEvery == kPolyEvery - 1) {
      ex2_fma_pair(t0, t1, p0, p1);
    } else {
      p0 = ex2(t0);
      p1 = ex2(t1);
    }
    if (i & 1) acc1 = f2_add(acc1, f2_pack(p0, p1));
    else acc0 = f2_add(acc0, f2_pack(p0, p1));
    p[i] = pack2<BF16>(p0, p1);
  }
  float s0, s1;
  f2_unpack(f2_add(acc0, acc1), s0, s1);
  return s0 + s1;
}

// Register budget: the kernel is launched with 128 registers per thread (two CTAs of 256
// threads per SM); the upper warpgroup then gives registers back and the softmax warps,
// which hold a 128-column score row per thread, take them.
constexpr int kRegsIssue = 48;
constexpr int kRegsSoftmax = 208;
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
      mbar_init(&sm.p_full[i], 4);  // one elected arrival per softmax warp
    }
    mbar_init(&sm.s_full, 1);
    mbar_init(&sm.s_free, 4);
    mbar_init(&sm.pv_done, 1);
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

  if (warp >= 4) {
    reg_dealloc<kRegsIssue>();  // executed by all four warps of the upper warpgroup at this one place
    if (warp == 4) {
      // ------------------------------------------------------------------ loader
      // The only role that reads the work list in global memory: entries arrive through 4-byte
      // asynchronous copies issued kEntAhead entries early, the next item is prefetched in
      // registers.  A CTA's items are consecutive and so are their lists.
      if (lane == 0 && item_begin < item_end) {
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
        const int ent_first = items[item_begin].entry_off;
        const AttnItem& zi = items[item_end - 1];
        const uint32_t total = static_cast<uint32_t>(zi.entry_off + zi.n_entries - ent_first);
        const int32_t* ent = entries + ent_first;
        auto fetch = [&](uint32_t i) {
          if (i < total) cp_async_4(&sm.ent_stage[i % kEntStage], ent + i);
          cp_async_commit();  // one group per entry, empty past the end: the wait below counts groups
        };
        for (uint32_t i = 0; i < kEntAhead; ++i) fetch(i);
        auto next_entry = [&](uint32_t i) {
          cp_async_wait<kEntAhead - 1>();  // the copy of entry i has landed
          const int e = *reinterpret_cast<volatile int32_t*>(&sm.ent_stage[i % kEntStage]);
          fetch(i + kEntAhead);
          return e;
        };
        uint32_t e_g = 0, step = 0, itn = 0;
        AttnItem it = items[item_begin];
        bool ok = true;
        for (int idx = item_begin; ok && idx < item_end; ++idx) {
          AttnItem nxt{};
          if (idx + 1 < item_end) nxt = items[idx + 1];  // in flight while this item's steps are issued
          const int n = it.n_entries;
          if (n > 0) {
            const int qb = itn & 1;
            if (!mbar_wait(&sm.q_empty[qb], ((itn >> 1) & 1) ^ 1, ab, 211)) break;
            mbar_arrive_expect_tx(&sm.q_full[qb], kStepBytes);
            tma_load_2d(sm.q[qb], &map_q, 0, it.q_row0, &sm.q_full[qb]);
            tma_load_2d(sm.q[qb] + kTileBytes, &map_q, 0, it.q_row1, &sm.q_full[qb]);
            for (int j = 0; j < n; j += 2, ++step) {
              const bool two = j + 1 < n;
              const int sk = step % kStagesK, sv = step % kStagesV;
              if (!mbar_wait(&sm.k_empty[sk], ((step / kStagesK) & 1) ^ 1, ab, 212)) { ok = false; break; }
              const int e0 = next_entry(e_g++);
              const int e1 = two ? next_entry(e_g++) : -1;
              const int row0 = it.kv_row0 + (e0 >> 2) * 64;
              const int row1 = two ? it.kv_row0 + (e1 >> 2) * 64 : row0;
              sm.step_ring[step % kStepRing] =
                  make_int4(e0 | (j == 0 ? kRecFirst : 0) | (j + 2 >= n ? kRecLast : 0), e1, row0, row1);
              // the record is written before the barrier is armed: whoever sees the keys arrive sees the record
              mbar_arrive_expect_tx(&sm.k_full[sk], two ? kStepBytes : kTileBytes);
              tma_load_2d(sm.k[sk], &map_k, 0, row0, &sm.k_full[sk]);
              if (two) tma_load_2d(sm.k[sk] + kTileBytes, &map_k, 0, row1, &sm.k_full[sk]);
              if (!mbar_wait(&sm.v_empty[sv], ((step / kStagesV) & 1) ^ 1, ab, 213)) { ok = false; break; }
              mbar_arrive_expect_tx(&sm.v_full[sv], two ? kStepBytes : kTileBytes);
              tma_load_2d(sm.v[sv], &map_v, 0, row0, &sm.v_full[sv]);
              if (two) tma_load_2d(sm.v[sv] + kTileBytes, &map_v, 0, row1, &sm.v_full[sv]);
            }
            ++itn;
          }
          it = nxt;
        }
        cp_async_wait<0>();
      }
    } else if (warp == 5) {
      // ------------------------------------------------------------------ MMA issuer, scores
      // The whole warp walks the loop (waits included) and one elected lane issues the MMAs and
      // commits: loop state and descriptors are then warp-uniform values, which the tensor-core
      // instructions take directly.  Scores and outputs have an issuing warp each: tcgen05.mma
      // blocks while the tensor pipe's queue is full, and one warp issuing both kinds held the
      // output MMAs of step g behind the score MMAs of step g+1 (and the reverse).
      if (item_begin < item_end) {
        const bool leader = elect_one();
        constexpr uint32_t idesc_s128 = make_idesc_f16(128, 128, BF16 ? 1 : 0, false);
        constexpr uint32_t idesc_s64 = make_idesc_f16(128, 64, BF16 ? 1 : 0, false);
        uint32_t total_steps = 0;
        for (int idx = item_begin; idx < item_end; ++idx) total_steps += steps_of(items[idx].n_entries);
        uint32_t s_itn = 0;
        const uint32_t q_addr = smem_u32(sm.q[0]), k_addr = smem_u32(sm.k[0]);
        for (uint32_t g = 0; g < total_steps; ++g) {
          // S = Q K^T of step g into the score columns, free once the softmax warps hold step g-1's scores
          if (g > 0) {
            if (!mbar_wait(&sm.s_free, (g - 1) & 1, ab, 220)) break;
          }
          const int sk = g % kStagesK;
          if (!mbar_wait(&sm.k_full[sk], (g / kStagesK) & 1, ab, 218)) break;
          const int4 rec = sm.step_ring[g % kStepRing];
          const int qb = s_itn & 1;
          if (rec.x & kRecFirst) {
            if (!mbar_wait(&sm.q_full[qb], (s_itn >> 1) & 1, ab, 219)) break;
          }
          tc_fence_after_sync();
          const uint64_t dq = make_smem_desc_sw128(q_addr + qb * kStepBytes);
          const uint64_t dk = make_smem_desc_sw128(k_addr + sk * kStepBytes);
          const uint32_t d = tmem_base + kColS;
          if (leader) {
            if (rec.y >= 0) {
#pragma unroll
              for (int k = 0; k < 4; ++k) mma_ss(d, dq + (k * 32 >> 4), dk + (k * 32 >> 4), idesc_s128, k ? 1u : 0u);
            } else {
#pragma unroll
              for (int k = 0; k < 4; ++k) mma_ss(d, dq + (k * 32 >> 4), dk + (k * 32 >> 4), idesc_s64, k ? 1u : 0u);
            }
            tc_commit(&sm.k_empty[sk]);
            tc_commit(&sm.s_full);
            if (rec.x & kRecLast) tc_commit(&sm.q_empty[qb]);
          }
          if (rec.x & kRecLast) ++s_itn;
          __syncwarp();
        }
      }
    } else if (warp == 6) {
      // ------------------------------------------------------------------ MMA issuer, outputs
      if (item_begin < item_end) {
        const bool leader = elect_one();
        constexpr uint32_t idesc_pv = make_idesc_f16(128, 64, BF16 ? 1 : 0, true);
        uint32_t total_steps = 0;
        for (int idx = item_begin; idx < item_end; ++idx) total_steps += steps_of(items[idx].n_entries);
        uint32_t pv_itn = 0;
        const uint32_t v_addr = smem_u32(sm.v[0]);
        for (uint32_t g = 0; g < total_steps; ++g) {
          const int sv = g % kStagesV;
          // the loader published the step's record before it armed the key barrier, and arms this one later
          if (!mbar_wait(&sm.v_full[sv], (g / kStagesV) & 1, ab, 214)) break;
          const int4 rec = sm.step_ring[g % kStepRing];
          const bool first = (rec.x & kRecFirst) != 0;
          if (first) {
            // the output tile is overwritten: the softmax warps must have read the previous item's result
            if (!mbar_wait(&sm.o_free, (pv_itn & 1) ^ 1, ab, 215)) break;
          }
          const uint32_t d = tmem_base + kColO;
          const uint32_t a = tmem_base + kColP;
          const uint64_t dv = make_smem_desc_sw128(v_addr + sv * kStepBytes);
          if (!mbar_wait(&sm.p_full[0], g & 1, ab, 216)) break;
          tc_fence_after_sync();
          if (leader) {
            if (first) {
#pragma unroll
              for (int k = 0; k < 4; ++k) mma_ts(d, a + k * 8, dv + (k * 2048 >> 4), idesc_pv, k ? 1u : 0u);
            } else {
#pragma unroll
              for (int k = 0; k < 4; ++k) mma_ts(d, a + k * 8, dv + (k * 2048 >> 4), idesc_pv, 1u);
            }
          }
          if (!mbar_wait(&sm.p_full[1], g & 1, ab, 217)) break;
          tc_fence_after_sync();
          if (leader) {
            if (rec.y >= 0) {  // a single-entry step has nothing in its second half
#pragma unroll
              for (int k = 0; k < 4; ++k)
                mma_ts(d, a + 32 + k * 8, dv + ((kTileBytes + k * 2048) >> 4), idesc_pv, 1u);
            }
            tc_commit(&sm.v_empty[sv]);
            tc_commit(&sm.pv_done);
          }
          if (rec.x & kRecLast) ++pv_itn;
          __syncwarp();
        }
      }
    }
  } else {
    reg_alloc<kRegsSoftmax>();
    // ------------------------------------------------------------------ softmax warps 0..3
    const int row = warp * 32 + lane;  // tile row == TMEM lane
    const int half = row >> 6;         // 0: query block A, 1: query block B
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    uint32_t g = 0;
    bool ok = true;
    bool pzero0 = false, pzero1 = false;  // this warp's probability columns of half-step 0 / 1 hold zeros
    // only the fields the softmax warps need: {n_entries, out_tok0, out_tok1, head}
    auto load_item = [&](int idx) {
      const int4 hi = reinterpret_cast<const int4*>(items + idx)[1];
      return hi;
    };
    int4 next_item = item_begin < item_end ? load_item(item_begin) : make_int4(0, 0, 0, 0);
    for (int it = item_begin; it < item_end && ok; ++it) {
      const int4 item = next_item;
      if (it + 1 < item_end) next_item = load_item(it + 1);  // in flight while this item is processed
      const int n_steps = steps_of(item.x);
      if (n_steps == 0) continue;
      float m_ref = -INFINITY;  // max the stored probabilities / output are relative to (log2 units)
      float l = 0.f;
      for (int j = 0; j < n_steps; ++j) {
        const uint32_t gj = g + j;
        if (!mbar_wait(&sm.s_full, gj & 1, ab, 221)) { ok = false; break; }
        tc_fence_after_sync();
        // the loader published this step's record before it loaded the keys of the score tile just waited for
        const int4 rec = sm.step_ring[gj % kStepRing];
        const bool two = rec.y >= 0;
        const bool act0 = ((rec.x >> half) & 1) != 0;
        const bool act1 = two && ((rec.y >> half) & 1) != 0;
        // always the whole row: loads under a condition leave the registers "maybe defined", which costs the
        // register allocator dozens of registers; unused columns are simply ignored
        uint32_t s[128];
        tmem_ld32(lane_base + kColS, s);
        tmem_ld32(lane_base + kColS + 32, s + 32);
        tmem_ld32(lane_base + kColS + 64, s + 64);
        tmem_ld32(lane_base + kColS + 96, s + 96);
        tc_wait_ld();
        // the score columns may be overwritten by the next step's S MMA
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.s_free);

        float alpha = 1.f;
        bool fix = false;
        if (act0 || act1) {
          float mx = -INFINITY;
          if (act0) mx = max64(s);
          if (act1) mx = fmaxf(mx, max64(s + 64));
          const float m_new = mx * scale_log2;
          if (m_ref == -INFINITY) {
            m_ref = m_new;  // nothing accumulated for this row yet (its output columns are still zero)
          } else if (m_new > m_ref + kRescaleThreshold) {
            alpha = ex2(m_ref - m_new);
            m_ref = m_new;
            fix = true;
          }
        }
        uint32_t p[32];
        if (act0) l = l * alpha + exp64<BF16>(s, p, scale_log2, m_ref);
        else l *= alpha;
        // the probability columns were last read by the PV MMAs of the previous step; with those complete the
        // output tile is at rest too
        if (j > 0) {
          if (!mbar_wait(&sm.pv_done, (gj - 1) & 1, ab, 223)) { ok = false; break; }
          tc_fence_after_sync();
        }
        if (__any_sync(0xffffffffu, fix) && j > 0) {
          // rescale this warp's rows of the output tile
#pragma unroll 1
          for (int c = 0; c < 64; c += 16) {
            uint32_t o[16];
            tmem_ld16(lane_base + kColO + c, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st16(lane_base + kColO + c, o);
          }
        }
        if (act0) {
          tmem_st32(lane_base + kColP, p);
          pzero0 = false;
        } else if (!pzero0) {
#pragma unroll
          for (int i = 0; i < 32; ++i) p[i] = 0u;
          tmem_st32(lane_base + kColP, p);
          pzero0 = true;
        }
        tc_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.p_full[0]);
        if (two) {
          if (act1) {
            l += exp64<BF16>(s + 64, p, scale_log2, m_ref);
            tmem_st32(lane_base + kColP + 32, p);
            pzero1 = false;
          } else if (!pzero1) {
#pragma unroll
            for (int i = 0; i < 32; ++i) p[i] = 0u;
            tmem_st32(lane_base + kColP + 32, p);
            pzero1 = true;
          }
          tc_wait_st();
          tc_fence_before_sync();
          __syncwarp();
        }
        if (lane == 0) mbar_arrive(&sm.p_full[1]);
      }
      if (!ok) break;
      g += n_steps;
      // final: the last PV MMA of the item completes the output tile
      if (!mbar_wait(&sm.pv_done, (g - 1) & 1, ab, 224)) { ok = false; break; }
      tc_fence_after_sync();
      const int tok0 = half == 0 ? item.y : item.z;
      const int slot = (item.w >> 8) - 1;  // >= 0: this item is one part of a split list
      const float inv = slot >= 0 ? 1.0f : 1.0f / l;
      uint16_t* dst = ctx + static_cast<size_t>((tok0 >= 0 ? tok0 : 0) + (row & 63)) * hidden + (item.w & 255) * 64;
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
    }
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
