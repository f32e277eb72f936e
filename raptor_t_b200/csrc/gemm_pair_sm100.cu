// Two-CTA (cta_group::2) variant of the tcgen05 GEMM: a cluster of two CTAs on neighbouring
// SMs computes one 256 x 256 output tile.  Each CTA loads its own 128 rows of A and its own
// 128 rows of W per 64-wide K slice (32 KB instead of the 48 KB a single-CTA 128 x 256 tile
// needs for the same MMA work), the leader CTA issues one M=256 N=256 K=16 MMA for the pair,
// and each CTA drains its own 128 accumulator rows.  The single-CTA kernel is bound by the
// L2 -> shared-memory traffic of its operand tiles; the pair moves a third less per FLOP.
//
// No TMA multicast is used: both CTAs issue plain (cta_group::2) loads of their own tiles
// whose byte counts land on the leader's barrier; tcgen05.commit multicasts the "slot free"
// and "accumulator ready" arrivals to both CTAs.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "common.h"
#include "device_error.h"
#include "gemm_epilogue.cuh"
#include "launch.h"
#include "launch_count.h"
#include "sm100_ptx.cuh"
#include "tma_host.h"

namespace rt {
int gemm_sm_count();  // gemm_sm100.cu
namespace {

using namespace ptx;
using namespace gemm_detail;

constexpr int kTileM = 256, kTileN = 256, kBK = 64;
constexpr int kStages = 6;
constexpr int kABytes = 128 * kBK * 2;  // this CTA's rows of A
constexpr int kBBytes = 128 * kBK * 2;  // this CTA's rows of W
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 320;           // warp 0 TMA, warp 1 MMA (leader only), warps 2-9 epilogue
constexpr int kEpilogueThreads = 256;
constexpr int kTmemCols = 512;          // two 256-column accumulators
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;

template <bool BF16, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                 uint16_t* __restrict__ C, const uint16_t* __restrict__ bias, int M, int N, int K, int* error_flag,
                 QkvEpilogue qkv) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full = bars;                  // leader's copy is the one in use
  uint64_t* empty = bars + kStages;       // each CTA waits on its own copy
  uint64_t* acc_full = bars + 2 * kStages;
  uint64_t* acc_empty = acc_full + 2;     // leader's copy collects both CTAs' epilogue threads
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  RT_PDL_LAUNCH_DEPENDENTS();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * kEpilogueThreads);
    }
    *cta_abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();  // the peer's barriers exist before anything remote touches them
  cluster_wait();
  tc_fence_after_sync();
  RT_PDL_WAIT();  // operands and the output buffer belong to the previous kernel until here
  const uint32_t tmem_base = *tmem_slot;
  AbortCtx ab{cta_abort, error_flag};

  const int n_tiles_n = N / kTileN;
  const int n_tiles_m = (M + kTileM - 1) / kTileM;
  const int n_tiles = n_tiles_m * n_tiles_n;
  const int k_blocks = K / kBK;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_w);
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < n_tiles && ok; t += n_pairs) {
        const int m0 = (t / n_tiles_n) * kTileM + rank * 128;
        const int n0 = (t % n_tiles_n) * kTileN + rank * 128;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, ab, 111)) { ok = false; break; }
          uint8_t* sa = smem + s * kStageBytes;
          if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * kStageBytes);  // both CTAs' bytes
          tma_load_2d_pair(sa, &map_a, kb * kBK, m0, &full[s]);
          tma_load_2d_pair(sa + kABytes, &map_w, kb * kBK, n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (leader CTA)
    // The whole warp walks the loop and one elected lane issues: descriptors and loop state are then
    // warp-uniform values, which the tensor-core instructions take directly (inside a single-lane branch
    // every descriptor is moved over from a per-thread register first, and that serial latency per
    // 64-wide K slice is of the order of the slice's 512 clocks of MMA work).
    if (rank == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kTileM, kTileN, BF16 ? 1 : 0, false);
      const bool leader = elect_one();
      const uint32_t smem_base = smem_u32(smem);
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int t = pair; t < n_tiles && ok; t += n_pairs, ++tile_it) {
        const int a = tile_it & 1;
        const uint32_t aph = (tile_it >> 1) & 1;
        if (!mbar_wait(&acc_empty[a], aph ^ 1, ab, 112)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + a * kTileN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&full[s], ph, ab, 113)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + s * kStageBytes;
          const uint64_t da = make_smem_desc_sw128(sa);
          const uint64_t db = make_smem_desc_sw128(sa + kABytes);
          if (leader) {
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              mma_ss_pair(d_tmem, da + (k * 32 >> 4), db + (k * 32 >> 4), idesc, (kb | k) ? 1u : 0u);
            tc_commit_pair(&empty[s], 3);  // slot free in both CTAs
          }
          __syncwarp();
        }
        if (ok && leader) tc_commit_pair(&acc_full[a], 3);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue warps 2..9 (both CTAs)
    const int quarter = warp & 3;
    const int chunk0 = (warp - 2) >> 2;
    const int row_in_tile = rank * 128 + quarter * 32 + lane;
    const uint32_t leader_acc_empty[2] = {leader_smem_u32(&acc_empty[0]), leader_smem_u32(&acc_empty[1])};
    uint32_t tile_it = 0;
    bool ok = true;
    for (int t = pair; t < n_tiles && ok; t += n_pairs, ++tile_it) {
      const int a = tile_it & 1;
      const uint32_t aph = (tile_it >> 1) & 1;
      const int m0 = (t / n_tiles_n) * kTileM, n0 = (t % n_tiles_n) * kTileN;
      if (!mbar_wait(&acc_full[a], aph, ab, 114)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = m0 + row_in_tile;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * kTileN;
      epilogue_row<kTileN, BF16, EPI>(taddr, row, n0, chunk0, M, N, C, bias, qkv);
      tc_fence_before_sync();
      mbar_arrive_cluster(leader_acc_empty[a]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();  // nobody leaves while its peer may still read its shared memory or signal its barriers
  cluster_wait();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <bool BF16, int EPI>
rt_status launch_pair(void* c, const void* a, const void* w, const void* bias, int M, int N, int K, cudaStream_t st,
                      const QkvEpilogue& qkv) {
  CUtensorMap ma, mw;
  RT_TRY(make_tensor_map_2d(&ma, a, M, K, K, 128, kBK, true));
  RT_TRY(make_tensor_map_2d(&mw, w, N, K, K, 128, kBK, true));
  auto kern = gemm_pair_kernel<BF16, EPI>;
  RT_TRY(ensure_kernel_smem(reinterpret_cast<const void*>(kern), kSmemBytes, false));
  int* err = device_error_word();
  RT_REQUIRE(err != nullptr, RT_ERR_CUDA, "gemm: cannot allocate the device error word");
  const int sms = gemm_sm_count();
  const int tiles = ((M + kTileM - 1) / kTileM) * (N / kTileN);
  const int pairs = std::min(tiles, sms / 2);
  RT_CHECK_CUDA(launch_kernel(kern, dim3(2 * pairs), dim3(kThreads), kSmemBytes, st, ma, mw, (uint16_t*)c,
                              (const uint16_t*)bias, M, N, K, err, qkv));
  count_launch();
  RT_CHECK_CUDA(cudaGetLastError());
  return RT_OK;
}

}  // namespace

// Entry used by rt_gemm / rt_gemm_qkv when the shape suits 256 x 256 pair tiles.
rt_status gemm_pair_dispatch(void* c, const void* a, const void* w, const void* bias, int M, int N, int K, int epi,
                             bool bf16, cudaStream_t st, const gemm_detail::QkvEpilogue& qkv) {
  switch (epi) {
    case RT_EPI_NONE:
      return bf16 ? launch_pair<true, RT_EPI_NONE>(c, a, w, bias, M, N, K, st, qkv)
                  : launch_pair<false, RT_EPI_NONE>(c, a, w, bias, M, N, K, st, qkv);
    case RT_EPI_BIAS:
      return bf16 ? launch_pair<true, RT_EPI_BIAS>(c, a, w, bias, M, N, K, st, qkv)
                  : launch_pair<false, RT_EPI_BIAS>(c, a, w, bias, M, N, K, st, qkv);
    case RT_EPI_BIAS_GELU:
      return bf16 ? launch_pair<true, RT_EPI_BIAS_GELU>(c, a, w, bias, M, N, K, st, qkv)
                  : launch_pair<false, RT_EPI_BIAS_GELU>(c, a, w, bias, M, N, K, st, qkv);
    case RT_EPI_BIAS_RESIDUAL:
      return bf16 ? launch_pair<true, RT_EPI_BIAS_RESIDUAL>(c, a, w, bias, M, N, K, st, qkv)
                  : launch_pair<false, RT_EPI_BIAS_RESIDUAL>(c, a, w, bias, M, N, K, st, qkv);
    case gemm_detail::kEpiQkv:
      return bf16 ? launch_pair<true, gemm_detail::kEpiQkv>(c, a, w, bias, M, N, K, st, qkv)
                  : launch_pair<false, gemm_detail::kEpiQkv>(c, a, w, bias, M, N, K, st, qkv);
  }
  return fail(RT_ERR_INVALID, "gemm: unknown epilogue %d", epi);
}

}  // namespace rt
