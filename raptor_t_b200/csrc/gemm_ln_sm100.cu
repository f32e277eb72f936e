// Projection GEMM with the whole residual + bias + LayerNorm epilogue fused in:
//   out[M][N] = LayerNorm(A[M][K] W[N][K]^T + bias + residual) * gamma + beta,   N = 768 or 1024.
//
// The two N = hidden projections of a layer (attention output and FFN down) are each followed
// by a LayerNorm over the whole row (layers/multi_headed_attention.cpp:206-210,
// layers/bert_output.cpp:19-23).  A 256 x 256 CTA-pair tile holds only a quarter or a third of
// a row, so here a CLUSTER of N/256 CTA pairs owns a block of 256 complete rows: pair p computes
// columns [256 p, 256 p + 256) with the same cta_group::2 main loop as gemm_pair_sm100.cu, and
// the epilogue
//   1. adds bias and residual to the fp32 accumulator (kept in TMEM, never rounded to 16 bits),
//      and sums x and x^2 over the thread's columns,
//   2. sends those partial sums to every CTA of the cluster that holds the same rows
//      (distributed shared memory: st.shared::cluster + a remote mbarrier arrival per partial),
//   3. waits for all partials of its rows, forms mean and 1/sigma, normalises its columns and
//      stores the 16-bit result.
// The pre-LayerNorm sum therefore never reaches HBM, the separate LayerNorm launch disappears,
// and one 16-bit rounding per sub-layer with it.  No TMA multicast is used anywhere.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>

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
constexpr int kThreads = 320;           // warp 0 TMA, warp 1 MMA (pair leaders only), warps 2-9 epilogue
constexpr int kEpilogueThreads = 256;
constexpr int kTmemCols = 512;          // two 256-column accumulators
constexpr int kMaxNT = 4;               // N up to 1024
// row statistics: [accumulator parity][partial slot = n-tile * 2 + column-parity warp][row of this CTA] {sum, sum of squares}
constexpr int kStatsBytes = 2 * (2 * kMaxNT) * 128 * 8;
constexpr int kSmemBytes = kStages * kStageBytes + kStatsBytes + 1024 + 256;

__device__ __forceinline__ uint32_t map_to_rank(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f2(uint32_t cluster_addr, float a, float b) {
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(cluster_addr), "f"(a), "f"(b) : "memory");
}
// arrival that publishes this thread's earlier shared::cluster stores to whoever acquires the barrier
__device__ __forceinline__ void mbar_arrive_release_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_acquire_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait with cluster-scope acquire (the partial sums were written by other CTAs)
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, const AbortCtx& ab, int where) {
  if (mbar_try_wait_acquire_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait_acquire_cluster(bar, parity)) return true;
    if (*ab.cta_flag) return false;
    if (clock64() - t0 > ab.limit) break;
  }
  *ab.cta_flag = 1;
  atomicCAS(ab.global_flag, 0, where);
  return false;
}
// TMA load into THIS CTA's shared memory whose bytes are counted on the pair leader's barrier
__device__ __forceinline__ void tma_load_2d_to_leader(void* smem_dst, const CUtensorMap* m, int x, int y, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(leader_bar)
      : "memory");
}

template <bool BF16, int NT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_ln_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               uint16_t* __restrict__ out, const uint16_t* __restrict__ bias, const uint16_t* __restrict__ residual,
               const uint16_t* __restrict__ gamma, const uint16_t* __restrict__ beta, int M, int K, float eps,
               int* error_flag) {
  constexpr int N = NT * kTileN;
  constexpr int kSlots = 2 * NT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float2* stats = reinterpret_cast<float2*>(smem + kStages * kStageBytes);  // [2][2 * kMaxNT][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + kStatsBytes);
  uint64_t* full = bars;                  // the pair leader's copy is the one in use
  uint64_t* empty = bars + kStages;       // each CTA waits on its own copy
  uint64_t* acc_full = bars + 2 * kStages;
  uint64_t* acc_empty = acc_full + 2;     // the pair leader's copy collects both CTAs' epilogue threads
  uint64_t* stats_full = acc_empty + 2;   // every CTA's own: partial sums of its rows from all NT column tiles
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stats_full + 2);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  RT_PDL_LAUNCH_DEPENDENTS();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 .. 2 NT - 1
  const uint32_t pair = rank >> 1;               // column tile of this CTA's pair
  const uint32_t hrow = rank & 1;                // which 128 of the tile's 256 rows this CTA holds
  const uint32_t leader = rank & ~1u;            // cluster rank of the pair's MMA-issuing CTA
  const int cluster_id = blockIdx.x / (2 * NT);
  const int n_clusters = gridDim.x / (2 * NT);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * kEpilogueThreads);
      mbar_init(&stats_full[a], NT * (kEpilogueThreads / 32));  // one arrival per epilogue warp of every peer
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
  cluster_arrive();  // every peer's barriers exist before anything remote touches them
  cluster_wait();
  tc_fence_after_sync();
  RT_PDL_WAIT();  // operands, residual and the output buffer belong to the previous kernel until here
  const uint32_t tmem_base = *tmem_slot;
  AbortCtx ab{cta_abort, error_flag};

  const int n_tiles_m = (M + kTileM - 1) / kTileM;
  const int k_blocks = K / kBK;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer (every CTA)
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_w);
      uint32_t it = 0;
      bool ok = true;
      const int n0 = pair * kTileN + hrow * 128;
      for (int t = cluster_id; t < n_tiles_m && ok; t += n_clusters) {
        const int m0 = t * kTileM + hrow * 128;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, ab, 121)) { ok = false; break; }
          uint8_t* sa = smem + s * kStageBytes;
          if (hrow == 0) mbar_arrive_expect_tx(&full[s], 2 * kStageBytes);  // both CTAs' bytes
          const uint32_t leader_bar = map_to_rank(&full[s], leader);
          tma_load_2d_to_leader(sa, &map_a, kb * kBK, m0, leader_bar);
          tma_load_2d_to_leader(sa + kABytes, &map_w, kb * kBK, n0, leader_bar);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (pair leaders)
    // the whole warp walks the loop, one elected lane issues (see gemm_pair_sm100.cu)
    if (hrow == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kTileM, kTileN, BF16 ? 1 : 0, false);
      const uint16_t pair_mask = static_cast<uint16_t>(3u << leader);
      const bool elected = elect_one();
      const uint32_t smem_base = smem_u32(smem);
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int t = cluster_id; t < n_tiles_m && ok; t += n_clusters, ++tile_it) {
        const int a = tile_it & 1;
        const uint32_t aph = (tile_it >> 1) & 1;
        if (!mbar_wait(&acc_empty[a], aph ^ 1, ab, 122)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + a * kTileN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&full[s], ph, ab, 123)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + s * kStageBytes;
          const uint64_t da = make_smem_desc_sw128(sa);
          const uint64_t db = make_smem_desc_sw128(sa + kABytes);
          if (elected) {
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              mma_ss_pair(d_tmem, da + (k * 32 >> 4), db + (k * 32 >> 4), idesc, (kb | k) ? 1u : 0u);
            tc_commit_pair(&empty[s], pair_mask);  // slot free in both CTAs of the pair
          }
          __syncwarp();
        }
        if (ok && elected) tc_commit_pair(&acc_full[a], pair_mask);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue warps 2..9 (every CTA)
    const int quarter = warp & 3;          // TMEM lane quarter
    const int chunk0 = (warp - 2) >> 2;    // this warp takes the 32-column chunks chunk0, chunk0 + 2, ...
    const int row_local = quarter * 32 + lane;
    const uint32_t leader_acc_empty[2] = {map_to_rank(&acc_empty[0], leader), map_to_rank(&acc_empty[1], leader)};
    const int n0 = pair * kTileN;
    const int slot = pair * 2 + chunk0;
    uint32_t tile_it = 0;
    bool ok = true;
    for (int t = cluster_id; t < n_tiles_m && ok; t += n_clusters, ++tile_it) {
      const int a = tile_it & 1;
      const uint32_t aph = (tile_it >> 1) & 1;
      const int row = t * kTileM + hrow * 128 + row_local;
      const bool live = row < M;
      if (!mbar_wait(&acc_full[a], aph, ab, 124)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * kTileN;
      // pass 1: x = acc + bias + residual, back into TMEM in fp32; partial sums of x and x^2.
      // The residual of all of this thread's columns is requested up front (4 chunks x 64 bytes), so that
      // its latency is paid once per tile and not once per chunk.
      float sum = 0.f, sq = 0.f;
      constexpr int kMyChunks = kTileN / 64;  // 4
      uint4 res[kMyChunks][4];
#pragma unroll
      for (int ci = 0; ci < kMyChunks; ++ci) {
        const int c = chunk0 + 2 * ci;
        if (live) {
          const uint4* rp = reinterpret_cast<const uint4*>(residual + static_cast<size_t>(row) * N + n0 + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) res[ci][q] = rp[q];
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q) res[ci][q] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int ci = 0; ci < kMyChunks; ++ci) {
        const int c = chunk0 + 2 * ci;
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tc_wait_ld();
        const uint4* bv = reinterpret_cast<const uint4*>(bias + n0 + c * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 b4 = __ldg(bv + q);
          const uint32_t bw[4] = {b4.x, b4.y, b4.z, b4.w};
          const uint32_t rw[4] = {res[ci][q].x, res[ci][q].y, res[ci][q].z, res[ci][q].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 bb = unpack2<BF16>(bw[j]);
            const float2 rr = unpack2<BF16>(rw[j]);
            const float x0 = __uint_as_float(r[q * 8 + 2 * j]) + bb.x + rr.x;
            const float x1 = __uint_as_float(r[q * 8 + 2 * j + 1]) + bb.y + rr.y;
            sum += x0 + x1;
            sq = fmaf(x0, x0, fmaf(x1, x1, sq));
            r[q * 8 + 2 * j] = __float_as_uint(x0);
            r[q * 8 + 2 * j + 1] = __float_as_uint(x1);
          }
        }
        tmem_st32(taddr + c * 32, r);
      }
      tc_wait_st();
      // the partial sums go to every CTA that holds these rows (same hrow, every column tile)
#pragma unroll
      for (int p = 0; p < NT; ++p) {
        const uint32_t peer = static_cast<uint32_t>(2 * p) + hrow;
        float2* dst = stats + (a * (2 * kMaxNT) + slot) * 128 + row_local;
        st_cluster_f2(map_to_rank(dst, peer), sum, sq);
      }
      // one arrival per warp and peer (hundreds of arrivals on one barrier would be serialised at the target):
      // the warp barrier orders the lanes' stores before lane 0's releasing arrival
      __syncwarp();
      if (lane == 0) {
#pragma unroll
        for (int p = 0; p < NT; ++p)
          mbar_arrive_release_cluster(map_to_rank(&stats_full[a], static_cast<uint32_t>(2 * p) + hrow));
      }
      if (!mbar_wait_cluster(&stats_full[a], aph, ab, 125)) { ok = false; break; }
      float tot = 0.f, tot_sq = 0.f;
#pragma unroll
      for (int sl = 0; sl < kSlots; ++sl) {
        const float2 v = stats[(a * (2 * kMaxNT) + sl) * 128 + row_local];
        tot += v.x;
        tot_sq += v.y;
      }
      const float mean = tot * (1.0f / N);
      const float var = fmaxf(tot_sq * (1.0f / N) - mean * mean, 0.f);
      const float rstd = rsqrtf(var + eps);
      // pass 2: normalise this thread's columns and store them
#pragma unroll 1
      for (int c = chunk0; c < kTileN / 32; c += 2) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tc_wait_ld();
        const uint4* gv = reinterpret_cast<const uint4*>(gamma + n0 + c * 32);
        const uint4* ev = reinterpret_cast<const uint4*>(beta + n0 + c * 32);
        uint32_t o[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 g4 = __ldg(gv + q), e4 = __ldg(ev + q);
          const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, ew[4] = {e4.x, e4.y, e4.z, e4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 gg = unpack2<BF16>(gw[j]), ee = unpack2<BF16>(ew[j]);
            const float y0 = (__uint_as_float(r[q * 8 + 2 * j]) - mean) * rstd * gg.x + ee.x;
            const float y1 = (__uint_as_float(r[q * 8 + 2 * j + 1]) - mean) * rstd * gg.y + ee.y;
            o[q * 4 + j] = pack2<BF16>(y0, y1);
          }
        }
        if (live) {
          uint16_t* dst = out + static_cast<size_t>(row) * N + n0 + c * 32;
          st_global_v8(dst, o);
          st_global_v8(dst + 16, o + 8);
        }
      }
      tc_fence_before_sync();
      mbar_arrive_cluster(leader_acc_empty[a]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();  // nobody leaves while a peer may still write its shared memory or signal its barriers
  cluster_wait();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <bool BF16, int NT>
rt_status launch_ln(void* out, const void* a, const void* w, const void* bias, const void* residual, const void* gamma,
                    const void* beta, int M, int K, float eps, cudaStream_t st) {
  constexpr int N = NT * kTileN;
  CUtensorMap ma, mw;
  RT_TRY(make_tensor_map_2d(&ma, a, M, K, K, 128, kBK, true));
  RT_TRY(make_tensor_map_2d(&mw, w, N, K, K, 128, kBK, true));
  auto kern = gemm_ln_kernel<BF16, NT>;
  RT_TRY(ensure_kernel_smem(reinterpret_cast<const void*>(kern), kSmemBytes, false));
  int* err = device_error_word();
  RT_REQUIRE(err != nullptr, RT_ERR_CUDA, "gemm_layernorm: cannot allocate the device error word");
  const int m_tiles = (M + kTileM - 1) / kTileM;
  // as many clusters as the device keeps resident at once (the kernel is persistent over row blocks)
  static int resident[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (resident[dev] == 0) {
    cudaLaunchConfig_t q{};
    q.gridDim = dim3(gemm_sm_count() / (2 * NT) * 2 * NT);
    q.blockDim = dim3(kThreads);
    q.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2 * NT;
    qa[0].val.clusterDim.y = 1;
    qa[0].val.clusterDim.z = 1;
    q.attrs = qa;
    q.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &q) != cudaSuccess || n <= 0) n = gemm_sm_count() / (2 * NT);
    resident[dev] = n;
  }
  const int clusters = std::max(1, std::min(m_tiles, resident[dev]));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(clusters * 2 * NT);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2 * NT;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  RT_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, ma, mw, static_cast<uint16_t*>(out), static_cast<const uint16_t*>(bias),
                                   static_cast<const uint16_t*>(residual), static_cast<const uint16_t*>(gamma),
                                   static_cast<const uint16_t*>(beta), M, K, eps, err));
  count_launch();
  RT_CHECK_CUDA(cudaGetLastError());
  return RT_OK;
}

}  // namespace
}  // namespace rt

using namespace rt;

extern "C" rt_status rt_gemm_bias_residual_layernorm(void* out_dev, const void* a_dev, const void* w_dev,
                                                     const void* bias_dev, const void* residual_dev,
                                                     const void* gamma_dev, const void* beta_dev, int M, int N, int K,
                                                     float eps, int dtype, void* stream) {
  RT_REQUIRE(out_dev && a_dev && w_dev && bias_dev && residual_dev && gamma_dev && beta_dev, RT_ERR_INVALID,
             "gemm_layernorm: null pointer");
  RT_REQUIRE(N == 768 || N == 1024, RT_ERR_UNSUPPORTED, "gemm_layernorm: N must be 768 or 1024 (got %d)", N);
  RT_REQUIRE(M >= 0 && K > 0 && K % 64 == 0, RT_ERR_INVALID, "gemm_layernorm: need K %% 64 == 0 (got M=%d K=%d)", M, K);
  RT_REQUIRE(dtype == RT_F16 || dtype == RT_BF16, RT_ERR_INVALID, "gemm_layernorm: unknown dtype %d", dtype);
  const uintptr_t all = reinterpret_cast<uintptr_t>(out_dev) | reinterpret_cast<uintptr_t>(a_dev) |
                        reinterpret_cast<uintptr_t>(w_dev) | reinterpret_cast<uintptr_t>(bias_dev) |
                        reinterpret_cast<uintptr_t>(residual_dev) | reinterpret_cast<uintptr_t>(gamma_dev) |
                        reinterpret_cast<uintptr_t>(beta_dev);
  RT_REQUIRE((all & 31u) == 0, RT_ERR_INVALID, "gemm_layernorm: pointers must be 32-byte aligned");
  if (M == 0) return RT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool bf = dtype == RT_BF16;
  if (N == 768)
    return bf ? launch_ln<true, 3>(out_dev, a_dev, w_dev, bias_dev, residual_dev, gamma_dev, beta_dev, M, K, eps, st)
              : launch_ln<false, 3>(out_dev, a_dev, w_dev, bias_dev, residual_dev, gamma_dev, beta_dev, M, K, eps, st);
  return bf ? launch_ln<true, 4>(out_dev, a_dev, w_dev, bias_dev, residual_dev, gamma_dev, beta_dev, M, K, eps, st)
            : launch_ln<false, 4>(out_dev, a_dev, w_dev, bias_dev, residual_dev, gamma_dev, beta_dev, M, K, eps, st);
}
