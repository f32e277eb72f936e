// Persistent, warp-specialised tcgen05 GEMM for sm_100a:
//     C[M][N] = A[M][K] * W[N][K]^T  (+ bias) (+ GELU),  16-bit in/out, fp32 accumulate.
//
// One CTA per SM walks 128 x BN output tiles.  Warp 0 streams A and W k-slices
// (64 elements = one 128-byte swizzle atom) into a shared-memory ring with TMA;
// warp 1 issues tcgen05.mma (M=128, N=BN, K=16) into one of two TMEM
// accumulators; warps 2-9 drain the other accumulator (tcgen05.ld), apply the
// epilogue and store, so the epilogue of tile i overlaps the main loop of
// tile i+1.  Stands in for the cuBLAS calls of layers/kernels/mat_mul.cpp:58-76
// (which accumulate in fp16; this kernel accumulates in fp32).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>

#include "common.h"
#include "device_error.h"
#include "gemm_epilogue.cuh"
#include "launch.h"
#include "launch_count.h"
#include "sm100_ptx.cuh"
#include "tma_host.h"

namespace rt {

// SM count of the current device (queried once per device).
int gemm_sm_count() {
  static std::atomic<int> cache[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
    cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

namespace {

using namespace ptx;
using namespace gemm_detail;

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 320;      // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue
constexpr int kEpilogueThreads = 256;  // two warps per TMEM lane quarter, alternating 32-column chunks

template <int BN>
struct GemmCfg {
  static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;  // power of two: 128, 256, 512
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN, bool BF16, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
            uint16_t* __restrict__ C, const uint16_t* __restrict__ bias, int M, int N, int K, int* error_flag,
            QkvEpilogue qkv) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + Cfg::kStages;
  uint64_t* acc_full = bars + 2 * Cfg::kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  RT_PDL_LAUNCH_DEPENDENTS();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], kEpilogueThreads);
    }
    *cta_abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  RT_PDL_WAIT();  // operands and the output buffer belong to the previous kernel until here
  const uint32_t tmem_base = *tmem_slot;
  AbortCtx ab{cta_abort, error_flag};

  const int n_tiles_n = N / BN;
  const int n_tiles_m = (M + kBM - 1) / kBM;
  const int n_tiles = n_tiles_m * n_tiles_n;
  const int k_blocks = K / kBK;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_w);
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        const int m0 = (t / n_tiles_n) * kBM, n0 = (t % n_tiles_n) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % Cfg::kStages;
          const uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, ab, 101)) { ok = false; break; }
          uint8_t* sa = smem + s * Cfg::kStageBytes;
          mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
          tma_load_2d(sa, &map_a, kb * kBK, m0, &full[s]);
          tma_load_2d(sa + Cfg::kABytes, &map_w, kb * kBK, n0, &full[s]);
        }
      }
      // A wait only gives up after the whole pipeline has been idle for the full
      // time-out, so no copy issued by this thread can still be in flight here.
      (void)ok;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    // the whole warp walks the loop, one elected lane issues (see gemm_pair_sm100.cu)
    {
      constexpr uint32_t idesc = make_idesc_f16(kBM, BN, BF16 ? 1 : 0, false);
      const bool elected = elect_one();
      const uint32_t smem_base = smem_u32(smem);
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++tile_it) {
        const int a = tile_it & 1;
        const uint32_t aph = (tile_it >> 1) & 1;
        if (!mbar_wait(&acc_empty[a], aph ^ 1, ab, 102)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % Cfg::kStages;
          const uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait(&full[s], ph, ab, 103)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + s * Cfg::kStageBytes;
          const uint64_t da = make_smem_desc_sw128(sa);
          const uint64_t db = make_smem_desc_sw128(sa + Cfg::kABytes);
          if (elected) {
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              mma_ss(d_tmem, da + (k * 32 >> 4), db + (k * 32 >> 4), idesc, (kb | k) ? 1u : 0u);
            tc_commit(&empty[s]);
          }
          __syncwarp();
        }
        if (ok && elected) tc_commit(&acc_full[a]);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue warps 2..9
    const int quarter = warp & 3;
    const int chunk0 = (warp - 2) >> 2;  // 0: even 32-column chunks, 1: odd chunks
    const int row_in_tile = quarter * 32 + lane;
    uint32_t tile_it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++tile_it) {
      const int a = tile_it & 1;
      const uint32_t aph = (tile_it >> 1) & 1;
      const int m0 = (t / n_tiles_n) * kBM, n0 = (t % n_tiles_n) * BN;
      if (!mbar_wait(&acc_full[a], aph, ab, 104)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = m0 + row_in_tile;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * BN;
      epilogue_row<BN, BF16, EPI>(taddr, row, n0, chunk0, M, N, C, bias, qkv);
      tc_fence_before_sync();
      mbar_arrive(&acc_empty[a]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN, bool BF16, int EPI>
rt_status launch(void* c, const void* a, const void* w, const void* bias, int M, int N, int K, cudaStream_t st,
                 const QkvEpilogue& qkv = QkvEpilogue{}) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap ma, mw;
  RT_TRY(make_tensor_map_2d(&ma, a, M, K, K, kBM, kBK, true));
  RT_TRY(make_tensor_map_2d(&mw, w, N, K, K, BN, kBK, true));
  auto kern = gemm_kernel<BN, BF16, EPI>;
  RT_TRY(ensure_kernel_smem(reinterpret_cast<const void*>(kern), Cfg::kSmemBytes, false));
  int* err = device_error_word();
  RT_REQUIRE(err != nullptr, RT_ERR_CUDA, "gemm: cannot allocate the device error word");
  const int tiles = ((M + kBM - 1) / kBM) * (N / BN);
  const int grid = std::min(tiles, gemm_sm_count());
  RT_CHECK_CUDA(launch_kernel(kern, dim3(grid), dim3(kGemmThreads), Cfg::kSmemBytes, st, ma, mw, (uint16_t*)c,
                              (const uint16_t*)bias, M, N, K, err, qkv));
  count_launch();
  RT_CHECK_CUDA(cudaGetLastError());
  return RT_OK;
}

template <int BN, bool BF16>
rt_status launch_epi(void* c, const void* a, const void* w, const void* bias, int M, int N, int K, int epi,
                     cudaStream_t st, const QkvEpilogue& qkv = QkvEpilogue{}) {
  switch (epi) {
    case RT_EPI_NONE: return launch<BN, BF16, RT_EPI_NONE>(c, a, w, bias, M, N, K, st);
    case RT_EPI_BIAS: return launch<BN, BF16, RT_EPI_BIAS>(c, a, w, bias, M, N, K, st);
    case RT_EPI_BIAS_GELU: return launch<BN, BF16, RT_EPI_BIAS_GELU>(c, a, w, bias, M, N, K, st);
    case RT_EPI_BIAS_RESIDUAL: return launch<BN, BF16, RT_EPI_BIAS_RESIDUAL>(c, a, w, bias, M, N, K, st, qkv);
  }
  return fail(RT_ERR_INVALID, "gemm: unknown epilogue %d", epi);
}

}  // namespace

rt_status gemm_pair_dispatch(void* c, const void* a, const void* w, const void* bias, int M, int N, int K, int epi,
                             bool bf16, cudaStream_t st, const gemm_detail::QkvEpilogue& qkv);

// 256 x 256 CTA-pair tiles pay off when there are enough of them to fill the SM pairs.
static bool use_pair_tiles(int M, int N) {
  return N % 256 == 0 && ((M + 255) / 256) * (N / 256) >= gemm_sm_count() / 2;
}

}  // namespace rt

using namespace rt;

static rt_status gemm_entry(void* c, const void* a, const void* w, const void* bias, int M, int N, int K, int epilogue,
                            int dtype, void* stream, const gemm_detail::QkvEpilogue& extra) {
  RT_REQUIRE(c && a && w, RT_ERR_INVALID, "gemm: null pointer");
  RT_REQUIRE(M >= 0 && N > 0 && K > 0 && N % 64 == 0 && K % 64 == 0, RT_ERR_INVALID,
             "gemm: need N %% 64 == 0 and K %% 64 == 0 (got M=%d N=%d K=%d)", M, N, K);
  RT_REQUIRE(epilogue == RT_EPI_NONE || bias != nullptr, RT_ERR_INVALID, "gemm: epilogue needs a bias vector");
  RT_REQUIRE(((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(bias)) &
              15u) == 0 && (reinterpret_cast<uintptr_t>(c) & 31u) == 0,
             RT_ERR_INVALID, "gemm: A, W and bias must be 16-byte aligned, C 32-byte aligned");
  RT_REQUIRE(dtype == RT_F16 || dtype == RT_BF16, RT_ERR_INVALID, "gemm: unknown dtype %d", dtype);
  if (M == 0) return RT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (use_pair_tiles(M, N))
    return gemm_pair_dispatch(c, a, w, bias, M, N, K, epilogue, dtype == RT_BF16, st, extra);
  // largest tile width that divides N and still gives every SM a tile; else the narrowest
  const int sms = gemm_sm_count();
  const int mt = (M + kBM - 1) / kBM;
  int bn = 64;
  if (N % 256 == 0 && mt * (N / 256) >= sms) bn = 256;
  else if (N % 128 == 0 && mt * (N / 128) >= sms) bn = 128;
  const bool bf = dtype == RT_BF16;
  if (bn == 256) return bf ? launch_epi<256, true>(c, a, w, bias, M, N, K, epilogue, st, extra)
                           : launch_epi<256, false>(c, a, w, bias, M, N, K, epilogue, st, extra);
  if (bn == 128) return bf ? launch_epi<128, true>(c, a, w, bias, M, N, K, epilogue, st, extra)
                           : launch_epi<128, false>(c, a, w, bias, M, N, K, epilogue, st, extra);
  return bf ? launch_epi<64, true>(c, a, w, bias, M, N, K, epilogue, st, extra)
            : launch_epi<64, false>(c, a, w, bias, M, N, K, epilogue, st, extra);
}

extern "C" rt_status rt_gemm(void* c, const void* a, const void* w, const void* bias, int M, int N, int K, int epilogue,
                             int dtype, void* stream) {
  RT_REQUIRE(epilogue == RT_EPI_NONE || epilogue == RT_EPI_BIAS || epilogue == RT_EPI_BIAS_GELU, RT_ERR_INVALID,
             "gemm: unknown epilogue %d", epilogue);
  return gemm_entry(c, a, w, bias, M, N, K, epilogue, dtype, stream, gemm_detail::QkvEpilogue{});
}

extern "C" rt_status rt_gemm_residual(void* c, const void* a, const void* w, const void* bias, const void* residual,
                                      int M, int N, int K, int dtype, void* stream) {
  RT_REQUIRE(residual != nullptr && (reinterpret_cast<uintptr_t>(residual) & 15u) == 0, RT_ERR_INVALID,
             "gemm_residual: residual must be a 16-byte aligned device pointer");
  gemm_detail::QkvEpilogue e{};
  e.residual = static_cast<const uint16_t*>(residual);
  return gemm_entry(c, a, w, bias, M, N, K, RT_EPI_BIAS_RESIDUAL, dtype, stream, e);
}

extern "C" rt_status rt_gemm_qkv(void* q, void* k, void* v, const void* a, const void* w, const void* bias,
                                 const int32_t* block_seq_dev, int M, int heads, int K, float q_scale, int dtype,
                                 void* stream) {
  RT_REQUIRE(q && k && v && a && w && bias && block_seq_dev, RT_ERR_INVALID, "gemm_qkv: null pointer");
  const int N = 3 * heads * 64;
  RT_REQUIRE(M >= 0 && M % 64 == 0 && heads > 0 && K > 0 && K % 64 == 0, RT_ERR_INVALID,
             "gemm_qkv: need M %% 64 == 0 and K %% 64 == 0 (got M=%d heads=%d K=%d)", M, heads, K);
  RT_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
               reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(bias)) &
              31u) == 0,
             RT_ERR_INVALID, "gemm_qkv: pointers must be 32-byte aligned");
  RT_REQUIRE(dtype == RT_F16 || dtype == RT_BF16, RT_ERR_INVALID, "gemm_qkv: unknown dtype %d", dtype);
  if (M == 0) return RT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  QkvEpilogue e{nullptr, (uint16_t*)q, (uint16_t*)k, (uint16_t*)v, reinterpret_cast<const int2*>(block_seq_dev), heads,
                q_scale};
  if (use_pair_tiles(M, N)) return gemm_pair_dispatch(nullptr, a, w, bias, M, N, K, kEpiQkv, dtype == RT_BF16, st, e);
  const int mt = (M + kBM - 1) / kBM;
  // tile width must divide 3*heads*64 and keep a 32-column chunk inside one head: 64, 128 and 256 all do
  const int sms = gemm_sm_count();
  const bool wide = N % 256 == 0 && mt * (N / 256) >= sms;
  const bool mid = N % 128 == 0 && mt * (N / 128) >= sms;
  const bool bf = dtype == RT_BF16;
  if (wide) return bf ? launch<256, true, kEpiQkv>(nullptr, a, w, bias, M, N, K, st, e)
                      : launch<256, false, kEpiQkv>(nullptr, a, w, bias, M, N, K, st, e);
  if (mid) return bf ? launch<128, true, kEpiQkv>(nullptr, a, w, bias, M, N, K, st, e)
                     : launch<128, false, kEpiQkv>(nullptr, a, w, bias, M, N, K, st, e);
  return bf ? launch<64, true, kEpiQkv>(nullptr, a, w, bias, M, N, K, st, e)
            : launch<64, false, kEpiQkv>(nullptr, a, w, bias, M, N, K, st, e);
}
