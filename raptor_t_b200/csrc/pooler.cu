// Pooler of the model head: pooled[s] = tanh(W hidden[first token of sequence s] + b).
//
// The reference keeps its pooler commented out (python/pybind.cpp:58-64,
// python/modeling_bert.py:281-300); its validation model applies
// tanh(Linear(sequence_output[:, 0, :])) (python/modeling_big_bird.py:1964, 2179).  On a
// padding-free varlen batch "token 0" of sequence s is the packed row seq_block_prefix[s] * 64.
// Tiny and bandwidth-trivial (one weight matrix read per batch): one warp per output element
// group, fp32 accumulation, 128-bit loads.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.h"
#include "launch.h"
#include "launch_count.h"

namespace rt {
namespace {

template <bool BF16>
__device__ __forceinline__ float2 unpack16x2(uint32_t w) {
  if constexpr (BF16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  else return __half22float2(*reinterpret_cast<__half2*>(&w));
}

// grid (hidden / 8, n_seq), 256 threads: warp w of a CTA produces output column blockIdx.x * 8 + w
template <bool BF16>
__global__ void __launch_bounds__(256) pooler_kernel(float* __restrict__ out, const uint16_t* __restrict__ hidden_states,
                                                     const int32_t* __restrict__ seq_block_prefix,
                                                     const uint16_t* __restrict__ w, const uint16_t* __restrict__ b,
                                                     int hidden) {
  RT_PDL_LAUNCH_DEPENDENTS();
  RT_PDL_WAIT();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 8 + warp;
  const int seq = blockIdx.y;
  const uint16_t* x = hidden_states + static_cast<size_t>(seq_block_prefix[seq]) * 64 * hidden;
  const uint16_t* wr = w + static_cast<size_t>(col) * hidden;
  float acc = 0.f;
  for (int k = lane * 8; k < hidden; k += 256) {
    const uint4 xv = *reinterpret_cast<const uint4*>(x + k);
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wr + k));
    const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, ws[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = unpack16x2<BF16>(xs[i]), c = unpack16x2<BF16>(ws[i]);
      acc = fmaf(a.x, c.x, fmaf(a.y, c.y, acc));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    const uint32_t bw = b[col];
    const float bias = BF16 ? __uint_as_float(bw << 16) : __half2float(*reinterpret_cast<const __half*>(&b[col]));
    out[static_cast<size_t>(seq) * hidden + col] = tanhf(acc + bias);
  }
}

}  // namespace
}  // namespace rt

using namespace rt;

extern "C" rt_status rt_pooler(float* pooled_dev, const void* hidden_dev, const int32_t* seq_block_prefix_dev, int n_seq,
                               const void* w_dev, const void* b_dev, int hidden, int dtype, void* stream) {
  RT_REQUIRE(pooled_dev && hidden_dev && seq_block_prefix_dev && w_dev && b_dev, RT_ERR_INVALID, "pooler: null pointer");
  RT_REQUIRE(n_seq > 0 && hidden > 0 && hidden % 8 == 0, RT_ERR_INVALID, "pooler: need n_seq > 0 and hidden %% 8 == 0");
  RT_REQUIRE(dtype == RT_F16 || dtype == RT_BF16, RT_ERR_INVALID, "pooler: unknown dtype %d", dtype);
  RT_REQUIRE(((reinterpret_cast<uintptr_t>(hidden_dev) | reinterpret_cast<uintptr_t>(w_dev)) & 15u) == 0, RT_ERR_INVALID,
             "pooler: hidden states and weight must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(hidden / 8, n_seq), block(256);
  if (dtype == RT_BF16)
    RT_CHECK_CUDA(launch_kernel(pooler_kernel<true>, grid, block, 0, st, pooled_dev, (const uint16_t*)hidden_dev,
                                seq_block_prefix_dev, (const uint16_t*)w_dev, (const uint16_t*)b_dev, hidden));
  else
    RT_CHECK_CUDA(launch_kernel(pooler_kernel<false>, grid, block, 0, st, pooled_dev, (const uint16_t*)hidden_dev,
                                seq_block_prefix_dev, (const uint16_t*)w_dev, (const uint16_t*)b_dev, hidden));
  count_launch();
  RT_CHECK_CUDA(cudaGetLastError());
  return RT_OK;
}
