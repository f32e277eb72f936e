// Memory-bound kernels of the encoder layer: residual + bias + LayerNorm,
// bias + GELU(tanh), QKV bias + scale + split + head-major transpose, and the
// embedding gather + LayerNorm.  All of them move 128-bit vectors, keep
// statistics in fp32 and are sized against HBM bandwidth, not FLOPs.
//
// Reference counterparts: layers/kernels/add_bias_and_layernorm.cu:191-285,
// layers/kernels/add_bias_act.cu:86-133, layers/kernels/add_bias_and_transpose.cu:118-233,
// python/modeling_bert.py:45-60.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.h"
#include "launch.h"
#include "launch_count.h"

namespace rt {
namespace {

template <typename T>
struct Vec8;  // 8 x 16-bit = 128 bits

template <>
struct Vec8<__half> {
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return v;
  }
};

template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------------------
// residual + bias + LayerNorm: one warp per row, NV 128-bit vectors per lane.
// Two-pass statistics on the register copy (mean, then sum of squared
// deviations), fp32 throughout.  Warps walk rows with a grid stride; bias, gamma
// and beta are staged once per CTA in shared memory so that the kernel keeps few
// registers and many warps (loads in flight) per SM.
// ---------------------------------------------------------------------------
template <typename T, int NV>
__global__ void __launch_bounds__(256, (NV <= 4 ? 3 : 2))
layernorm_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ bias,
                 const T* __restrict__ residual, const T* __restrict__ gamma, const T* __restrict__ beta, int rows,
                 int hidden, float eps) {
  // bias, gamma and beta sit in shared memory: re-read per row at shared-memory latency
  // without holding registers across rows
  extern __shared__ uint4 s_par[];  // [3][hidden / 8]
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int warp = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int total_warps = gridDim.x * warps_per_block;
  const int vecs = hidden >> 3;
  const float inv_h = 1.0f / static_cast<float>(hidden);
  RT_PDL_LAUNCH_DEPENDENTS();
  uint4* s_bias = s_par;
  uint4* s_gamma = s_par + vecs;
  uint4* s_beta = s_par + 2 * vecs;
  for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
    s_bias[i] = bias ? reinterpret_cast<const uint4*>(bias)[i] : make_uint4(0, 0, 0, 0);
    s_gamma[i] = reinterpret_cast<const uint4*>(gamma)[i];
    s_beta[i] = reinterpret_cast<const uint4*>(beta)[i];
  }
  __syncthreads();
  RT_PDL_WAIT();

  for (int row = warp; row < rows; row += total_warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * hidden);
    const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + static_cast<size_t>(row) * hidden) : nullptr;
    uint4 xv[NV], rv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < vecs) {
        xv[i] = xr[c];
        rv[i] = rr ? rr[c] : make_uint4(0, 0, 0, 0);
      }
    }
    float v[NV][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < vecs) {
        float a[8], r[8], bb[8];
        Vec8<T>::unpack(xv[i], a);
        Vec8<T>::unpack(rv[i], r);
        Vec8<T>::unpack(s_bias[c], bb);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          v[i][k] = a[k] + bb[k] + r[k];
          sum += v[i][k];
        }
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[i][k] = 0.f;
      }
    }
    const float mean = warp_sum(sum) * inv_h;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < vecs) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float d = v[i][k] - mean;
          sq += d * d;
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) * inv_h + eps);
    uint4* orow = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * hidden);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < vecs) {
        float gg[8], be[8], o[8];
        Vec8<T>::unpack(s_gamma[c], gg);
        Vec8<T>::unpack(s_beta[c], be);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = (v[i][k] - mean) * rstd * gg[k] + be[k];
        orow[c] = Vec8<T>::pack(o);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// bias + GELU (tanh form), in place, one 128-bit vector per thread per step.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}

template <typename T, int UNROLL>
__global__ void __launch_bounds__(256) bias_gelu_kernel(T* __restrict__ x, const T* __restrict__ bias,
                                                        size_t total_vecs, int vecs_per_row) {
  RT_PDL_LAUNCH_DEPENDENTS();
  RT_PDL_WAIT();
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  uint4* xv = reinterpret_cast<uint4*>(x);
  const uint4* bv = reinterpret_cast<const uint4*>(bias);
  for (; i + (UNROLL - 1) * stride < total_vecs; i += UNROLL * stride) {
    uint4 a[UNROLL], b[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      a[u] = xv[i + u * stride];
      b[u] = bv[(i + u * stride) % vecs_per_row];
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float f[8], bb[8];
      Vec8<T>::unpack(a[u], f);
      Vec8<T>::unpack(b[u], bb);
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = gelu_tanh(f[k] + bb[k]);
      xv[i + u * stride] = Vec8<T>::pack(f);
    }
  }
  for (; i < total_vecs; i += stride) {
    float f[8], bb[8];
    Vec8<T>::unpack(xv[i], f);
    Vec8<T>::unpack(bv[i % vecs_per_row], bb);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = gelu_tanh(f[k] + bb[k]);
    xv[i] = Vec8<T>::pack(f);
  }
}

// ---------------------------------------------------------------------------
// QKV bias + scale + split + transpose to per-sequence head-major layout.
// One CTA per (64-token block, q|k|v part).  Every 128-byte chunk (one token,
// one head) is read and written whole, so both sides are fully coalesced.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) qkv_transpose_kernel(const T* __restrict__ qkv, const T* __restrict__ bias,
                                                            T* __restrict__ q, T* __restrict__ k, T* __restrict__ v,
                                                            const int32_t* __restrict__ seq_prefix, int n_seq,
                                                            int heads, float q_scale) {
  RT_PDL_LAUNCH_DEPENDENTS();
  RT_PDL_WAIT();
  const int blk = blockIdx.x;   // packed 64-token block
  const int part = blockIdx.y;  // 0 q, 1 k, 2 v
  __shared__ int s_first_blk, s_nblk;
  if (threadIdx.x == 0) {
    int lo = 0, hi = n_seq;  // largest s with seq_prefix[s] <= blk
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (seq_prefix[mid] <= blk) lo = mid; else hi = mid;
    }
    s_first_blk = seq_prefix[lo];
    s_nblk = seq_prefix[lo + 1] - seq_prefix[lo];
  }
  __syncthreads();
  const int hidden = heads * 64;
  const int vec_per_part = hidden >> 3;                 // vectors per token in this part
  const int seq_tok0 = s_first_blk * 64;
  const int seq_len = s_nblk * 64;
  const int tok_in_seq0 = (blk - s_first_blk) * 64;
  T* dst_base = (part == 0 ? q : part == 1 ? k : v) + static_cast<size_t>(seq_tok0) * hidden;
  const float scale = part == 0 ? q_scale : 1.0f;
  const uint4* src = reinterpret_cast<const uint4*>(qkv);
  const uint4* bsrc = reinterpret_cast<const uint4*>(bias) + part * vec_per_part;
  const int total = 64 * vec_per_part;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int t = i / vec_per_part;       // token in block
    const int c = i - t * vec_per_part;   // vector in this part's row
    const int h = c >> 3, dv = c & 7;
    const size_t tok = static_cast<size_t>(blk) * 64 + t;
    const uint4 a = src[tok * (3 * vec_per_part) + part * vec_per_part + c];
    float f[8], bb[8];
    Vec8<T>::unpack(a, f);
    if (bias) {
      Vec8<T>::unpack(bsrc[c], bb);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = (f[e] + bb[e]) * scale;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] *= scale;
    }
    const size_t row = static_cast<size_t>(h) * seq_len + tok_in_seq0 + t;
    reinterpret_cast<uint4*>(dst_base + row * 64)[dv] = Vec8<T>::pack(f);
  }
}

// ---------------------------------------------------------------------------
// embeddings: fp32 tables, one warp per token, same statistics as LayerNorm.
// ---------------------------------------------------------------------------
template <typename T, int NV>
__global__ void __launch_bounds__(256) embeddings_kernel(T* __restrict__ out, const int32_t* __restrict__ ids,
                                                         const int32_t* __restrict__ pos_ids,
                                                         const int32_t* __restrict__ type_ids,
                                                         const float* __restrict__ word, const float* __restrict__ pos,
                                                         const float* __restrict__ type, const float* __restrict__ gamma,
                                                         const float* __restrict__ beta, int tokens, int hidden,
                                                         float eps) {
  RT_PDL_LAUNCH_DEPENDENTS();
  RT_PDL_WAIT();
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp >= tokens) return;
  const int vecs = hidden >> 3;
  const size_t wi = static_cast<size_t>(ids[warp]) * hidden;
  const size_t pi = static_cast<size_t>(pos_ids ? pos_ids[warp] : 0) * hidden;
  const size_t ti = static_cast<size_t>(type_ids ? type_ids[warp] : 0) * hidden;
  float v[NV][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
#pragma unroll
    for (int k = 0; k < 8; ++k) v[i][k] = 0.f;
    if (c < vecs) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const float4 a = *reinterpret_cast<const float4*>(word + wi + c * 8 + half * 4);
        const float4 p = *reinterpret_cast<const float4*>(pos + pi + c * 8 + half * 4);
        const float4 t = *reinterpret_cast<const float4*>(type + ti + c * 8 + half * 4);
        v[i][half * 4 + 0] = a.x + t.x + p.x;
        v[i][half * 4 + 1] = a.y + t.y + p.y;
        v[i][half * 4 + 2] = a.z + t.z + p.z;
        v[i][half * 4 + 3] = a.w + t.w + p.w;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) sum += v[i][k];
    }
  }
  const float inv_h = 1.0f / static_cast<float>(hidden);
  const float mean = warp_sum(sum) * inv_h;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + 32 * i < vecs) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float d = v[i][k] - mean;
        sq += d * d;
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) * inv_h + eps);
  uint4* orow = reinterpret_cast<uint4*>(out + static_cast<size_t>(warp) * hidden);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < vecs) {
      float o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = (v[i][k] - mean) * rstd * gamma[c * 8 + k] + beta[c * 8 + k];
      orow[c] = Vec8<T>::pack(o);
    }
  }
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

template <typename T>
static rt_status layernorm_launch(void* out, const void* x, const void* bias, const void* residual, const void* gamma,
                                  const void* beta, int rows, int hidden, float eps, cudaStream_t st) {
  const int nv = (hidden / 8 + 31) / 32;
  const int threads = 256, wpb = threads / 32;
  // at most two waves of resident CTAs (3 per SM); warps walk the rows with a grid stride, so the
  // parameters are staged in shared memory a few times per SM instead of once per 8 rows
  int blocks = std::min((rows + wpb - 1) / wpb, sm_count() * 6);
  if (blocks < 1) blocks = 1;
#define RT_LN_CASE(NV)                                                                                           \
  case NV:                                                                                                       \
    launch_kernel(layernorm_kernel<T, NV>, dim3(blocks), dim3(threads), 3 * (hidden / 8) * sizeof(uint4), st,   \
                  (T*)out, (const T*)x, (const T*)bias, (const T*)residual, (const T*)gamma, (const T*)beta, rows, \
                  hidden, eps);                                                                                  \
    break;
  switch (nv) {
    RT_LN_CASE(1)
    RT_LN_CASE(2)
    RT_LN_CASE(3)
    RT_LN_CASE(4)
    RT_LN_CASE(6)
    RT_LN_CASE(8)
    default:
      return fail(RT_ERR_UNSUPPORTED, "layernorm: hidden=%d not supported (<=1024, 1536 or 2048)", hidden);
  }
#undef RT_LN_CASE
  count_launch();
  RT_CHECK_CUDA(cudaGetLastError());
  return RT_OK;
}

}  // namespace rt

using namespace rt;

extern "C" rt_status rt_bias_residual_layernorm(void* out, const void* x, const void* bias, const void* residual,
                                                const void* gamma, const void* beta, int rows, int hidden, float eps,
                                                int dtype, void* stream) {
  RT_REQUIRE(out && x && gamma && beta, RT_ERR_INVALID, "layernorm: null pointer");
  RT_REQUIRE(rows >= 0 && hidden > 0 && hidden % 8 == 0, RT_ERR_INVALID, "layernorm: hidden must be a multiple of 8");
  RT_REQUIRE(aligned16(out) && aligned16(x) && aligned16(gamma) && aligned16(beta) && aligned16(bias) &&
                 aligned16(residual),
             RT_ERR_INVALID, "layernorm: pointers must be 16-byte aligned");
  if (rows == 0) return RT_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == RT_F16) return layernorm_launch<__half>(out, x, bias, residual, gamma, beta, rows, hidden, eps, st);
  if (dtype == RT_BF16)
    return layernorm_launch<__nv_bfloat16>(out, x, bias, residual, gamma, beta, rows, hidden, eps, st);
  return fail(RT_ERR_INVALID, "layernorm: unknown dtype %d", dtype);
}

extern "C" rt_status rt_bias_gelu(void* x, const void* bias, int rows, int cols, int dtype, void* stream) {
  RT_REQUIRE(x && bias, RT_ERR_INVALID, "bias_gelu: null pointer");
  RT_REQUIRE(rows >= 0 && cols > 0 && cols % 8 == 0, RT_ERR_INVALID, "bias_gelu: cols must be a multiple of 8");
  RT_REQUIRE(aligned16(x) && aligned16(bias), RT_ERR_INVALID, "bias_gelu: pointers must be 16-byte aligned");
  if (rows == 0) return RT_OK;
  const size_t total = static_cast<size_t>(rows) * (cols / 8);
  const int threads = 256;
  constexpr int UNROLL = 4;
  size_t want = (total + threads * UNROLL - 1) / (threads * UNROLL);
  int blocks = static_cast<int>(std::min<size_t>(want, static_cast<size_t>(sm_count()) * 16));
  if (blocks < 1) blocks = 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == RT_F16)
    launch_kernel(bias_gelu_kernel<__half, UNROLL>, dim3(blocks), dim3(threads), 0, st, (__half*)x,
                  (const __half*)bias, total, cols / 8);
  else if (dtype == RT_BF16)
    launch_kernel(bias_gelu_kernel<__nv_bfloat16, UNROLL>, dim3(blocks), dim3(threads), 0, st, (__nv_bfloat16*)x,
                  (const __nv_bfloat16*)bias, total, cols / 8);
  else
    return fail(RT_ERR_INVALID, "bias_gelu: unknown dtype %d", dtype);
  count_launch();
  RT_CHECK_CUDA(cudaGetLastError());
  return RT_OK;
}

extern "C" rt_status rt_qkv_bias_transpose(const void* qkv, const void* bias, void* q, void* k, void* v,
                                           const int32_t* seq_block_prefix_dev, int n_seq, int total_blocks, int heads,
                                           float q_scale, int dtype, void* stream) {
  RT_REQUIRE(qkv && q && k && v && seq_block_prefix_dev, RT_ERR_INVALID, "qkv_transpose: null pointer");
  RT_REQUIRE(n_seq > 0 && total_blocks >= 0 && heads > 0, RT_ERR_INVALID, "qkv_transpose: bad sizes");
  RT_REQUIRE(aligned16(qkv) && aligned16(bias) && aligned16(q) && aligned16(k) && aligned16(v), RT_ERR_INVALID,
             "qkv_transpose: pointers must be 16-byte aligned");
  if (total_blocks == 0) return RT_OK;
  dim3 grid(total_blocks, 3);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == RT_F16)
    launch_kernel(qkv_transpose_kernel<__half>, grid, dim3(256), 0, st, (const __half*)qkv, (const __half*)bias,
                  (__half*)q, (__half*)k, (__half*)v, seq_block_prefix_dev, n_seq, heads, q_scale);
  else if (dtype == RT_BF16)
    launch_kernel(qkv_transpose_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, (const __nv_bfloat16*)qkv,
                  (const __nv_bfloat16*)bias, (__nv_bfloat16*)q, (__nv_bfloat16*)k, (__nv_bfloat16*)v,
                  seq_block_prefix_dev, n_seq, heads, q_scale);
  else
    return fail(RT_ERR_INVALID, "qkv_transpose: unknown dtype %d", dtype);
  count_launch();
  RT_CHECK_CUDA(cudaGetLastError());
  return RT_OK;
}

extern "C" rt_status rt_embeddings(void* out, const int32_t* ids, const int32_t* pos_ids, const int32_t* type_ids,
                                   const void* word, const void* pos, const void* type, const void* gamma,
                                   const void* beta, int tokens, int hidden, float eps, int dtype, void* stream) {
  RT_REQUIRE(out && ids && word && pos && type && gamma && beta, RT_ERR_INVALID, "embeddings: null pointer");
  RT_REQUIRE(hidden > 0 && hidden % 8 == 0 && hidden <= 1024, RT_ERR_UNSUPPORTED,
             "embeddings: hidden=%d not supported (multiple of 8, <= 1024)", hidden);
  RT_REQUIRE(aligned16(out) && aligned16(word) && aligned16(pos) && aligned16(type), RT_ERR_INVALID,
             "embeddings: pointers must be 16-byte aligned");
  if (tokens == 0) return RT_OK;
  const int nv = (hidden / 8 + 31) / 32;
  const int threads = 256, wpb = 8;
  const int blocks = (tokens + wpb - 1) / wpb;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define RT_EMB(T, NV)                                                                                          \
  launch_kernel(embeddings_kernel<T, NV>, dim3(blocks), dim3(threads), 0, st, (T*)out, ids, pos_ids, type_ids, \
                (const float*)word, (const float*)pos, (const float*)type, (const float*)gamma,                \
                (const float*)beta, tokens, hidden, eps)
  if (dtype == RT_F16) {
    switch (nv) { case 1: RT_EMB(__half, 1); break; case 2: RT_EMB(__half, 2); break; case 3: RT_EMB(__half, 3); break; default: RT_EMB(__half, 4); }
  } else if (dtype == RT_BF16) {
    switch (nv) { case 1: RT_EMB(__nv_bfloat16, 1); break; case 2: RT_EMB(__nv_bfloat16, 2); break; case 3: RT_EMB(__nv_bfloat16, 3); break; default: RT_EMB(__nv_bfloat16, 4); }
  } else {
    return fail(RT_ERR_INVALID, "embeddings: unknown dtype %d", dtype);
  }
#undef RT_EMB
  count_launch();
  RT_CHECK_CUDA(cudaGetLastError());
  return RT_OK;
}
