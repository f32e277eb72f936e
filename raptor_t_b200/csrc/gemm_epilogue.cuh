// Shared epilogue of the tcgen05 GEMM kernels: one thread owns one accumulator row (TMEM
// lane), walks its 32-column chunks (tcgen05.ld), applies bias / GELU / the QKV scatter and
// stores 64 bytes per chunk with two 256-bit stores.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.h"
#include "sm100_ptx.cuh"

namespace rt {
namespace gemm_detail {

using namespace ptx;

__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}

// tanh-form GELU of two values with packed fp32x2 arithmetic (half the issue slots):
//   u = x * (k0 + k1 x^2),  gelu = 0.5 x + 0.5 x tanh(u)
__device__ __forceinline__ void gelu_tanh_f2(float& x0, float& x1) {
  unsigned long long x, x2, u, k0, k1, h;
  asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(x0), "f"(x1));
  asm("mov.b64 %0, {%1, %1};" : "=l"(k0) : "f"(0.7978845608028654f));
  asm("mov.b64 %0, {%1, %1};" : "=l"(k1) : "f"(0.7978845608028654f * 0.044715f));
  asm("mov.b64 %0, {%1, %1};" : "=l"(h) : "f"(0.5f));
  asm("mul.rn.f32x2 %0, %1, %1;" : "=l"(x2) : "l"(x));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(u) : "l"(x2), "l"(k1), "l"(k0));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(u) : "l"(u), "l"(x));
  float u0, u1, t0, t1;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(u0), "=f"(u1) : "l"(u));
  asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(u0));
  asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(u1));
  unsigned long long t, hx, r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(t) : "f"(t0), "f"(t1));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(hx) : "l"(x), "l"(h));
  asm("fma.rn.f32x2 %0, %1, %2, %1;" : "=l"(r) : "l"(hx), "l"(t));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(r));
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
template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (BF16) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&w));
  }
}

// Extra arguments of the QKV epilogue: the [T][3H] result is never written; each
// 64-wide head slice of a row goes, with bias added (and the query scaled), straight to
// the per-sequence head-major q / k / v buffers the attention kernel reads
// (row (seq_first_token*heads + head*seq_len + token_in_seq) of a [T*heads][64] matrix).
struct QkvEpilogue {
  const uint16_t* residual;  // RT_EPI_BIAS_RESIDUAL: [M][N], added after the bias
  uint16_t* q;
  uint16_t* k;
  uint16_t* v;
  const int2* block_seq;  // per packed 64-token block: {first token of its sequence, sequence length}
  int heads;
  float q_scale;
};
constexpr int kEpiQkv = 3;

// One 32-column chunk of one accumulator row: r[] holds the fp32 accumulators.
template <int BN, bool BF16, int EPI>
__device__ __forceinline__ void epilogue_chunk(const uint32_t* r, int c, int row, int n0, int M, int N,
                                               uint16_t* __restrict__ C, const uint16_t* __restrict__ bias,
                                               const QkvEpilogue& qkv) {
  uint32_t o[16];
  if constexpr (EPI == RT_EPI_NONE) {
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j] = pack2<BF16>(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
  } else {
    uint32_t res[16];
    if constexpr (EPI == RT_EPI_BIAS_RESIDUAL) {
      if (row < M) {
        const uint4* rp = reinterpret_cast<const uint4*>(qkv.residual + static_cast<size_t>(row) * N + n0 + c * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 t = rp[q];
          res[4 * q] = t.x;
          res[4 * q + 1] = t.y;
          res[4 * q + 2] = t.z;
          res[4 * q + 3] = t.w;
        }
      } else {
#pragma unroll
        for (int q = 0; q < 16; ++q) res[q] = 0u;
      }
    }
    const uint4* bv = reinterpret_cast<const uint4*>(bias + n0 + c * 32);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 b4 = __ldg(bv + q);
      const uint32_t bw[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 bb = unpack2<BF16>(bw[j]);
        float x0 = __uint_as_float(r[q * 8 + 2 * j]) + bb.x;
        float x1 = __uint_as_float(r[q * 8 + 2 * j + 1]) + bb.y;
        if constexpr (EPI == RT_EPI_BIAS_GELU) gelu_tanh_f2(x0, x1);
        if constexpr (EPI == RT_EPI_BIAS_RESIDUAL) {
          const float2 rr = unpack2<BF16>(res[q * 4 + j]);
          x0 += rr.x;
          x1 += rr.y;
        }
        if constexpr (EPI == kEpiQkv) {
          if (n0 + c * 32 < qkv.heads * 64) {  // query part
            x0 *= qkv.q_scale;
            x1 *= qkv.q_scale;
          }
        }
        o[q * 4 + j] = pack2<BF16>(x0, x1);
      }
    }
  }
  if (row < M) {
    uint16_t* dst;
    if constexpr (EPI == kEpiQkv) {
      const int hidden = qkv.heads * 64;
      const int n = n0 + c * 32;
      const int part = n / hidden;
      const int hcol = n - part * hidden;
      const int2 bs = __ldg(qkv.block_seq + (row >> 6));
      const size_t drow = static_cast<size_t>(bs.x) * qkv.heads + static_cast<size_t>(hcol >> 6) * bs.y + (row - bs.x);
      dst = (part == 0 ? qkv.q : part == 1 ? qkv.k : qkv.v) + drow * 64 + (hcol & 63);
    } else {
      dst = C + static_cast<size_t>(row) * N + n0 + c * 32;
    }
    st_global_v8(dst, o);
    st_global_v8(dst + 16, o + 8);
  }
}

// Drains columns [32*c] for c = chunk0, chunk0+2, ... < BN/32 of one accumulator row, two
// chunks per step so that the second TMEM load is in flight while the first chunk is processed.
//   taddr: TMEM address of column 0 of this thread's lane quarter; row: global output row.
template <int BN, bool BF16, int EPI>
__device__ __forceinline__ void epilogue_row(uint32_t taddr, int row, int n0, int chunk0, int M, int N,
                                             uint16_t* __restrict__ C, const uint16_t* __restrict__ bias,
                                             const QkvEpilogue& qkv) {
  constexpr int kChunks = BN / 32;
#pragma unroll 1
  for (int c = chunk0; c < kChunks; c += 4) {
    uint32_t r0[32], r1[32];
    const bool two = c + 2 < kChunks;
    tmem_ld32(taddr + c * 32, r0);
    if (two) tmem_ld32(taddr + (c + 2) * 32, r1);
    tc_wait_ld();
    epilogue_chunk<BN, BF16, EPI>(r0, c, row, n0, M, N, C, bias, qkv);
    if (two) epilogue_chunk<BN, BF16, EPI>(r1, c + 2, row, n0, M, N, C, bias, qkv);
  }
}

}  // namespace gemm_detail
}  // namespace rt
