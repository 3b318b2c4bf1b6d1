// Gate-weighted un-permute and sum over the top-k picks.
//
// Replaces `y_e = expert(x_e) * w_e; out.index_add_(0, tok_e, y_e)`
// (models/decoder_moe.py:270-271): out[t] = sum_j gates[t,j] * y[route_row[t*k+j]],
// accumulated in fp32 in ascending j and rounded once.  One warp per token,
// 128-bit loads and stores; HBM-bound (k rows read + one row written per token).
#include "common.cuh"

namespace moe {
namespace {

constexpr int kWarps = 8;

template <typename T2>
__device__ __forceinline__ float2 unpack2(uint32_t u);
template <>
__device__ __forceinline__ float2 unpack2<__half2>(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat162>(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}
template <typename T2>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half2>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat162>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Vector path: d % 8 == 0 and 16-byte aligned bases.
template <typename T2, int TOPK>
__global__ void __launch_bounds__(kWarps * 32)
combine_vec_kernel(const uint4* __restrict__ y, const float* __restrict__ gates,
                   const int32_t* __restrict__ route_row, uint4* __restrict__ out, int tokens,
                   int n_vec, int top_k_rt, int total_rows) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const int top_k = TOPK > 0 ? TOPK : top_k_rt;
  const uint4* src[8];
  float g[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (j < top_k) {
      int row = route_row[(size_t)t * top_k + j];
      g[j] = gates[(size_t)t * top_k + j];
      if ((unsigned)row >= (unsigned)total_rows) { row = 0; g[j] = 0.f; }  // never read out of bounds
      src[j] = y + (size_t)row * n_vec;
    }
  }
  uint4* dst = out + (size_t)t * n_vec;
  constexpr int U = 4;
  for (int v0 = lane; v0 < n_vec; v0 += U * 32) {
    float acc[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[u][i] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < top_k) {
        uint4 r[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (v0 + u * 32 < n_vec) r[u] = __ldg(src[j] + v0 + u * 32);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (v0 + u * 32 < n_vec) {
            const uint32_t w[4] = {r[u].x, r[u].y, r[u].z, r[u].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = unpack2<T2>(w[i]);
              acc[u][2 * i] = fmaf(g[j], f.x, acc[u][2 * i]);
              acc[u][2 * i + 1] = fmaf(g[j], f.y, acc[u][2 * i + 1]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (v0 + u * 32 < n_vec) {
        uint4 o;
        o.x = pack2<T2>(acc[u][0], acc[u][1]);
        o.y = pack2<T2>(acc[u][2], acc[u][3]);
        o.z = pack2<T2>(acc[u][4], acc[u][5]);
        o.w = pack2<T2>(acc[u][6], acc[u][7]);
        dst[v0 + u * 32] = o;
      }
    }
  }
}

// Scalar path for any d / alignment.
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
combine_scalar_kernel(const T* __restrict__ y, const float* __restrict__ gates,
                      const int32_t* __restrict__ route_row, T* __restrict__ out, int tokens, int d,
                      int top_k, int total_rows) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (t >= tokens) return;
  for (int c = lane; c < d; c += 32) {
    float acc = 0.f;
    for (int j = 0; j < top_k; ++j) {
      const int row = route_row[(size_t)t * top_k + j];
      if ((unsigned)row < (unsigned)total_rows)
        acc = fmaf(gates[(size_t)t * top_k + j], to_float(y[(size_t)row * d + c]), acc);
    }
    out[(size_t)t * d + c] = from_float<T>(acc);
  }
}

template <typename T, typename T2>
int launch_combine(const void* y, const float* gates, const int32_t* route_row, int tokens, int d,
                   int top_k, void* out, cudaStream_t s) {
  const int grid = (tokens + kWarps - 1) / kWarps;
  const int total_rows = tokens * top_k;
  const uintptr_t align = reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out);
  if ((align & 15) == 0 && d % 8 == 0) {
    const uint4* yy = static_cast<const uint4*>(y);
    uint4* oo = static_cast<uint4*>(out);
    if (top_k == 2)
      combine_vec_kernel<T2, 2><<<grid, kWarps * 32, 0, s>>>(yy, gates, route_row, oo, tokens, d / 8, top_k, total_rows);
    else
      combine_vec_kernel<T2, 0><<<grid, kWarps * 32, 0, s>>>(yy, gates, route_row, oo, tokens, d / 8, top_k, total_rows);
  } else {
    combine_scalar_kernel<T><<<grid, kWarps * 32, 0, s>>>(static_cast<const T*>(y), gates, route_row,
                                                         static_cast<T*>(out), tokens, d, top_k, total_rows);
  }
  return check_launch("combine_kernel");
}

}  // namespace
}  // namespace moe

extern "C" int moe_combine(const void* y, int dtype, const float* gates, const int32_t* route_row,
                           int tokens, int d, int top_k, void* out, void* stream) {
  using namespace moe;
  if (tokens < 0 || d <= 0) return fail(MOE_ERR_ARG, "moe_combine: bad shape");
  if (top_k < 1 || top_k > 8) return fail(MOE_ERR_UNSUPPORTED, "moe_combine: top_k must be in [1,8], got %d", top_k);
  if (tokens == 0) return MOE_OK;
  if (!y || !gates || !route_row || !out) return fail(MOE_ERR_ARG, "moe_combine: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case MOE_F16: return launch_combine<__half, __half2>(y, gates, route_row, tokens, d, top_k, out, s);
    case MOE_BF16: return launch_combine<__nv_bfloat16, __nv_bfloat162>(y, gates, route_row, tokens, d, top_k, out, s);
    default: return fail(MOE_ERR_ARG, "moe_combine: dtype must be fp16 or bf16");
  }
}
