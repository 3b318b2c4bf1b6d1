// Top-k selection over router logits, one warp per token row.
//
// Replaces fused_select_cuda.forward(logits, k) (called at
// models/decoder_moe.py:150), torch.topk + softmax (models/decoder_moe.py:58-62)
// and top2_select_64_kernel (kernels/fused_select.cu:47-113).
//
// Each lane owns NPL consecutive columns (column = lane*NPL + i).  A pick is a
// warp-wide arg-max under the ordering "larger value, then lower index"; the
// winner is retired through a per-lane bit mask (not by overwriting the value,
// so rows that contain -inf still select in index order).  Gates are the
// softmax over the picked values, in fp32.
#include "common.cuh"

namespace moe {
namespace {

constexpr int kWarpsPerCta = 8;

// WARPS rows per CTA.  With HIST the CTA covers exactly one 32-token tile (WARPS == kTileTokens) and
// also writes that tile's per-expert histogram, which the pack consumes: select + count in one launch.
template <typename T, int NPL, int WARPS, bool HIST>
__global__ void __launch_bounds__(WARPS * 32)
topk_select_kernel(const T* __restrict__ logits, int32_t* __restrict__ out_idx,
                   float* __restrict__ out_w, int tokens, int experts, int top_k,
                   int32_t* __restrict__ tile_hist) {
  extern __shared__ int32_t s_hist[];  // [experts], HIST only
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (HIST) {
    for (int e = threadIdx.x; e < experts; e += WARPS * 32) s_hist[e] = 0;
    __syncthreads();
  }
  if (row < tokens) {
  const T* src = logits + (size_t)row * experts;

  float v[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int col = lane * NPL + i;
    v[i] = (col < experts) ? to_float(src[col]) : -INFINITY;
  }
  uint32_t taken = 0;
#pragma unroll
  for (int i = 0; i < NPL; ++i)
    if (lane * NPL + i >= experts) taken |= 1u << i;  // padding columns are never picked

  float pick_v[8];
  int pick_i[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (j < top_k) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const int col = lane * NPL + i;
        if (!((taken >> i) & 1u) && better(v[i], col, bv, bi)) { bv = v[i]; bi = col; }
      }
#pragma unroll
      for (int ofs = 16; ofs > 0; ofs >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, ofs);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, ofs);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
      }
      // every lane now holds the same winner
      if (bi != 0x7fffffff && bi / NPL == lane) taken |= 1u << (bi % NPL);
      pick_v[j] = bv;
      pick_i[j] = (bi == 0x7fffffff) ? 0 : bi;
    }
  }

  if (lane == 0) {
    const float m = pick_v[0];
    float e[8];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < top_k) { e[j] = expf(pick_v[j] - m); sum += e[j]; }
    const float inv = 1.f / fmaxf(sum, 1e-9f);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < top_k) {
        out_idx[(size_t)row * top_k + j] = pick_i[j];
        out_w[(size_t)row * top_k + j] = e[j] * inv;
        if (HIST) atomicAdd(&s_hist[pick_i[j]], 1);
      }
  }
  }  // row < tokens
  if (HIST) {
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += WARPS * 32) tile_hist[(size_t)blockIdx.x * experts + e] = s_hist[e];
  }
}


// ---------------------------------------------------------------------------
// Fast path for 16-bit logits (fp16 / bf16) whose rows are a multiple of 16 bytes: 32 rows per CTA
// (one histogram tile), four threads per row.  A thread loads its 8-column pieces with 128-bit loads
// and keeps its best KMAX candidates as 32-bit keys whose unsigned order is "larger value, then
// lower column" (the 16 value bits mapped to an order-preserving code, -0 folded onto +0, above
// 0xFFFF - column); the four lists of a row are merged with two shuffle steps.  Same selection and
// gates as the warp-per-row kernel below, at a third of its time (one memory round trip, no
// per-pick warp reductions).
__device__ __forceinline__ uint32_t key16(uint32_t hb, int col) {
  if (hb == 0x8000u) hb = 0u;
  const uint32_t code = (hb & 0x8000u) ? (~hb & 0xFFFFu) : (hb | 0x8000u);
  return (code << 16) | (0xFFFFu - (uint32_t)col);
}
template <bool BF16>
__device__ __forceinline__ float key16_value(uint32_t key) {
  const uint32_t code = key >> 16;
  const uint32_t hb = (code & 0x8000u) ? (code & 0x7FFFu) : (~code & 0xFFFFu);
  return BF16 ? __bfloat162float(__ushort_as_bfloat16((unsigned short)hb))
              : __half2float(__ushort_as_half((unsigned short)hb));
}
template <int KMAX>
__device__ __forceinline__ void key16_insert(uint32_t (&keys)[KMAX], uint32_t c) {
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    const uint32_t m = max(keys[j], c);
    c = min(keys[j], c);
    keys[j] = m;
  }
}

constexpr int kFastRows = kTileTokens;  // rows per CTA
constexpr int kFastTpr = 4;             // threads per row

template <int KMAX, bool BF16>
__global__ void __launch_bounds__(kFastRows * kFastTpr)
topk_select16_kernel(const uint16_t* __restrict__ logits, int32_t* __restrict__ out_idx, float* __restrict__ out_w,
                     int tokens, int experts, int top_k, int32_t* __restrict__ tile_hist) {
  extern __shared__ int32_t s_hist[];  // [experts], only with tile_hist
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a scatter behind us may prefetch its rows
  if (tile_hist != nullptr) {
    for (int e = threadIdx.x; e < experts; e += kFastRows * kFastTpr) s_hist[e] = 0;
    __syncthreads();
  }
  const int row = blockIdx.x * kFastRows + (int)threadIdx.x / kFastTpr;
  const int cg = (int)threadIdx.x % kFastTpr;
  uint32_t keys[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j) keys[j] = 0u;
  if (row < tokens) {
    const uint4* src = reinterpret_cast<const uint4*>(logits + (size_t)row * experts);
    for (int ch = cg; ch < experts / 8; ch += kFastTpr) {
      const uint4 v = __ldg(src + ch);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        key16_insert<KMAX>(keys, key16(w[u] & 0xFFFFu, ch * 8 + 2 * u));
        key16_insert<KMAX>(keys, key16(w[u] >> 16, ch * 8 + 2 * u + 1));
      }
    }
  }
#pragma unroll
  for (int ofs = 1; ofs < kFastTpr; ofs <<= 1) {
    uint32_t other[KMAX];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) other[j] = __shfl_xor_sync(0xffffffffu, keys[j], ofs);
#pragma unroll
    for (int j = 0; j < KMAX; ++j) key16_insert<KMAX>(keys, other[j]);
  }
  if (cg == 0 && row < tokens) {
    const float m = key16_value<BF16>(keys[0]);
    float e[KMAX];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < KMAX; ++j)
      if (j < top_k) { e[j] = expf(key16_value<BF16>(keys[j]) - m); sum += e[j]; }
    const float inv = 1.f / fmaxf(sum, 1e-9f);
#pragma unroll
    for (int j = 0; j < KMAX; ++j)
      if (j < top_k) {
        const int pick = (int)(0xFFFFu - (keys[j] & 0xFFFFu));
        out_idx[(size_t)row * top_k + j] = pick;
        out_w[(size_t)row * top_k + j] = e[j] * inv;
        if (tile_hist != nullptr) atomicAdd(&s_hist[pick], 1);
      }
  }
  if (tile_hist != nullptr) {
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += kFastRows * kFastTpr) tile_hist[(size_t)blockIdx.x * experts + e] = s_hist[e];
  }
}

template <bool BF16>
int launch_select16(const void* logits, int tokens, int experts, int top_k, int32_t* idx, float* w, int32_t* tile_hist,
                    cudaStream_t s) {
  const uint16_t* p = static_cast<const uint16_t*>(logits);
  const int grid = (tokens + kFastRows - 1) / kFastRows;
  const size_t smem = tile_hist != nullptr ? experts * sizeof(int32_t) : 0;
  const int kmax = top_k <= 1 ? 1 : (top_k <= 2 ? 2 : (top_k <= 4 ? 4 : 8));
#define MOE_SEL16(K) topk_select16_kernel<K, BF16><<<grid, kFastRows * kFastTpr, smem, s>>>(p, idx, w, tokens, experts, top_k, tile_hist)
  if (kmax == 1) MOE_SEL16(1);
  else if (kmax == 2) MOE_SEL16(2);
  else if (kmax == 4) MOE_SEL16(4);
  else MOE_SEL16(8);
#undef MOE_SEL16
  return check_launch("topk_select16_kernel");
}

template <typename T>
int launch_select(const void* logits, int tokens, int experts, int top_k, int32_t* idx, float* w,
                  int32_t* tile_hist, cudaStream_t s) {
  const T* p = static_cast<const T*>(logits);
  const int npl = (experts + 31) / 32;
  const bool hist = tile_hist != nullptr;
  const int grid = hist ? (tokens + kTileTokens - 1) / kTileTokens : (tokens + kWarpsPerCta - 1) / kWarpsPerCta;
#define MOE_SEL(N)                                                                                     \
  if (hist)                                                                                            \
    topk_select_kernel<T, N, kTileTokens, true><<<grid, kTileTokens * 32, experts * sizeof(int32_t), s>>>( \
        p, idx, w, tokens, experts, top_k, tile_hist);                                                 \
  else                                                                                                 \
    topk_select_kernel<T, N, kWarpsPerCta, false><<<grid, kWarpsPerCta * 32, 0, s>>>(p, idx, w, tokens, experts, \
                                                                                    top_k, nullptr)
  if (npl <= 1) { MOE_SEL(1); }
  else if (npl <= 2) { MOE_SEL(2); }
  else if (npl <= 4) { MOE_SEL(4); }
  else if (npl <= 8) { MOE_SEL(8); }
  else if (npl <= 16) { MOE_SEL(16); }
  else { MOE_SEL(32); }
#undef MOE_SEL
  return check_launch("topk_select_kernel");
}

}  // namespace

// select (+ per-tile histogram when tile_hist is given) for any logits dtype
int launch_select_any(const void* logits, int logits_dtype, int tokens, int experts, int top_k, int32_t* idx,
                      float* gates, int32_t* tile_hist, cudaStream_t s) {
  // 16-bit logits with 16-byte rows: the key-based kernel (every pick of a row must exist: top_k <= experts)
  if ((logits_dtype == MOE_F16 || logits_dtype == MOE_BF16) && experts % 8 == 0 && experts <= 1024 &&
      (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
    return logits_dtype == MOE_F16 ? launch_select16<false>(logits, tokens, experts, top_k, idx, gates, tile_hist, s)
                                   : launch_select16<true>(logits, tokens, experts, top_k, idx, gates, tile_hist, s);
  }
  switch (logits_dtype) {
    case MOE_F16: return launch_select<__half>(logits, tokens, experts, top_k, idx, gates, tile_hist, s);
    case MOE_BF16: return launch_select<__nv_bfloat16>(logits, tokens, experts, top_k, idx, gates, tile_hist, s);
    case MOE_F32: return launch_select<float>(logits, tokens, experts, top_k, idx, gates, tile_hist, s);
    default: return fail(MOE_ERR_ARG, "logits must be fp16/bf16/fp32");
  }
}

}  // namespace moe

extern "C" int moe_topk_select(const void* logits, int logits_dtype, int tokens, int experts,
                               int top_k, int32_t* idx, float* gates, void* stream) {
  using namespace moe;
  if (tokens < 0 || experts <= 0) return fail(MOE_ERR_ARG, "moe_topk_select: bad shape [%d,%d]", tokens, experts);
  if (top_k < 1 || top_k > 8) return fail(MOE_ERR_UNSUPPORTED, "moe_topk_select: top_k must be in [1,8], got %d", top_k);
  if (top_k > experts) return fail(MOE_ERR_ARG, "moe_topk_select: top_k must be <= n_experts");
  if (experts > 1024) return fail(MOE_ERR_UNSUPPORTED, "moe_topk_select: experts must be <= 1024, got %d", experts);
  if (tokens == 0) return MOE_OK;
  if (!logits || !idx || !gates) return fail(MOE_ERR_ARG, "moe_topk_select: null pointer");
  return launch_select_any(logits, logits_dtype, tokens, experts, top_k, idx, gates, nullptr,
                           static_cast<cudaStream_t>(stream));
}
