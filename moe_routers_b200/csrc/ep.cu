// Expert-parallel re-bucketing of dispatched rows.
//
// After the dispatch all-to-all a rank holds, for each source rank s in turn, that rank's rows for
// the local experts, expert-sorted inside the block of s ("source-major": [s][e][rows]).  The
// grouped GEMM wants each local expert's rows contiguous ("expert-major": [e][s][rows]).  This
// kernel moves rows between the two orders (forward before the expert FFN, backward after it, so
// that the combine all-to-all can return each source its rows in the order it sent them).
// It replaces the argsort / index_select / bincount bucketing of received rows in
// bench_2gpu_pcie.py:130-171.  Segment lengths come from the all-gathered per-rank expert counts;
// every CTA recomputes the few prefix sums it needs (world * local_experts <= 1024 values).
#include "common.cuh"

namespace moe {
namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
ep_rebucket_kernel(const char* __restrict__ src, char* __restrict__ dst, const int32_t* __restrict__ counts_all,
                   int experts, int world, int rank, int skip_src, int backward, size_t row_bytes,
                   int e_lo, int el, int32_t* __restrict__ local_offsets) {
  __shared__ int s_a, s_b, s_len;
  const int e_base = rank * (experts / world) + e_lo;  // first global expert of the range
  const int seg = blockIdx.x;  // seg = s * el + e  (e counts inside the range)
  const int s = seg / el, e = seg % el;
  if (threadIdx.x < 32) {
    // A = rows before (s, e) in source-major order, B = rows before it in expert-major order
    int a = 0, b = 0, len = 0, total = 0;
    for (int i = threadIdx.x; i < world * el; i += 32) {
      const int ss = i / el, ee = i % el;
      const int l = (ss == skip_src) ? 0 : counts_all[(size_t)ss * experts + e_base + ee];
      if (ss < s || (ss == s && ee < e)) a += l;
      if (ee < e || (ee == e && ss < s)) b += l;
      if (ss == s && ee == e) len = l;
      total += l;
    }
#pragma unroll
    for (int ofs = 16; ofs > 0; ofs >>= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, ofs);
      b += __shfl_xor_sync(0xffffffffu, b, ofs);
      len += __shfl_xor_sync(0xffffffffu, len, ofs);
      total += __shfl_xor_sync(0xffffffffu, total, ofs);
    }
    if (threadIdx.x == 0) {
      s_a = a; s_b = b; s_len = len;
      if (local_offsets != nullptr && blockIdx.y == 0) {
        if (s == 0) local_offsets[e] = b;  // first row of expert e in expert-major order
        if (seg == 0) local_offsets[el] = total;
      }
    }
  }
  __syncthreads();
  const size_t from = (size_t)(backward ? s_b : s_a) * row_bytes;
  const size_t to = (size_t)(backward ? s_a : s_b) * row_bytes;
  const size_t bytes = (size_t)s_len * row_bytes;
  // the segment is one contiguous byte range on both sides
  const size_t chunk = ((bytes / gridDim.y + 15) / 16 + 1) * 16;
  const size_t lo = (size_t)blockIdx.y * chunk;
  const size_t hi = lo + chunk < bytes ? lo + chunk : bytes;
  if (lo >= hi) return;
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | row_bytes) & 15) == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src + from + lo);
    uint4* d4 = reinterpret_cast<uint4*>(dst + to + lo);
    const size_t n = (hi - lo) / 16;
    size_t i = threadIdx.x;
    for (; i + 3 * kThreads < n; i += 4 * kThreads) {
      const uint4 r0 = __ldg(s4 + i), r1 = __ldg(s4 + i + kThreads), r2 = __ldg(s4 + i + 2 * kThreads),
                  r3 = __ldg(s4 + i + 3 * kThreads);
      d4[i] = r0; d4[i + kThreads] = r1; d4[i + 2 * kThreads] = r2; d4[i + 3 * kThreads] = r3;
    }
    for (; i < n; i += kThreads) d4[i] = __ldg(s4 + i);
  } else {
    for (size_t i = lo + threadIdx.x; i < hi; i += kThreads) dst[to + i] = src[from + i];
  }
}

}  // namespace
}  // namespace moe

extern "C" int moe_ep_rebucket(const void* src, void* dst, const int32_t* counts_all, int experts, int world,
                               int rank, int skip_src, int backward, int d, int elem_bytes, int first_local_expert,
                               int num_local_experts, int32_t* local_offsets, void* stream) {
  using namespace moe;
  if (experts <= 0 || world <= 0 || experts % world != 0)
    return fail(MOE_ERR_ARG, "experts must be divisible by world_size");
  if (rank < 0 || rank >= world) return fail(MOE_ERR_ARG, "moe_ep_rebucket: bad rank");
  if (d <= 0 || (elem_bytes != 2 && elem_bytes != 4)) return fail(MOE_ERR_ARG, "moe_ep_rebucket: bad row shape");
  if (!src || !dst || !counts_all) return fail(MOE_ERR_ARG, "moe_ep_rebucket: null pointer");
  const int el_all = experts / world;
  if (first_local_expert < 0 || num_local_experts <= 0 || first_local_expert + num_local_experts > el_all)
    return fail(MOE_ERR_ARG, "moe_ep_rebucket: bad local expert range");
  const int segs = world * num_local_experts;
  dim3 grid(segs, 16, 1);
  ep_rebucket_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const char*>(src), static_cast<char*>(dst), counts_all, experts, world, rank, skip_src,
      backward ? 1 : 0, (size_t)d * elem_bytes, first_local_expert, num_local_experts, local_offsets);
  return check_launch("ep_rebucket_kernel");
}
