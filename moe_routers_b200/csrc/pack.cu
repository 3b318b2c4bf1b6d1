// Count, scan and pack: expert-contiguous copy of raw token rows.
//
// Replaces count_expert_kernel, the CUB scan + host read-back and
// pack_copy_kernel (kernels/fused_select.cu:116-198, :256-308) and the torch
// pack bench_router.py:57-78.
//
// Data flow (tile = 32 consecutive tokens = 32*k routes):
//   pack_hist_kernel     idx -> tile_hist[tile][expert]           (skipped when the router GEMM
//                                                                  epilogue already produced it)
//   pack_scan_kernel     tile_hist -> tile_base (exclusive prefix down the tiles, per expert),
//                        counts, offsets
//   pack_scatter_kernel  per tile: ranks inside the tile by warp match/ballot, destination row =
//                        offsets[e] + tile_base[tile][e] + rank, then 128-bit row copies
// A destination row is a pure function of (idx, route id): the order inside an
// expert segment is ascending route id, run to run.  There is no host
// synchronisation: total rows = tokens * top_k is known in advance.
#include "common.cuh"

namespace moe {
namespace {

constexpr int kScatterThreads = 256;
constexpr int kMaxTileRoutes = kTileTokens * 8;  // top_k <= 8

// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
pack_hist_kernel(const int32_t* __restrict__ idx, int32_t* __restrict__ tile_hist, int tokens,
                 int experts, int top_k, int32_t* status) {
  extern __shared__ int32_t s_hist[];
  const int tile = blockIdx.x;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) s_hist[e] = 0;
  __syncthreads();
  const int r0 = tile * kTileTokens * top_k;
  const int r1 = min(tokens, (tile + 1) * kTileTokens) * top_k;
  for (int r = r0 + threadIdx.x; r < r1; r += blockDim.x) {
    const int e = idx[r];
    if ((unsigned)e < (unsigned)experts) atomicAdd(&s_hist[e], 1);
    else record_error(status, kErrBadIndex);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    tile_hist[(size_t)tile * experts + e] = s_hist[e];
}

// ---------------------------------------------------------------------------
// One CTA.  Warp per expert column: exclusive prefix down the tiles; then an
// exclusive scan over the expert totals gives offsets.
__global__ void __launch_bounds__(1024)
pack_scan_kernel(const int32_t* __restrict__ tile_hist, int32_t* __restrict__ tile_base,
                 int32_t* __restrict__ counts, int32_t* __restrict__ offsets, int num_tiles,
                 int experts) {
  extern __shared__ int32_t s_tot[];  // [experts] totals, then scanned in place
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  for (int e = warp; e < experts; e += nwarps) {
    int running = 0;
    for (int base = 0; base < num_tiles; base += 32) {
      const int tile = base + lane;
      const int h = (tile < num_tiles) ? tile_hist[(size_t)tile * experts + e] : 0;
      int incl = h;
#pragma unroll
      for (int ofs = 1; ofs < 32; ofs <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, ofs);
        if (lane >= ofs) incl += n;
      }
      if (tile < num_tiles) tile_base[(size_t)tile * experts + e] = running + incl - h;
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) { s_tot[e] = running; counts[e] = running; }
  }
  __syncthreads();
  // exclusive scan over experts (experts <= 1024): serial per 32-chunk carry, warp 0
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < experts; base += 32) {
      const int e = base + lane;
      const int c = (e < experts) ? s_tot[e] : 0;
      int incl = c;
#pragma unroll
      for (int ofs = 1; ofs < 32; ofs <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, ofs);
        if (lane >= ofs) incl += n;
      }
      if (e < experts) offsets[e] = carry + incl - c;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) offsets[experts] = carry;
  }
}

// ---------------------------------------------------------------------------
template <typename V>
__device__ __forceinline__ void copy_row(const char* __restrict__ src, char* const* dst, int n_dst,
                                         int n_vec, int lane) {
  const V* s = reinterpret_cast<const V*>(src);
  constexpr int U = 8;
  int v = lane;
  for (; v + (U - 1) * 32 < n_vec; v += U * 32) {
    V r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) r[u] = __ldg(s + v + u * 32);
    for (int j = 0; j < n_dst; ++j) {
      V* d = reinterpret_cast<V*>(dst[j]);
#pragma unroll
      for (int u = 0; u < U; ++u) d[v + u * 32] = r[u];
    }
  }
  for (; v < n_vec; v += 32) {
    const V r = __ldg(s + v);
    for (int j = 0; j < n_dst; ++j) reinterpret_cast<V*>(dst[j])[v] = r;
  }
}

// grid = num_tiles * split; CTA (tile, part) ranks the whole tile (cheap) and
// copies tokens [part*tokens_per_cta, ...) of it.
template <typename V>
__global__ void __launch_bounds__(kScatterThreads)
pack_scatter_kernel(const char* __restrict__ x, const int32_t* __restrict__ idx,
                    const int32_t* __restrict__ tile_base, const int32_t* __restrict__ offsets,
                    char* __restrict__ packed, int32_t* __restrict__ row_route,
                    int32_t* __restrict__ route_row, int tokens, size_t row_bytes, int experts,
                    int top_k, int split, int32_t* status) {
  extern __shared__ int32_t s_mem[];
  int32_t* s_base = s_mem;           // [experts]   next free row per expert inside this tile
  int32_t* s_dst = s_mem + experts;  // [kMaxTileRoutes] destination row of each route (-1 = skip)

  const int tile = blockIdx.x / split;
  const int part = blockIdx.x % split;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int t0 = tile * kTileTokens;
  const int tile_tokens = min(kTileTokens, tokens - t0);
  const int tile_routes = tile_tokens * top_k;

  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    s_base[e] = offsets[e] + tile_base[(size_t)tile * experts + e];
  __syncthreads();

  if (warp == 0) {
    for (int c = 0; c < tile_routes; c += 32) {
      const int r = c + lane;
      const bool in_tile = r < tile_routes;
      const int e = in_tile ? idx[(size_t)t0 * top_k + r] : -1;
      const bool valid = in_tile && (unsigned)e < (unsigned)experts;
      if (in_tile && !valid) record_error(status, kErrBadIndex);
      const unsigned key = valid ? (unsigned)e : (0x40000000u + lane);
      const unsigned peers = __match_any_sync(0xffffffffu, key);
      const int rank = __popc(peers & lanemask_lt());
      const int leader = __ffs(peers) - 1;
      int base = 0;
      if (valid && lane == leader) {
        base = s_base[e];
        s_base[e] = base + __popc(peers);
      }
      base = __shfl_sync(0xffffffffu, base, leader);
      if (in_tile) {
        const int dst = valid ? base + rank : -1;
        s_dst[r] = dst;
        if (valid && part == 0) {
          const int route = t0 * top_k + r;
          row_route[dst] = route;
          if (route_row != nullptr) route_row[route] = dst;
        }
      }
      __syncwarp();
    }
  }
  __syncthreads();
  if (packed == nullptr) return;

  const int per_cta = kTileTokens / split;
  const int lt0 = part * per_cta;
  const int lt1 = min(tile_tokens, lt0 + per_cta);
  const int n_vec = (int)(row_bytes / sizeof(V));
  for (int lt = lt0 + warp; lt < lt1; lt += kScatterThreads / 32) {
    char* dst[8];
    int n_dst = 0;
    for (int j = 0; j < top_k; ++j) {
      const int d = s_dst[lt * top_k + j];
      if (d >= 0) dst[n_dst++] = packed + (size_t)d * row_bytes;
    }
    copy_row<V>(x + (size_t)(t0 + lt) * row_bytes, dst, n_dst, n_vec, lane);
  }
}

int pick_split(int num_tiles) {
  // aim for a few CTAs per SM (148 SMs) without dropping below one token per warp
  int split = 1;
  while (split < 4 && num_tiles * split < 148 * 3) split *= 2;
  return split;
}

}  // namespace

// Shared by moe_pack and moe_route_fused: scan + scatter from ready tile histograms.
int launch_scan_scatter(const void* x, int elem_bytes, const int32_t* idx, int tokens, int d,
                        int experts, int top_k, int32_t* counts, int32_t* offsets, void* packed,
                        int32_t* row_route, int32_t* route_row, const Workspace& ws,
                        cudaStream_t s) {
  pack_scan_kernel<<<1, 1024, experts * sizeof(int32_t), s>>>(ws.tile_hist, ws.tile_base, counts,
                                                             offsets, tokens > 0 ? ws.num_tiles : 0,
                                                             experts);
  int rc = check_launch("pack_scan_kernel");
  if (rc != MOE_OK || tokens == 0) return rc;

  const size_t row_bytes = (size_t)d * elem_bytes;
  const int split = pick_split(ws.num_tiles);
  const int grid = ws.num_tiles * split;
  const size_t smem = (size_t)(experts + kMaxTileRoutes) * sizeof(int32_t);
  const uintptr_t align = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed) | row_bytes;
  const char* xs = static_cast<const char*>(x);
  char* ps = static_cast<char*>(packed);
#define MOE_SCATTER(V)                                                                          \
  pack_scatter_kernel<V><<<grid, kScatterThreads, smem, s>>>(xs, idx, ws.tile_base, offsets, ps, \
                                                             row_route, route_row, tokens,      \
                                                             row_bytes, experts, top_k, split,  \
                                                             ws.status)
  if ((align & 15) == 0) MOE_SCATTER(uint4);
  else if ((align & 3) == 0) MOE_SCATTER(uint32_t);
  else MOE_SCATTER(uint16_t);
#undef MOE_SCATTER
  return check_launch("pack_scatter_kernel");
}

}  // namespace moe

extern "C" int moe_pack(const void* x, int elem_bytes, const int32_t* idx, int tokens, int d,
                        int experts, int top_k, int32_t* counts, int32_t* offsets, void* packed,
                        int32_t* row_route, int32_t* route_row, void* workspace,
                        size_t workspace_bytes, void* stream) {
  using namespace moe;
  if (tokens < 0 || d <= 0 || experts <= 0) return fail(MOE_ERR_ARG, "moe_pack: bad shape");
  if (top_k < 1 || top_k > 8) return fail(MOE_ERR_UNSUPPORTED, "moe_pack: top_k must be in [1,8], got %d", top_k);
  if (experts > 1024) return fail(MOE_ERR_UNSUPPORTED, "moe_pack: experts must be <= 1024");
  if (elem_bytes != 2 && elem_bytes != 4) return fail(MOE_ERR_ARG, "moe_pack: elem_bytes must be 2 or 4");
  if ((long long)tokens * top_k > 0x7fffffffLL) return fail(MOE_ERR_UNSUPPORTED, "moe_pack: too many routes");
  if (!counts || !offsets) return fail(MOE_ERR_ARG, "moe_pack: null counts/offsets");
  if (tokens > 0 && (!idx || !row_route || (packed && !x)))
    return fail(MOE_ERR_ARG, "moe_pack: null pointer");
  if (!workspace || workspace_bytes < workspace_bytes_for(tokens, experts, top_k))
    return fail(MOE_ERR_WORKSPACE, "moe_pack: workspace too small (need %zu bytes)",
                workspace_bytes_for(tokens, experts, top_k));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Workspace ws = carve(workspace, tokens, experts);
  if (tokens > 0) {
    pack_hist_kernel<<<ws.num_tiles, 256, experts * sizeof(int32_t), s>>>(idx, ws.tile_hist, tokens,
                                                                         experts, top_k, ws.status);
    int rc = check_launch("pack_hist_kernel");
    if (rc != MOE_OK) return rc;
  }
  return launch_scan_scatter(x, elem_bytes, idx, tokens, d, experts, top_k, counts, offsets, packed,
                             row_route, route_row, ws, s);
}
