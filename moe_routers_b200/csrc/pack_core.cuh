// Device pieces shared by the pack kernels and the single-launch fused route: where the rows of a
// 32-token tile go, and the bulk-copy (TMA) primitives that move them.
#pragma once

#include "sm100.cuh"

namespace moe {

constexpr int kMaxTileRoutes = kTileTokens * 8;  // top_k <= 8
constexpr int kChunkBytes = 8192;                // a row longer than this moves in chunks

// Loads below use ld.global.cg: the histograms and indices may have been written earlier in the
// same kernel by other CTAs (fused route), so they are read at L2, never from a stale L1 line.
// Where a tile's rows start: offsets[e] (exclusive scan of the expert totals) plus the number of
// routes to e in earlier tiles.  With tile_base == nullptr every CTA derives both from the tile
// histograms itself (they are L2-resident and small); otherwise pack_scan_kernel has produced
// tile_base and counts.  Then warp 0 ranks the routes of the tile with match/ballot.  On return
// s_dst[r] holds the destination row of route r of the tile (-1 = skip) and the maps are written;
// s_total[e] holds offsets[e] (first row of expert e) and, when s_exp is given, s_exp[r] the expert
// of route r.  `publish` marks the one CTA of the grid that writes counts and offsets.
__device__ __forceinline__ void tile_destinations(const int32_t* __restrict__ idx,
                                                  const int32_t* __restrict__ tile_hist,
                                                  const int32_t* __restrict__ tile_base,
                                                  int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                                                  int32_t* __restrict__ row_route,
                                                  int32_t* __restrict__ route_row, int tile, int t0,
                                                  int tile_routes, int experts, int top_k, int num_tiles,
                                                  bool publish, bool write_maps, int32_t* s_base,
                                                  int32_t* s_total, int32_t* s_dst, int32_t* status,
                                                  int32_t* s_exp = nullptr) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  // warp 0 ranks the routes later; it fetches their expert ids now so that the loads overlap the
  // histogram pass (at most 8 chunks of 32 routes per tile)
  int my_e[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int r = c * 32 + lane;
    my_e[c] = (warp == 0 && r < tile_routes) ? __ldcg(idx + (size_t)t0 * top_k + r) : -1;
  }
  if (tile_base != nullptr) {
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
      s_base[e] = tile_base[(size_t)tile * experts + e];
      s_total[e] = counts[e];
    }
  } else {
    for (int e = threadIdx.x; e < experts; e += blockDim.x) { s_base[e] = 0; s_total[e] = 0; }
    __syncthreads();
    if ((experts & 3) == 0 && experts / 4 <= (int)blockDim.x) {
      // 128-bit loads: a thread owns 4 consecutive experts and every `parts`-th tile, so that all of
      // its loads (num_tiles / parts of them) are in flight together - one L2 round trip, not four
      const int vecs = experts / 4;
      const int parts = (int)blockDim.x / vecs;
      const int v = threadIdx.x % vecs;
      const int pt = threadIdx.x / vecs;
      if (pt < parts) {
        int before[4] = {0, 0, 0, 0}, total[4] = {0, 0, 0, 0};
        const int4* th4 = reinterpret_cast<const int4*>(tile_hist);
        int t = pt;
        for (; t + 7 * parts < num_tiles; t += 8 * parts) {
          int4 h[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) h[u] = __ldcg(th4 + (size_t)(t + u * parts) * vecs + v);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const bool early = t + u * parts < tile;
            total[0] += h[u].x; total[1] += h[u].y; total[2] += h[u].z; total[3] += h[u].w;
            if (early) { before[0] += h[u].x; before[1] += h[u].y; before[2] += h[u].z; before[3] += h[u].w; }
          }
        }
        for (; t < num_tiles; t += parts) {
          const int4 h = __ldcg(th4 + (size_t)t * vecs + v);
          total[0] += h.x; total[1] += h.y; total[2] += h.z; total[3] += h.w;
          if (t < tile) { before[0] += h.x; before[1] += h.y; before[2] += h.z; before[3] += h.w; }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          atomicAdd(&s_base[4 * v + i], before[i]);
          atomicAdd(&s_total[4 * v + i], total[i]);
        }
      }
    } else {
      const int parts = max(1, (int)blockDim.x / experts);
      for (int cell = threadIdx.x; cell < experts * parts; cell += blockDim.x) {
        const int e = cell % experts;
        const int pt = cell / experts;
        int before = 0, total = 0;
        for (int t = pt; t < num_tiles; t += parts) {
          const int h = __ldcg(tile_hist + (size_t)t * experts + e);
          total += h;
          if (t < tile) before += h;
        }
        atomicAdd(&s_base[e], before);
        atomicAdd(&s_total[e], total);
      }
    }
  }
  __syncthreads();
  if (warp == 0) {
    // exclusive scan of the totals over experts; s_base becomes the first row of this tile per expert
    int carry = 0;
    for (int eb = 0; eb < experts; eb += 32) {
      const int e = eb + lane;
      const int c = (e < experts) ? s_total[e] : 0;
      int incl = c;
#pragma unroll
      for (int ofs = 1; ofs < 32; ofs <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, ofs);
        if (lane >= ofs) incl += n;
      }
      if (e < experts) {
        const int excl = carry + incl - c;
        s_base[e] += excl;
        s_total[e] = excl;
        if (publish) {
          offsets[e] = excl;
          if (tile_base == nullptr) counts[e] = c;
        }
      }
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (publish && lane == 0) offsets[experts] = carry;
    __syncwarp();

#pragma unroll
    for (int ci = 0; ci < 8; ++ci) {
      const int c = ci * 32;
      if (c >= tile_routes) break;
      const int r = c + lane;
      const bool in_tile = r < tile_routes;
      const int e = my_e[ci];
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
        if (s_exp != nullptr) s_exp[r] = e;
        if (valid && write_maps) {
          const int route = t0 * top_k + r;
          row_route[dst] = route;
          if (route_row != nullptr) route_row[route] = dst;
        }
      }
      __syncwarp();
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
               : "memory");
}

}  // namespace moe
