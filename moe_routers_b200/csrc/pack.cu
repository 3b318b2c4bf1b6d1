// Count, scan and pack: expert-contiguous copy of raw token rows.
//
// Replaces count_expert_kernel, the CUB scan + host read-back and
// pack_copy_kernel (kernels/fused_select.cu:116-198, :256-308) and the torch
// pack bench_router.py:57-78.
//
// Data flow (tile = 32 consecutive tokens = 32*k routes):
//   pack_hist_kernel     idx -> tile_hist[tile][expert]           (skipped when the router GEMM
//                                                                  epilogue already produced it)
//   pack_scan_kernel     (only above 256 tiles) tile_hist -> tile_base: exclusive prefix down the
//                        tiles per expert, and counts
//   pack_scatter_kernel  per tile: offsets (scan of the expert totals) and the tile's base per
//                        expert, ranks inside the tile by warp match/ballot, destination row =
//                        offsets[e] + routes to e in earlier tiles + rank, then 128-bit row copies
// A destination row is a pure function of (idx, route id): the order inside an
// expert segment is ascending route id, run to run.  There is no host
// synchronisation: total rows = tokens * top_k is known in advance.
#include <cstdlib>
#include <mutex>

#include "pack_core.cuh"

namespace moe {
namespace {

constexpr int kScatterThreads = 256;
constexpr int kFusedPrefixTiles = 256;           // up to this many tiles each scatter CTA sums the histograms itself

// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
pack_hist_kernel(const int32_t* __restrict__ idx, int32_t* __restrict__ tile_hist, int tokens,
                 int experts, int top_k, int32_t* status) {
  extern __shared__ int32_t s_hist[];
  const int tile = blockIdx.x;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the scatter may prefetch its rows
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
// Large inputs only (more than kFusedPrefixTiles tiles): one CTA per expert column computes the
// exclusive prefix of that expert's tile counts down the tiles, and the expert's total.
__global__ void __launch_bounds__(256)
pack_scan_kernel(const int32_t* __restrict__ tile_hist, int32_t* __restrict__ tile_base,
                 int32_t* __restrict__ counts, int num_tiles, int experts) {
  __shared__ int32_t s_warp[8];
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  int running = 0;
  for (int base = 0; base < num_tiles; base += 256) {
    const int tile = base + threadIdx.x;
    const int h = (tile < num_tiles) ? tile_hist[(size_t)tile * experts + e] : 0;
    int incl = h;
#pragma unroll
    for (int ofs = 1; ofs < 32; ofs <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, ofs);
      if (lane >= ofs) incl += n;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    int warp_ofs = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int v = s_warp[w];
      if (w < warp) warp_ofs += v;
      total += v;
    }
    if (tile < num_tiles) tile_base[(size_t)tile * experts + e] = running + warp_ofs + incl - h;
    running += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = running;
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

// ---------------------------------------------------------------------------
// Load/store scatter for rows that are not 16-byte friendly.  grid = num_tiles * split; CTA
// (tile, part) ranks the whole tile (cheap) and copies tokens [part*tokens_per_cta, ...) of it.
template <typename V>
__global__ void __launch_bounds__(kScatterThreads)
pack_scatter_kernel(const char* __restrict__ x, const int32_t* __restrict__ idx,
                    const int32_t* __restrict__ tile_hist, const int32_t* __restrict__ tile_base,
                    int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                    char* __restrict__ packed, int32_t* __restrict__ row_route,
                    int32_t* __restrict__ route_row, int tokens, size_t row_bytes, int experts,
                    int top_k, int split, int num_tiles, int32_t* status) {
  extern __shared__ int32_t s_mem[];
  int32_t* s_base = s_mem;               // [experts]
  int32_t* s_total = s_mem + experts;    // [experts]
  int32_t* s_dst = s_mem + 2 * experts;  // [kMaxTileRoutes]

  const int tile = blockIdx.x / split;
  const int part = blockIdx.x % split;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int t0 = tile * kTileTokens;
  const int tile_tokens = min(kTileTokens, tokens - t0);

  // a kernel launched behind this one with programmatic stream serialisation (the next route's
  // router GEMM) may set itself up as soon as every CTA of this grid is running
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  tile_destinations(idx, tile_hist, tile_base, counts, offsets, row_route, route_row, tile, t0,
                    tile_tokens * top_k, experts, top_k, num_tiles, blockIdx.x == 0, part == 0, s_base,
                    s_total, s_dst, status);
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

// ---------------------------------------------------------------------------
// Bulk-copy scatter (rows a multiple of 16 bytes, 16-byte aligned bases): one CTA per tile of 32
// tokens.  Token rows are staged through a ring of shared-memory buffers by the TMA engine:
//   global --cp.async.bulk--> shared (mbarrier complete_tx) --cp.async.bulk--> top_k global rows.
// A row longer than kChunkBytes is moved in chunks.  Lane 0 of each of the 8 warps drives every
// 8th item (item = row chunk); buffer (item % NBUF) with NBUF a multiple of 8, so a buffer is only
// ever reused by the thread that filled it, after that thread's stores have finished reading it.
// The first loads are issued before the destinations are known: they do not depend on the routing.
constexpr int kBulkIssuers = kScatterThreads / 32;

__global__ void __launch_bounds__(kScatterThreads, 1)
pack_scatter_bulk_kernel(const char* __restrict__ x, const int32_t* __restrict__ idx,
                         const int32_t* __restrict__ tile_hist, const int32_t* __restrict__ tile_base,
                         int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                         char* __restrict__ packed, int32_t* __restrict__ row_route,
                         int32_t* __restrict__ route_row, int tokens, size_t row_bytes, int experts,
                         int top_k, int num_tiles, int nbuf, int chunk_bytes, int32_t* status,
                         char* const* __restrict__ seg_base) {
  extern __shared__ __align__(128) uint8_t s_raw[];
  uint8_t* s_buf = s_raw;                                                        // [nbuf][chunk_bytes]
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_buf + (size_t)nbuf * chunk_bytes);  // [nbuf]
  int32_t* s_base = reinterpret_cast<int32_t*>(s_bar + nbuf);                    // [experts]
  int32_t* s_total = s_base + experts;                                           // [experts]
  int32_t* s_dst = s_total + experts;                                            // [kMaxTileRoutes]
  int32_t* s_exp = s_dst + kMaxTileRoutes;                                       // [kMaxTileRoutes], seg_base only

  const int tile = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int t0 = tile * kTileTokens;
  const int tile_tokens = min(kTileTokens, tokens - t0);
  const int chunks = (int)((row_bytes + chunk_bytes - 1) / chunk_bytes);
  const int items = (packed != nullptr || seg_base != nullptr) ? tile_tokens * chunks : 0;
  const int depth = nbuf / kBulkIssuers;  // buffers owned by each issuing thread

  // a kernel launched behind this one with programmatic stream serialisation (the next route's
  // router GEMM) may set itself up as soon as every CTA of this grid is running
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int b = 0; b < nbuf; ++b)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(s_bar + b)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const uint32_t buf0 = (uint32_t)__cvta_generic_to_shared(s_buf);
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(s_bar);
  // item m of this thread is tile item (warp + m*8); it lives in buffer (warp + (m % depth)*8)
  // (rows of at most one chunk, the usual case, need no division)
  auto item_src = [&](int it, uint32_t& bytes) -> const char* {
    const int row = chunks == 1 ? it : it / chunks, ch = chunks == 1 ? 0 : it % chunks;
    const size_t ofs = (size_t)ch * chunk_bytes;
    bytes = (uint32_t)min((size_t)chunk_bytes, row_bytes - ofs);
    return x + (size_t)(t0 + row) * row_bytes + ofs;
  };
  if (lane == 0) {
    for (int m = 0; m < depth; ++m) {
      const int it = warp + m * kBulkIssuers;
      if (it >= items) break;
      uint32_t bytes;
      const char* src = item_src(it, bytes);
      const int b = warp + m * kBulkIssuers;
      bulk_load(buf0 + (uint32_t)b * chunk_bytes, src, bytes, bar0 + 8u * b);
    }
  }
  __syncwarp();

  asm volatile("griddepcontrol.wait;" ::: "memory");
  tile_destinations(idx, tile_hist, tile_base, counts, offsets, row_route, route_row, tile, t0,
                    tile_tokens * top_k, experts, top_k, num_tiles, blockIdx.x == 0, true, s_base, s_total,
                    s_dst, status, seg_base != nullptr ? s_exp : nullptr);

  if (lane == 0) {
    bool ok = true;
    int slot = 0;        // m % depth and the parity of m / depth, advanced without divisions
    uint32_t par = 0;
    for (int m = 0; ok; ++m) {
      const int it = warp + m * kBulkIssuers;
      if (it >= items) break;
      const int b = warp + slot * kBulkIssuers;
      ok = sm100::mbar_wait(bar0 + 8u * b, par, status, 8);
      if (!ok) break;
      if (++slot == depth) { slot = 0; par ^= 1u; }
      const int row = chunks == 1 ? it : it / chunks, ch = chunks == 1 ? 0 : it % chunks;
      uint32_t bytes;
      (void)item_src(it, bytes);
      for (int j = 0; j < top_k; ++j) {
        const int d = s_dst[row * top_k + j];
        if (d < 0) continue;
        char* dst_row;
        if (seg_base == nullptr) {
          dst_row = packed + (size_t)d * row_bytes;
        } else {
          // rows of expert e form one segment that starts at seg_base[e] (possibly in a peer's memory)
          const int e = s_exp[row * top_k + j];
          dst_row = seg_base[e] + (size_t)(d - s_total[e]) * row_bytes;
        }
        bulk_store(dst_row + (size_t)ch * chunk_bytes, buf0 + (uint32_t)b * chunk_bytes, bytes);
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      const int nxt = it + depth * kBulkIssuers;
      if (nxt < items) {
        // the buffer is refilled once the stores just issued have finished reading it
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        uint32_t nbytes;
        const char* src = item_src(nxt, nbytes);
        bulk_load(buf0 + (uint32_t)b * chunk_bytes, src, nbytes, bar0 + 8u * b);
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all stores complete before the CTA retires
  }
  __syncwarp();
}

__global__ void pack_zero_kernel(int32_t* counts, int32_t* offsets, int experts) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e < experts) counts[e] = 0;
  if (e <= experts) offsets[e] = 0;
}

int pick_split(int num_tiles) {
  // aim for a few CTAs per SM (148 SMs) without dropping below one token per warp
  int split = 1;
  while (split < 4 && num_tiles * split < 148 * 3) split *= 2;
  return split;
}

}  // namespace

// Shared by moe_pack and moe_route_fused: offsets + scatter from ready tile histograms.
int launch_scan_scatter(const void* x, int elem_bytes, const int32_t* idx, int tokens, int d,
                        int experts, int top_k, int32_t* counts, int32_t* offsets, void* packed,
                        int32_t* row_route, int32_t* route_row, const Workspace& ws,
                        cudaStream_t s, void* const* seg_base = nullptr) {
  if (tokens == 0) {
    pack_zero_kernel<<<(experts + 256) / 256, 256, 0, s>>>(counts, offsets, experts);
    return check_launch("pack_zero_kernel");
  }
  const int32_t* tile_base = nullptr;
  if (ws.num_tiles > kFusedPrefixTiles) {
    pack_scan_kernel<<<experts, 256, 0, s>>>(ws.tile_hist, ws.tile_base, counts, ws.num_tiles, experts);
    const int rc = check_launch("pack_scan_kernel");
    if (rc != MOE_OK) return rc;
    tile_base = ws.tile_base;
  }
  const size_t row_bytes = (size_t)d * elem_bytes;
  const uintptr_t align = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed) | row_bytes;
  const char* xs = static_cast<const char*>(x);
  char* ps = static_cast<char*>(packed);
  const int32_t* th = ws.tile_hist;
  int32_t* st = ws.status;
  const int nt = ws.num_tiles;

  // Programmatic dependent launch: the scatter may become resident while the producer of the tile
  // histograms (router GEMM or histogram kernel) is still running; it prefetches token rows and
  // then blocks in griddepcontrol.wait until that kernel has completed.
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kScatterThreads, 1, 1);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (tile_base == nullptr && pdl_enabled()) ? 1 : 0;
  cudaError_t err;

  char* const* sb = reinterpret_cast<char* const*>(seg_base);
  if ((align & 15) == 0 && (packed != nullptr || sb != nullptr)) {
    const int chunk = (int)(row_bytes < (size_t)kChunkBytes ? row_bytes : (size_t)kChunkBytes);
    const int chunks = (int)((row_bytes + chunk - 1) / chunk);
    const size_t fixed = (size_t)(2 * experts + 2 * kMaxTileRoutes) * sizeof(int32_t) + 64 * sizeof(uint64_t) + 128;
    int nbuf = (int)((227 * 1024 - fixed) / chunk);
    const int want = ((kTileTokens * chunks + kBulkIssuers - 1) / kBulkIssuers) * kBulkIssuers;
    if (nbuf > want) nbuf = want;
    if (nbuf > 64) nbuf = 64;
    nbuf = (nbuf / kBulkIssuers) * kBulkIssuers;
    if (nbuf >= kBulkIssuers) {
      const size_t smem = (size_t)nbuf * chunk + (size_t)nbuf * sizeof(uint64_t) +
                         (size_t)(2 * experts + 2 * kMaxTileRoutes) * sizeof(int32_t);
      err = cudaFuncSetAttribute(pack_scatter_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return fail(MOE_ERR_LAUNCH, "pack_scatter_bulk_kernel: %s", cudaGetErrorString(err));
      cfg.gridDim = dim3(nt, 1, 1);
      cfg.dynamicSmemBytes = smem;
      err = cudaLaunchKernelEx(&cfg, pack_scatter_bulk_kernel, xs, idx, th, tile_base, counts, offsets, ps,
                               row_route, route_row, tokens, row_bytes, experts, top_k, nt, nbuf, chunk, st, sb);
      if (err != cudaSuccess) return fail(MOE_ERR_LAUNCH, "pack_scatter_bulk_kernel: %s", cudaGetErrorString(err));
      note_launch();
      return MOE_OK;
    }
  }
  if (sb != nullptr)
    return fail(MOE_ERR_UNSUPPORTED, "moe_pack_scatter_to: rows must be a multiple of 16 bytes, 16-byte aligned, "
                                     "and fit the staging ring");

  const int split = pick_split(nt);
  cfg.gridDim = dim3(nt * split, 1, 1);
  cfg.dynamicSmemBytes = (size_t)(2 * experts + kMaxTileRoutes) * sizeof(int32_t);
#define MOE_SCATTER(V)                                                                            \
  err = cudaLaunchKernelEx(&cfg, pack_scatter_kernel<V>, xs, idx, th, tile_base, counts, offsets, ps, \
                           row_route, route_row, tokens, row_bytes, experts, top_k, split, nt, st)
  if ((align & 15) == 0) MOE_SCATTER(uint4);
  else if ((align & 3) == 0) MOE_SCATTER(uint32_t);
  else MOE_SCATTER(uint16_t);
#undef MOE_SCATTER
  if (err != cudaSuccess) return fail(MOE_ERR_LAUNCH, "pack_scatter_kernel: %s", cudaGetErrorString(err));
  note_launch();
  return MOE_OK;
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

// ---------------------------------------------------------------------------
// Allocation-free variant of moe_pack.
//
// Some callers cannot hand the library a workspace because they cannot allocate device memory at
// the point of the call: code running under a memory plan fixed in advance (an inference engine
// that has already carved up its arena), a plugin whose host forbids cudaMalloc inside its
// execute hook, or a latency-critical loop where an allocator call may synchronise the device.
// For them the tile histograms live in a fixed array that is part of the loaded library image.
namespace moe {
namespace {

constexpr int kStaticMaxTokens = 8192;   // 256 tiles of 32 tokens
constexpr int kStaticMaxExperts = 256;
constexpr size_t kStaticScratchBytes =
    (size_t)(kStaticMaxTokens / kTileTokens) * kStaticMaxExperts * sizeof(int32_t);  // 262,144 bytes

// Held by every GPU that loads the library, until the process exits.
static __device__ __align__(256) unsigned char g_pack_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
void* g_static_ptr[kMaxDevices] = {};

// The array's name is only a host-side handle; kernels need its device address, which is looked up
// once per device (with that device current) and cached.
int static_scratch_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "moe_pack_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(MOE_ERR_UNSUPPORTED, "moe_pack_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_pack_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(MOE_ERR_LAUNCH, "moe_pack_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return MOE_OK;
}

}  // namespace
}  // namespace moe

extern "C" int moe_pack_static(const void* x, int elem_bytes, const int32_t* idx, int tokens, int d, int experts,
                               int top_k, int32_t* counts, int32_t* offsets, void* packed, int32_t* row_route,
                               int32_t* route_row, int32_t* device_status, void* stream) {
  using namespace moe;
  if (tokens < 0 || d <= 0 || experts <= 0) return fail(MOE_ERR_ARG, "moe_pack_static: bad shape");
  if (top_k < 1 || top_k > 8) return fail(MOE_ERR_UNSUPPORTED, "moe_pack_static: top_k must be in [1,8], got %d", top_k);
  if (tokens > kStaticMaxTokens || experts > kStaticMaxExperts)
    return fail(MOE_ERR_UNSUPPORTED,
                "moe_pack_static: at most %d tokens and %d experts fit the built-in scratch (got %d, %d); "
                "use moe_pack with a caller-owned workspace", kStaticMaxTokens, kStaticMaxExperts, tokens, experts);
  if (elem_bytes != 2 && elem_bytes != 4) return fail(MOE_ERR_ARG, "moe_pack_static: elem_bytes must be 2 or 4");
  if (!counts || !offsets) return fail(MOE_ERR_ARG, "moe_pack_static: null counts/offsets");
  if (tokens > 0 && (!idx || !row_route || (packed && !x))) return fail(MOE_ERR_ARG, "moe_pack_static: null pointer");
  void* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc != MOE_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Workspace ws;
  ws.status = device_status;  // may be null: errors are then not recorded
  ws.control = nullptr;
  ws.tile_hist = static_cast<int32_t*>(scratch);
  ws.tile_base = nullptr;     // never used: at most 256 tiles, every scatter CTA sums the histograms
  ws.fscratch = nullptr;
  ws.num_tiles = num_tiles_for(tokens > 0 ? tokens : 1);
  if (tokens > 0) {
    // every histogram word that is read below is written here first: nothing in the array has to
    // start at zero, whatever the previous call left behind
    pack_hist_kernel<<<ws.num_tiles, 256, experts * sizeof(int32_t), s>>>(idx, ws.tile_hist, tokens, experts, top_k,
                                                                         ws.status);
    rc = check_launch("pack_hist_kernel");
    if (rc != MOE_OK) return rc;
  }
  return launch_scan_scatter(x, elem_bytes, idx, tokens, d, experts, top_k, counts, offsets, packed, row_route,
                             route_row, ws, s);
}

namespace moe {
int launch_select_any(const void* logits, int logits_dtype, int tokens, int experts, int top_k, int32_t* idx,
                      float* gates, int32_t* tile_hist, cudaStream_t s);
}

// The reference's whole operator in two launches: select (+ tile histograms), then scatter.
extern "C" int moe_fused_select(const void* logits, int logits_dtype, const void* x, int elem_bytes, int tokens,
                                int d, int experts, int top_k, int32_t* idx, float* gates, int32_t* counts,
                                int32_t* offsets, void* packed, int32_t* row_route, int32_t* route_row,
                                void* workspace, size_t workspace_bytes, void* stream) {
  using namespace moe;
  if (tokens < 0 || d <= 0 || experts <= 0) return fail(MOE_ERR_ARG, "moe_fused_select: bad shape");
  if (top_k < 1 || top_k > 8) return fail(MOE_ERR_UNSUPPORTED, "moe_fused_select: top_k must be in [1,8], got %d", top_k);
  if (top_k > experts) return fail(MOE_ERR_ARG, "moe_fused_select: top_k must be <= n_experts");
  if (experts > 1024) return fail(MOE_ERR_UNSUPPORTED, "moe_fused_select: experts must be <= 1024");
  if (elem_bytes != 2 && elem_bytes != 4) return fail(MOE_ERR_ARG, "moe_fused_select: elem_bytes must be 2 or 4");
  if (!counts || !offsets) return fail(MOE_ERR_ARG, "moe_fused_select: null counts/offsets");
  if (tokens > 0 && (!logits || !idx || !gates || !row_route || (packed && !x)))
    return fail(MOE_ERR_ARG, "moe_fused_select: null pointer");
  if (!workspace || workspace_bytes < workspace_bytes_for(tokens, experts, top_k))
    return fail(MOE_ERR_WORKSPACE, "moe_fused_select: workspace too small (need %zu bytes)",
                workspace_bytes_for(tokens, experts, top_k));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Workspace ws = carve(workspace, tokens, experts);
  if (tokens > 0) {
    const int rc = launch_select_any(logits, logits_dtype, tokens, experts, top_k, idx, gates, ws.tile_hist, s);
    if (rc != MOE_OK) return rc;
  }
  return launch_scan_scatter(x, elem_bytes, idx, tokens, d, experts, top_k, counts, offsets, packed, row_route,
                             route_row, ws, s);
}

// The scatter half on its own: offsets + ranks + row copies from tile histograms that a preceding
// call (moe_router_gemm_select, moe_route_fused or moe_fused_select with the same workspace, token
// count and expert count) left in the workspace.
extern "C" int moe_pack_scatter(const void* x, int elem_bytes, const int32_t* idx, int tokens, int d, int experts,
                                int top_k, int32_t* counts, int32_t* offsets, void* packed, int32_t* row_route,
                                int32_t* route_row, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace moe;
  if (tokens < 0 || d <= 0 || experts <= 0) return fail(MOE_ERR_ARG, "moe_pack_scatter: bad shape");
  if (top_k < 1 || top_k > 8) return fail(MOE_ERR_UNSUPPORTED, "moe_pack_scatter: top_k must be in [1,8], got %d", top_k);
  if (experts > 1024) return fail(MOE_ERR_UNSUPPORTED, "moe_pack_scatter: experts must be <= 1024");
  if (elem_bytes != 2 && elem_bytes != 4) return fail(MOE_ERR_ARG, "moe_pack_scatter: elem_bytes must be 2 or 4");
  if (!counts || !offsets) return fail(MOE_ERR_ARG, "moe_pack_scatter: null counts/offsets");
  if (tokens > 0 && (!idx || !row_route || (packed && !x))) return fail(MOE_ERR_ARG, "moe_pack_scatter: null pointer");
  if (!workspace || workspace_bytes < workspace_bytes_for(tokens, experts, top_k))
    return fail(MOE_ERR_WORKSPACE, "moe_pack_scatter: workspace too small (need %zu bytes)",
                workspace_bytes_for(tokens, experts, top_k));
  Workspace ws = carve(workspace, tokens, experts);
  return launch_scan_scatter(x, elem_bytes, idx, tokens, d, experts, top_k, counts, offsets, packed, row_route,
                             route_row, ws, static_cast<cudaStream_t>(stream), nullptr);
}

// The scatter with one destination segment per expert: the rows routed to expert e are stored, in
// canonical order, from seg_base[e] on (device array of `experts` 16-byte aligned addresses), instead
// of at packed[offsets[e]].  The expert-parallel layer points every segment into the inbox of the rank
// that owns the expert (a peer mapping, bulk stores over NVLink): dispatch without a local packed copy.
extern "C" int moe_pack_scatter_to(const void* x, int elem_bytes, const int32_t* idx, int tokens, int d, int experts,
                                   int top_k, int32_t* counts, int32_t* offsets, void* const* seg_base,
                                   int32_t* row_route, int32_t* route_row, void* workspace, size_t workspace_bytes,
                                   void* stream) {
  using namespace moe;
  if (tokens < 0 || d <= 0 || experts <= 0) return fail(MOE_ERR_ARG, "moe_pack_scatter_to: bad shape");
  if (top_k < 1 || top_k > 8) return fail(MOE_ERR_UNSUPPORTED, "moe_pack_scatter_to: top_k must be in [1,8], got %d", top_k);
  if (experts > 1024) return fail(MOE_ERR_UNSUPPORTED, "moe_pack_scatter_to: experts must be <= 1024");
  if (elem_bytes != 2 && elem_bytes != 4) return fail(MOE_ERR_ARG, "moe_pack_scatter_to: elem_bytes must be 2 or 4");
  if (!counts || !offsets || !seg_base) return fail(MOE_ERR_ARG, "moe_pack_scatter_to: null counts/offsets/seg_base");
  if (tokens > 0 && (!idx || !row_route || !x)) return fail(MOE_ERR_ARG, "moe_pack_scatter_to: null pointer");
  if (!workspace || workspace_bytes < workspace_bytes_for(tokens, experts, top_k))
    return fail(MOE_ERR_WORKSPACE, "moe_pack_scatter_to: workspace too small (need %zu bytes)",
                workspace_bytes_for(tokens, experts, top_k));
  Workspace ws = carve(workspace, tokens, experts);
  return launch_scan_scatter(x, elem_bytes, idx, tokens, d, experts, top_k, counts, offsets, nullptr, row_route,
                             route_row, ws, static_cast<cudaStream_t>(stream), seg_base);
}
