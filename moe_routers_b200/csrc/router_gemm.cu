// Router logit GEMM with a fused select epilogue (tcgen05 / TMEM / TMA).
//
// Replaces `logits = x @ w.t(); logits[:, :n] += bias` (bench_router.py:512-516,
// bench_2gpu_pcie.py:426-428, models/decoder_moe.py:201) followed by the
// top-k selection (kernels/fused_select.cu:47-113, models/decoder_moe.py:58-62)
// and the per-expert count (kernels/fused_select.cu:116-143).  The logits stay
// on chip: TMEM accumulators -> distributed shared memory -> registers.
//
// Work split: one cluster of SPLITK CTAs per tile of 128 tokens; CTA r of the
// cluster multiplies its slice of the K dimension (d / SPLITK) on the tensor
// core (UMMA 128 x E x 16, fp32 accumulate in TMEM).  The four 32-row blocks of
// the partial tile are then pushed to their owner CTA (row block b -> CTA
// b % SPLITK) through distributed shared memory, summed there in a fixed
// order, rounded to fp16 (the dtype the reference holds its logits in),
// biased, and scanned once per row for the top-k under the ordering "larger
// value, then lower index".  Each 32-row block also yields the per-expert
// histogram of its routes, which the pack kernels consume.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner and MMA
// issuer, warps 2..5 = epilogue (warp w reads TMEM lanes 32*(w%4)...).
#include <cstdlib>

#include "pack_core.cuh"

namespace moe {
namespace {

using namespace sm100;

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;   // 64 fp16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr int kABytes = kBlockM * kBlockK * 2;
constexpr int kMaxStages = 8;
constexpr int kSmemLimit = 227 * 1024;

struct RouterParams {
  int tokens, d, experts, top_k;
  int skew_experts;
  float skew_bias;
  int bf16;  // 0: fp16 tokens / weights / logits, 1: bf16
  int epad;  // experts rounded up to the UMMA N granule (16); padded logit columns are never selected
  int kblocks, splitk, stages, tmem_cols, num_tiles;
  int32_t* idx;
  float* gates;
  float* logits_out;
  int32_t* tile_hist;
  int32_t* status;
  // single-launch fused route only: the pack runs in the same kernel after a grid barrier
  const char* x;
  char* packed;
  size_t row_bytes;
  int chunk_bytes, nbuf;
  int32_t* counts;
  int32_t* offsets;
  int32_t* row_route;
  int32_t* route_row;
  int32_t* control;
};

constexpr int kMaxRowBufs = 48;
constexpr int kIssuers = 6;  // lane 0 of each warp drives bulk copies in the fused pack phase

// A logit that has been rounded to fp16 and its column pack into one 32-bit key whose unsigned
// order is "larger value first, then lower column": high half = the fp16 bits mapped to an
// order-preserving unsigned code (-0 folded onto +0), low half = 0xFFFF - column.
__device__ __forceinline__ uint32_t make_key(uint32_t hb, int col) {
  if (hb == 0x8000u) hb = 0u;
  const uint32_t code = (hb & 0x8000u) ? (~hb & 0xFFFFu) : (hb | 0x8000u);
  return (code << 16) | (0xFFFFu - (uint32_t)col);
}
// Rounding to the 16-bit logit type and back (fp16 or bf16: both are sign-magnitude with the exponent
// on top, so the same order-preserving code works for either).
__device__ __forceinline__ uint32_t round16(float v, bool bf16) {
  return bf16 ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v)) : (uint32_t)__half_as_ushort(__float2half_rn(v));
}
__device__ __forceinline__ float widen16(uint32_t bits, bool bf16) {
  return bf16 ? __bfloat162float(__ushort_as_bfloat16((unsigned short)bits))
              : __half2float(__ushort_as_half((unsigned short)bits));
}
__device__ __forceinline__ float key_value(uint32_t key, bool bf16) {
  const uint32_t code = key >> 16;
  const uint32_t hb = (code & 0x8000u) ? (code & 0x7FFFu) : (~code & 0xFFFFu);
  return widen16(hb, bf16);
}
__device__ __forceinline__ int key_column(uint32_t key) { return (int)(0xFFFFu - (key & 0xFFFFu)); }

// Insert into a descending list: a max/min ladder, two integer instructions per slot.
template <int KMAX>
__device__ __forceinline__ void key_insert(uint32_t (&keys)[KMAX], uint32_t c) {
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    const uint32_t m = max(keys[j], c);
    c = min(keys[j], c);
    keys[j] = m;
  }
}

// One thread = one token row: sum the S split-K partials of its quarter of the columns in a fixed
// order, round to fp16, add the skew bias (rounded again), and keep the best KMAX keys.
// `prow` points at this row in the first partial; partial `src` is src*32*EP floats further.
// The column body is branch-free (selects), padding columns get key 0 and can never be picked.
template <int KMAX, int S, bool WRITE_LOGITS>
__device__ __forceinline__ void scan_columns(const float* __restrict__ prow, int E, int n_valid, int EP, int wq,
                                             int skew_experts, float skew_bias, float* __restrict__ logits_row,
                                             bool bf16, uint32_t (&keys)[KMAX]) {
#pragma unroll
  for (int j = 0; j < KMAX; ++j) keys[j] = 0u;
  const int cols = E / 4;
  for (int c0 = wq * cols; c0 < (wq + 1) * cols; c0 += 4) {
    float4 a = *reinterpret_cast<const float4*>(prow + c0);
#pragma unroll
    for (int src = 1; src < S; ++src) {
      const float4 b = *reinterpret_cast<const float4*>(prow + (size_t)src * 32 * EP + c0);
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    const float acc[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u;
      const uint32_t h0 = round16(acc[u], bf16);
      const uint32_t h1 = round16(widen16(h0, bf16) + skew_bias, bf16);
      const uint32_t h = c < skew_experts ? h1 : h0;
      if (WRITE_LOGITS) {
        if (logits_row != nullptr && c < n_valid) logits_row[c] = widen16(h, bf16);
      }
      const uint32_t key = make_key(h, c);
      key_insert<KMAX>(keys, c < n_valid ? key : 0u);
    }
  }
}

#ifdef MOE_ROUTER_TRACE
// Probe build only: logits_out is reinterpreted as a per-CTA array of 16 clock64 stamps.
#define MOE_TRACE(slot, cond)                                                                      \
  if (cond) {                                                                                      \
    long long t_;                                                                                  \
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_)::"memory");                                   \
    reinterpret_cast<long long*>(p.logits_out)[(size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 16 + (slot)] = t_; \
  }
#define MOE_TRACE_G(slot, cond)                                                                    \
  if (cond) {                                                                                      \
    long long t_;                                                                                  \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)::"memory");                               \
    reinterpret_cast<long long*>(p.logits_out)[(size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 16 + (slot)] = t_; \
  }
#define MOE_LOGITS_OUT static_cast<float*>(nullptr)
#else
#define MOE_TRACE(slot, cond)
#define MOE_TRACE_G(slot, cond)
#define MOE_LOGITS_OUT p.logits_out
#endif

// Epilogue phase B for the four epilogue warps: reduce the split-K partials, round, bias, top-k,
// gates, histogram.  Warp wq scans a quarter of the expert columns for all 32 rows of a block
// (thread = row), keeps its local top-k as sortable 32-bit keys, and one warp merges the four
// lists of a row.  With `real` false nothing leaves the CTA's scratch.
template <int KMAX>
__device__ __forceinline__ void select_phase(const RouterParams& p, const float* s_partial, int32_t* s_hist,
                                          uint32_t* s_cand, int wq, int lane, int m_tile, int krank, bool real) {
  const int E = p.epad, EL = p.experts, EP = p.epad + 4, S = p.splitk;
  const int nslots = 4 / S;
  for (int s = 0; s < nslots; ++s) {
    const int rb = s * S + krank;
    const int row = m_tile * kBlockM + rb * 32 + lane;
    float* lo = (real && MOE_LOGITS_OUT != nullptr && row < p.tokens) ? MOE_LOGITS_OUT + (size_t)row * EL : nullptr;
    const float* prow = s_partial + (size_t)((s * S) * 32 + lane) * EP;
    uint32_t keys[KMAX];
    if (MOE_LOGITS_OUT != nullptr) {  // verification path: also writes the logits
      if (S == 4) scan_columns<KMAX, 4, true>(prow, E, EL, EP, wq, p.skew_experts, p.skew_bias, lo, p.bf16 != 0, keys);
      else if (S == 2) scan_columns<KMAX, 2, true>(prow, E, EL, EP, wq, p.skew_experts, p.skew_bias, lo, p.bf16 != 0, keys);
      else scan_columns<KMAX, 1, true>(prow, E, EL, EP, wq, p.skew_experts, p.skew_bias, lo, p.bf16 != 0, keys);
    } else {
      if (S == 4) scan_columns<KMAX, 4, false>(prow, E, EL, EP, wq, p.skew_experts, p.skew_bias, lo, p.bf16 != 0, keys);
      else if (S == 2) scan_columns<KMAX, 2, false>(prow, E, EL, EP, wq, p.skew_experts, p.skew_bias, lo, p.bf16 != 0, keys);
      else scan_columns<KMAX, 1, false>(prow, E, EL, EP, wq, p.skew_experts, p.skew_bias, lo, p.bf16 != 0, keys);
    }
#pragma unroll
    for (int j = 0; j < KMAX; ++j) s_cand[((s * 4 + wq) * KMAX + j) * 32 + lane] = keys[j];
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
  if (wq < nslots) {
    const int s = wq;
    const int rb = s * S + krank;
    const int row = m_tile * kBlockM + rb * 32 + lane;
    const bool live = real && row < p.tokens;
    uint32_t keys[KMAX];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) keys[j] = s_cand[((s * 4 + 0) * KMAX + j) * 32 + lane];
#pragma unroll
    for (int w4 = 1; w4 < 4; ++w4)
#pragma unroll
      for (int j = 0; j < KMAX; ++j) key_insert<KMAX>(keys, s_cand[((s * 4 + w4) * KMAX + j) * 32 + lane]);
    float e[KMAX];
    float sum = 0.f;
    const float v0 = key_value(keys[0], p.bf16 != 0);
#pragma unroll
    for (int j = 0; j < KMAX; ++j)
      if (j < p.top_k) { e[j] = expf(key_value(keys[j], p.bf16 != 0) - v0); sum += e[j]; }
    const float inv = 1.f / fmaxf(sum, 1e-9f);
#pragma unroll
    for (int j = 0; j < KMAX; ++j)
      if (j < p.top_k) {
        const int pick = keys[j] == 0u ? 0 : min(key_column(keys[j]), EL - 1);  // never index past the experts
        if (live) {
          p.idx[(size_t)row * p.top_k + j] = pick;
          p.gates[(size_t)row * p.top_k + j] = e[j] * inv;
          atomicAdd(&s_hist[s * E + pick], 1);
        }
      }
    __syncwarp();
    const int tile = m_tile * (kBlockM / kTileTokens) + rb;
    if (real && p.tile_hist != nullptr && tile < p.num_tiles)
      for (int e2 = lane; e2 < EL; e2 += 32) p.tile_hist[(size_t)tile * EL + e2] = s_hist[s * E + e2];
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");  // scratch is reused by the next call
}

template <int KMAX, bool FUSED>
__global__ void __launch_bounds__(kThreads, 1)
router_gemm_select_kernel(const __grid_constant__ CUtensorMap tmap_x,
                          const __grid_constant__ CUtensorMap tmap_w, const RouterParams p) {
  // 128-byte-swizzled TMA tiles need a 1024-byte aligned base; the pointers are derived from the
  // array itself so that the compiler keeps them in the shared address space.
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {  // uniform over the grid: every CTA would see the same offset
    record_error(p.status, kErrBadIndex | 0xff);
    return;
  }

  const int E = p.epad;      // accumulator / shared-memory width
  const int EL = p.experts;  // real experts
  const int b_bytes = E * kBlockK * 2;
  uint8_t* sA = smem;
  uint8_t* sB = sA + (size_t)p.stages * kABytes;
  const int EP = E + 4;  // padded row of a partial tile: conflict-free 128-bit accesses, thread = row
  float* s_partial = reinterpret_cast<float*>(sB + (size_t)p.stages * b_bytes);  // [4][32][EP]
  int32_t* s_hist = reinterpret_cast<int32_t*>(s_partial + 4 * 32 * EP);        // [4][E]
  uint32_t* s_cand = reinterpret_cast<uint32_t*>(s_hist + 4 * E);               // [4][4][KMAX][32]
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_cand + 16 * KMAX * 32);       // full[], empty[], tmem_full
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_bar + 2 * kMaxStages + 1);
  uint64_t* s_rowbar = reinterpret_cast<uint64_t*>(s_tmem + 2);  // [kMaxRowBufs], fused route only

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tile = blockIdx.x;
  const int krank = (int)cluster_ctarank();
  const int S = p.splitk;
  const int kb0 = (int)(((long long)p.kblocks * krank) / S);
  const int kb1 = (int)(((long long)p.kblocks * (krank + 1)) / S);
  const int nkb = kb1 - kb0;

  MOE_TRACE(0, threadIdx.x == 0);
  MOE_TRACE_G(15, threadIdx.x == 0);
  const uint32_t full0 = smem_u32(s_bar);
  const uint32_t empty0 = smem_u32(s_bar + kMaxStages);
  const uint32_t tmem_full = smem_u32(s_bar + 2 * kMaxStages);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(tmem_full, 1);
    if (FUSED)
      for (int b = 0; b < p.nbuf; ++b) mbar_init(smem_u32(s_rowbar + b), 1);
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&tmap_x);
    prefetch_tensormap(&tmap_w);
  }
  for (int i = threadIdx.x; i < 4 * E; i += kThreads) s_hist[i] = 0;
  if (warp == 1) {
    tmem_alloc(smem_u32(s_tmem), (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  // Let a dependent kernel (launched with programmatic stream serialisation) start its own
  // input prefetch now; it still waits for this grid to finish before reading what we write.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  MOE_TRACE(1, threadIdx.x == 0);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, 1)) break;
        mbar_expect_tx(full0 + 8 * s, (uint32_t)(kABytes + b_bytes));
        tma_load_2d(smem_u32(sA + (size_t)s * kABytes), &tmap_x, full0 + 8 * s, (kb0 + i) * kBlockK,
                    m_tile * kBlockM);
        tma_load_2d(smem_u32(sB + (size_t)s * b_bytes), &tmap_w, full0 + 8 * s, (kb0 + i) * kBlockK, 0);
        MOE_TRACE(2, i == 0);
      }
      if (FUSED) {
        // The token rows this CTA will scatter do not depend on the routing.  Once the last MMA has
        // read the pipeline stages, the stage area becomes the row ring: fetch the first rows now, so
        // that they arrive while the select epilogue and the grid barrier run.
        if (mbar_wait(tmem_full, 0, p.status, 5)) {
          const int t0 = (m_tile * 4 + krank) * kTileTokens;
          const int tile_tokens = max(0, min(kTileTokens, p.tokens - t0));
          const int chunks = (int)((p.row_bytes + p.chunk_bytes - 1) / p.chunk_bytes);
          const int items = tile_tokens * chunks;
          for (int it = 0; it < p.nbuf && it < items; ++it) {
            const int row = it / chunks, ch = it % chunks;
            const size_t ofs = (size_t)ch * p.chunk_bytes;
            const uint32_t bytes = (uint32_t)min((size_t)p.chunk_bytes, p.row_bytes - ofs);
            bulk_load(smem_u32(smem) + (uint32_t)it * (uint32_t)p.chunk_bytes,
                      p.x + (size_t)(t0 + row) * p.row_bytes + ofs, bytes, smem_u32(s_rowbar + it));
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(kBlockM, E, p.bf16, 0, 0);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
        if (!mbar_wait(full0 + 8 * s, ph, p.status, 2)) break;
        MOE_TRACE(3, i == 0);
        tc_fence_after();
        const uint64_t adesc = make_desc_kmajor_sw128(smem_u32(sA + (size_t)s * kABytes));
        const uint64_t bdesc = make_desc_kmajor_sw128(smem_u32(sB + (size_t)s * b_bytes));
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
          // +32 bytes per K step inside the 128-byte swizzle row (address field is in 16-byte units)
          umma_f16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (uint32_t)((i | k) != 0));
        }
        umma_commit(empty0 + 8 * s);  // stage may be refilled once these MMAs have read it
      }
      umma_commit(tmem_full);  // accumulator complete
      MOE_TRACE(4, true);
    }
    __syncwarp();
  } else {
    // -------------- epilogue phase A: TMEM -> owner CTA's shared memory --------------
    const int q = warp & 3;  // TMEM lane quadrant == 32-row block of the tile
    const bool ok = mbar_wait(tmem_full, 0, p.status, 3);
    MOE_TRACE(5, threadIdx.x == 64);
    tc_fence_after();
    const int dest = q % S;
    const int slot = q / S;
    const uint32_t remote = map_to_cta(smem_u32(s_partial), (uint32_t)dest);
    const uint32_t base = remote + (uint32_t)(((slot * S + krank) * 32 + lane) * EP) * 4u;
#pragma unroll 1
    for (int c0 = 0; c0 < E; c0 += 16) {
      float v[16];
      if (ok) {
        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 16; i += 4)
        st_cluster_v4(base + (uint32_t)(c0 + i) * 4u, v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
    MOE_TRACE(6, threadIdx.x == 64);
  }

  tc_fence_before();
  __syncwarp();
  cluster_sync_all();  // partial tiles of all K slices are now in their owner's shared memory
  MOE_TRACE(7, threadIdx.x == 64);

  if (warp >= 2) {
    select_phase<KMAX>(p, s_partial, s_hist, s_cand, warp - 2, lane, m_tile, krank, true);
    MOE_TRACE(8, threadIdx.x == 64);
  }

  MOE_TRACE(9, threadIdx.x == 64);
  MOE_TRACE_G(14, threadIdx.x == 64);

  if constexpr (FUSED) {
    // ------------------------------ pack phase (fused route) ------------------------------
    // Every CTA has published the histogram of its 32-token tile; after the grid barrier each CTA
    // derives the offsets and the first row of its tile per expert from all histograms, ranks its
    // routes and stores its (already prefetched) token rows to their top_k destinations.
    __shared__ int s_ok;
    const bool ok = grid_barrier(p.control, (int)(gridDim.x * gridDim.y), p.status, &s_ok);
    const int tile = m_tile * 4 + krank;
    const int t0 = tile * kTileTokens;
    const int tile_tokens = max(0, min(kTileTokens, p.tokens - t0));
    int32_t* s_base = reinterpret_cast<int32_t*>(s_partial);  // the partial tiles are no longer needed
    int32_t* s_total = s_base + EL;
    int32_t* s_dst = s_total + EL;
    if (ok) {
      tile_destinations(p.idx, p.tile_hist, nullptr, p.counts, p.offsets, p.row_route, p.route_row, tile, t0,
                        tile_tokens * p.top_k, EL, p.top_k, p.num_tiles, blockIdx.x == 0 && blockIdx.y == 0, true,
                        s_base, s_total, s_dst, p.status);
      if (lane == 0 && warp < kIssuers) {
        const int chunks = (int)((p.row_bytes + p.chunk_bytes - 1) / p.chunk_bytes);
        const int items = tile_tokens * chunks;
        const int depth = p.nbuf / kIssuers;
        const uint32_t buf0 = smem_u32(smem);
        for (int m = 0;; ++m) {
          const int it = warp + m * kIssuers;
          if (it >= items) break;
          const int b = warp + (m % depth) * kIssuers;
          if (!mbar_wait(smem_u32(s_rowbar + b), (uint32_t)(m / depth) & 1u, p.status, 6)) break;
          const int row = it / chunks, ch = it % chunks;
          const size_t ofs = (size_t)ch * p.chunk_bytes;
          const uint32_t bytes = (uint32_t)min((size_t)p.chunk_bytes, p.row_bytes - ofs);
          for (int j = 0; j < p.top_k; ++j) {
            const int dr = s_dst[row * p.top_k + j];
            if (dr >= 0) bulk_store(p.packed + (size_t)dr * p.row_bytes + ofs, buf0 + (uint32_t)b * (uint32_t)p.chunk_bytes, bytes);
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          const int nxt = it + depth * kIssuers;
          if (nxt < items) {
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            const int nrow = nxt / chunks, nch = nxt % chunks;
            const size_t nofs = (size_t)nch * p.chunk_bytes;
            const uint32_t nbytes = (uint32_t)min((size_t)p.chunk_bytes, p.row_bytes - nofs);
            bulk_load(buf0 + (uint32_t)b * (uint32_t)p.chunk_bytes, p.x + (size_t)(t0 + nrow) * p.row_bytes + nofs,
                      nbytes, smem_u32(s_rowbar + b));
          }
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      }
      __syncwarp();
    }
  }

  tc_fence_before();
  __syncthreads();
  MOE_TRACE(10, threadIdx.x == 0);
  MOE_TRACE_G(13, threadIdx.x == 0);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// Outputs of the pack when the whole route runs as one launch.
struct FusedPack {
  void* packed;
  int32_t* counts;
  int32_t* offsets;
  int32_t* row_route;
  int32_t* route_row;
};

// MOE_B200_FUSED=1 in the environment runs the route as ONE launch (pack phase behind a grid
// barrier inside the router kernel).  Off by default: with the launches captured in a CUDA graph
// the two-launch route measured faster on B200 (31.3 vs 34.7 us at T=4096, d=4096, E=64); the
// single launch is for callers that pay full launch latency per kernel.
bool fused_enabled() {
  static const bool on = [] {
    const char* v = getenv("MOE_B200_FUSED");
    return v && v[0] == '1';
  }();
  return on;
}

// Launches the router GEMM + select kernel.  With `fp` non-null it tries the single-launch fused
// route (pack phase behind a grid barrier in the same kernel) and sets *did_fuse; that needs the
// 4-way K split and every cluster of the grid resident at once, otherwise the plain kernel runs
// and the caller launches the scatter.
int launch_router(const void* x, const void* w, int tokens, int d, int experts, int top_k, int skew_experts,
                  float skew_bias, int dtype, int32_t* idx, float* gates, float* logits_out, const Workspace& ws,
                  cudaStream_t stream, const FusedPack* fp = nullptr, bool* did_fuse = nullptr) {
  if (did_fuse) *did_fuse = false;
  CUtensorMap tmap_x, tmap_w;
  int rc = encode_tmap_2d(&tmap_x, x, (uint64_t)tokens, (uint64_t)d, (uint64_t)d * 2, kBlockK, kBlockM);
  if (rc != MOE_OK) return rc;
  const int epad = (experts + 15) / 16 * 16;  // W rows past `experts` are zero-filled by the TMA unit
  rc = encode_tmap_2d(&tmap_w, w, (uint64_t)experts, (uint64_t)d, (uint64_t)d * 2, kBlockK, (uint32_t)epad);
  if (rc != MOE_OK) return rc;

  RouterParams p;
  p.tokens = tokens; p.d = d; p.experts = experts; p.top_k = top_k; p.epad = epad;
  p.bf16 = dtype == MOE_BF16;
  p.skew_experts = skew_experts < 0 ? 0 : (skew_experts > experts ? experts : skew_experts);
  p.skew_bias = skew_bias;
  if (skew_bias == 0.0f) p.skew_experts = 0;
  p.kblocks = (d + kBlockK - 1) / kBlockK;
  p.splitk = p.kblocks >= 16 ? 4 : (p.kblocks >= 4 ? 2 : 1);
  int cols = 32;
  while (cols < epad) cols *= 2;
  p.tmem_cols = cols;
  p.num_tiles = ws.num_tiles;
  const int stage_bytes = kABytes + epad * kBlockK * 2;
  const int kmax = top_k <= 1 ? 1 : (top_k <= 2 ? 2 : (top_k <= 4 ? 4 : 8));
  const int fixed = 4 * 32 * (epad + 4) * 4 + 4 * epad * 4 + 16 * kmax * 32 * 4 + (2 * kMaxStages + 1) * 8 + 16 +
                    kMaxRowBufs * 8;
  int stages = (kSmemLimit - 1024 - fixed) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  const int max_nkb = (p.kblocks + p.splitk - 1) / p.splitk;
  if (stages > max_nkb) stages = max_nkb;
  if (stages < 1) return fail(MOE_ERR_UNSUPPORTED, "router GEMM: shared memory budget exceeded for experts=%d", experts);
  p.stages = stages;
  p.idx = idx; p.gates = gates; p.logits_out = logits_out;
  p.tile_hist = ws.tile_hist; p.status = ws.status;
  const size_t smem = 1024 + (size_t)stages * stage_bytes + fixed;

  p.x = static_cast<const char*>(x);
  p.packed = nullptr; p.row_bytes = (size_t)d * 2; p.chunk_bytes = 0; p.nbuf = 0;
  p.counts = nullptr; p.offsets = nullptr; p.row_route = nullptr; p.route_row = nullptr;
  p.control = ws.control;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((tokens + kBlockM - 1) / kBlockM, p.splitk, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = p.splitk;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeCooperative;
  attr[1].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;

  if (fp != nullptr && fp->packed != nullptr && p.splitk == 4 && fused_enabled() && ws.num_tiles <= 256) {
    auto fkernel = kmax == 1 ? router_gemm_select_kernel<1, true>
                   : kmax == 2 ? router_gemm_select_kernel<2, true>
                   : kmax == 4 ? router_gemm_select_kernel<4, true>
                               : router_gemm_select_kernel<8, true>;
    const int chunk = (int)(p.row_bytes < (size_t)kChunkBytes ? p.row_bytes : (size_t)kChunkBytes);
    int nbuf = (int)(((size_t)stages * stage_bytes) / chunk);
    if (nbuf > kMaxRowBufs) nbuf = kMaxRowBufs;
    nbuf = (nbuf / kIssuers) * kIssuers;
    e = cudaFuncSetAttribute(fkernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    int max_clusters = 0;
    if (e == cudaSuccess && nbuf >= kIssuers) {
      cfg.numAttrs = 1;  // occupancy is asked for the cluster shape
      e = cudaOccupancyMaxActiveClusters(&max_clusters, fkernel, &cfg);
    }
    if (e == cudaSuccess && nbuf >= kIssuers && max_clusters >= (int)cfg.gridDim.x) {
      p.packed = static_cast<char*>(fp->packed);
      p.chunk_bytes = chunk; p.nbuf = nbuf;
      p.counts = fp->counts; p.offsets = fp->offsets; p.row_route = fp->row_route; p.route_row = fp->route_row;
      cfg.numAttrs = 2;  // cluster + cooperative: all CTAs resident, the grid barrier cannot starve
      e = cudaLaunchKernelEx(&cfg, fkernel, tmap_x, tmap_w, p);
      if (e == cudaSuccess) {
        if (did_fuse) *did_fuse = true;
        return MOE_OK;
      }
      (void)cudaGetLastError();  // this launch shape is not available: fall through to two launches
      p.packed = nullptr; p.chunk_bytes = 0; p.nbuf = 0;
    } else {
      (void)cudaGetLastError();
    }
    cfg.numAttrs = 1;
  }

  auto kernel = kmax == 1 ? router_gemm_select_kernel<1, false>
                : kmax == 2 ? router_gemm_select_kernel<2, false>
                : kmax == 4 ? router_gemm_select_kernel<4, false>
                            : router_gemm_select_kernel<8, false>;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "router GEMM: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  e = cudaLaunchKernelEx(&cfg, kernel, tmap_x, tmap_w, p);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "router_gemm_select_kernel: %s", cudaGetErrorString(e));
  return MOE_OK;
}

int check_router_args(const char* who, const void* x, const void* w, int tokens, int d, int experts, int top_k,
                      int dtype, const void* idx, const void* gates, const void* workspace,
                      size_t workspace_bytes) {
  if (tokens < 0 || d <= 0 || experts <= 0) return fail(MOE_ERR_ARG, "%s: bad shape", who);
  if (dtype != MOE_F16 && dtype != MOE_BF16) return fail(MOE_ERR_ARG, "%s: x must be fp16 or bf16", who);
  if (top_k < 1 || top_k > 8) return fail(MOE_ERR_UNSUPPORTED, "%s: top_k must be in [1,8], got %d", who, top_k);
  if (top_k > experts) return fail(MOE_ERR_ARG, "%s: top_k must be <= n_experts", who);
  if (experts > 256) return fail(MOE_ERR_UNSUPPORTED, "%s: experts must be <= 256, got %d", who, experts);
  if (d % 8 != 0) return fail(MOE_ERR_UNSUPPORTED, "%s: d_model must be a multiple of 8, got %d", who, d);
  if (tokens > 0 && (!x || !w || !idx || !gates)) return fail(MOE_ERR_ARG, "%s: null pointer", who);
  if (!workspace || workspace_bytes < workspace_bytes_for(tokens, experts, top_k))
    return fail(MOE_ERR_WORKSPACE, "%s: workspace too small (need %zu bytes)", who,
                workspace_bytes_for(tokens, experts, top_k));
  return MOE_OK;
}

}  // namespace

int launch_scan_scatter(const void* x, int elem_bytes, const int32_t* idx, int tokens, int d, int experts,
                        int top_k, int32_t* counts, int32_t* offsets, void* packed, int32_t* row_route,
                        int32_t* route_row, const Workspace& ws, cudaStream_t s, void* const* seg_base = nullptr);

}  // namespace moe

extern "C" int moe_router_gemm_select(const void* x, const void* w_router, int dtype, int tokens, int d, int experts,
                                      int top_k, int skew_experts, float skew_bias, int32_t* idx, float* gates,
                                      float* logits_out, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace moe;
  int rc = check_router_args("moe_router_gemm_select", x, w_router, tokens, d, experts, top_k, dtype, idx, gates,
                             workspace, workspace_bytes);
  if (rc != MOE_OK || tokens == 0) return rc;
  Workspace ws = carve(workspace, tokens, experts);
  return launch_router(x, w_router, tokens, d, experts, top_k, skew_experts, skew_bias, dtype, idx, gates, logits_out,
                       ws, static_cast<cudaStream_t>(stream));
}

extern "C" int moe_route_fused(const void* x, const void* w_router, int dtype, int tokens, int d, int experts, int top_k,
                               int skew_experts, float skew_bias, int32_t* idx, float* gates, int32_t* counts,
                               int32_t* offsets, void* packed, int32_t* row_route, int32_t* route_row,
                               float* logits_out, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace moe;
  int rc = check_router_args("moe_route_fused", x, w_router, tokens, d, experts, top_k, dtype, idx, gates, workspace,
                             workspace_bytes);
  if (rc != MOE_OK) return rc;
  if (!counts || !offsets || (tokens > 0 && !row_route)) return fail(MOE_ERR_ARG, "moe_route_fused: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Workspace ws = carve(workspace, tokens, experts);
  if (tokens > 0) {
    FusedPack fp{packed, counts, offsets, row_route, route_row};
    bool fused = false;
    rc = launch_router(x, w_router, tokens, d, experts, top_k, skew_experts, skew_bias, dtype, idx, gates, logits_out,
                       ws, s, &fp, &fused);
    if (rc != MOE_OK || fused) return rc;
  }
  return launch_scan_scatter(x, 2, idx, tokens, d, experts, top_k, counts, offsets, packed, row_route, route_row,
                             ws, s);
}
