// Grouped expert GEMM over expert-contiguous rows (tcgen05 / TMEM / TMA).
//
// Replaces grouped_ffn_forward (kernels/grouped_ffn.cu:53-136, a CUTLASS mma.sync grouped GEMM fed
// by host-built pointer arrays) and the per-expert Python loops around cuBLAS
// (bench_2gpu_pcie.py:123-171, models/decoder_moe.py:256-273, fused_select.py:74-93).
//
//   for every expert e:  C[off[e]:off[e+1], :] = act( A[off[e]:off[e+1], :] @ W[e] ) (* row_scale)
//
// A persistent grid (one CTA per SM) walks the tile list (expert, n-tile, m-tile); the list is
// derived on the device from the pack offsets, so there is no host synchronisation and no
// per-call pointer table.  Tiles of one expert that share a weight n-tile are adjacent in the
// list, so CTAs that run at the same time read the same weight tile through L2.
//
// Tile 128 x BN x 64, UMMA 128 x BN x 16 (fp16 in, fp32 accumulate in TMEM); an expert's last tile
// with at most 64 rows is issued as UMMA 64 x BN x 16 instead.  Two TMEM accumulators:
// the epilogue of tile i (TMEM -> registers -> activation -> fp16 -> global, rows past the end of
// the expert's segment masked) overlaps the main loop of tile i+1.
// Pair mode (experts with many rows, 256 accumulator columns): a work unit is two adjacent 128-row
// tiles of one expert that share every weight stage, one per TMEM accumulator, so the weight tile
// is fetched from L2 once per 256 rows instead of once per 128 (operand traffic per FLOP drops by a
// third; with 128 x 256 tiles the kernel is bound by L2 -> shared-memory traffic, not by the tensor
// pipe).  Both accumulators then belong to the same unit, so the epilogue overlaps the next unit's
// main loop only from its second half on.  An expert with an odd number of tiles ends with a
// single-tile unit.  (Those experts run on the two-CTA kernel further down unless it is switched
// off; pair mode is what remains then.)
// Warp roles (352 threads): warps 0 and 10 = TMA producers, warp 1 = TMEM owner + MMA issuer,
// warps 2..9 = epilogue (warp w reads TMEM lanes 32*(w%4)..; the two warps of a lane quarter split
// the tile's columns).
// Two kernels serve a call: this one-CTA kernel and grouped_gemm_cta2_kernel; the routed row count,
// read on the device, decides which of them works (the other returns at once).
//
// Scattered output (`c_rows`): instead of row r of a dense C, every output row goes to its own base
// address, which may lie in another GPU's memory (a peer mapping).  The expert-parallel layer uses
// this for the combine direction: the second expert GEMM stores each result row straight into the
// packed slot of the rank the row came from, over NVLink, from the same kernel that computes it
// (plain 128-bit stores; no TMA and no multicast on peer memory).  The epilogue warp stages 32 rows
// x 64 columns in shared memory and stores them as 128-byte row pieces, 4 rows per instruction,
// so that a peer store is a full 128-byte write, not 32 scattered 16-byte ones.
#include <atomic>
#include <cstdlib>

#include "sm100.cuh"

namespace moe {
namespace {

using namespace sm100;

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kUK = 16;
constexpr int kThreads = 352;  // warp 0 producer, warp 1 MMA issuer, warps 2..9 epilogue, warp 10 second producer
constexpr int kEpiThreads = 256;
constexpr int kProducerWarps = 2;
constexpr int kABytes = kBM * kBK * 2;
constexpr int kMaxStages = 8;
constexpr int kMaxExperts = 1024;

struct GParams {
  const int32_t* offsets;
  int experts, rows, K, n_out, bn, n_tiles, kblocks, stages;
  int w_kn;     // 1: weights stored [K, N] (N contiguous) -> MN-major B operand
  int act;      // MOE_ACT_*
  const float* row_scale;
  const uint16_t* bias;  // [experts, n_w] in the data type, or null
  int bf16;              // 0: fp16 data, 1: bf16 data
  uint16_t* c;
  uint16_t* const* c_rows;  // null: dense C; else base address of every output row
  int pair_min_avg;         // pair mode when the experts hold at least this many rows on average (0: never)
  int stages_pair;          // pipeline depth in pair mode (stages: single-tile units)
  int stage_area;           // bytes reserved for the stage ring (the larger of the two layouts)
  int producers;            // warps that issue TMA copies with single-tile units (1..2)
  int m64;                  // 1: a last tile of <= 64 rows runs as UMMA M=64; 0: every tile is 128 rows
  int cta2_min_avg;         // two-CTA kernel when the experts hold at least this many rows on average (0: never)
  int stages_cta2;          // pipeline depth of the two-CTA kernel
  int cta2_issuers;         // its MMA-issuing threads (1 or 2)
  int32_t* status;
};

constexpr int kStageRowBytes = 144;               // 64 columns x 2 B + 16 B pad: conflict-free both ways
constexpr int kStageWarpBytes = 32 * kStageRowBytes;

__device__ __forceinline__ float gelu_erf(float v) { return 0.5f * v * (1.f + erff(v * 0.70710678118654752f)); }
__device__ __forceinline__ float silu(float v) { return v / (1.f + __expf(-v)); }

// An expert's segment [seg_lo, seg_hi) of the row buffer, whatever the offsets array holds: both ends
// are forced into [0, rows] and hi >= lo, so offsets that are not (yet) valid - read before the
// kernel that writes them has run, say - cost at most rows/128 + experts tiles and never address a
// row outside the buffer.
__device__ __forceinline__ int seg_lo(const GParams& p, int e) { return max(0, min(p.offsets[e], p.rows)); }
__device__ __forceinline__ int seg_hi(const GParams& p, int e) { return max(seg_lo(p, e), min(p.offsets[e + 1], p.rows)); }
__device__ __forceinline__ int routed_rows(const GParams& p) { return max(0, min(p.offsets[p.experts], p.rows)); }

// Whether this call runs on the two-CTA kernel: decided on the device from the number of rows
// actually routed (the host only knows the capacity of the row buffer); both kernels of a call
// evaluate it and exactly one of them does the work.
__device__ __forceinline__ bool cta2_mode(const GParams& p, int routed) {
  return p.cta2_min_avg > 0 && (long long)routed >= (long long)p.cta2_min_avg * p.experts;
}

// Work unit id -> (expert, n tile, first row, whether the unit has a second 128-row tile).
// Units [0, n_a * n_tiles) are class A: single 128-row tiles, or in pair mode the full two-tile
// units; s_a[e] = class A units (per n tile) of experts < e.  In pair mode the experts with an odd
// number of tiles add one single-tile unit each, class B, listed after all of class A (s_b[e] = such
// experts < e): equal-cost units stay together, so the round-robin over the persistent CTAs hands
// every CTA the same mix.  Inside a class, units of one expert that share a weight n tile are adjacent.
struct Unit {
  int e, nt, row0;
  bool two;
};
__device__ __forceinline__ int last_not_above(const int32_t* pre, int n, int n_tiles, int t) {
  int lo = 0, hi = n;  // largest e with pre[e] * n_tiles <= t
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if ((long long)pre[mid] * n_tiles <= t) lo = mid; else hi = mid;
  }
  return lo;
}
__device__ __forceinline__ Unit decode_unit(const int32_t* s_a, const int32_t* s_b, const GParams& p, int pair, int t) {
  Unit u;
  const int experts = p.experts, n_tiles = p.n_tiles;
  const int total_a = s_a[experts] * n_tiles;
  if (t < total_a) {
    u.e = last_not_above(s_a, experts, n_tiles, t);
    const int per = s_a[u.e + 1] - s_a[u.e];
    const int local = t - s_a[u.e] * n_tiles;
    u.nt = local / per;
    u.row0 = seg_lo(p, u.e) + (local % per) * (pair ? 2 * kBM : kBM);
    u.two = pair != 0;
  } else {
    const int tb = t - total_a;
    u.e = last_not_above(s_b, experts, n_tiles, tb);
    u.nt = tb - s_b[u.e] * n_tiles;
    const int lo = seg_lo(p, u.e), cnt = seg_hi(p, u.e) - lo;
    u.row0 = lo + ((cnt + kBM - 1) / kBM - 1) * kBM;  // the expert's last tile
    u.two = false;
  }
  return u;
}

template <int W>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float (&v)[W]) {
  if constexpr (W == 32) tmem_ld32(taddr, v); else tmem_ld16(taddr, v);
}

__device__ __forceinline__ float load16(const uint16_t* p, bool bf16) {
  return bf16 ? __bfloat162float(__ushort_as_bfloat16(*p)) : __half2float(__ushort_as_half(*p));
}
__device__ __forceinline__ uint32_t pack16x2(float a, float b, bool bf16) {
  if (bf16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// W accumulator columns of one row: TMEM -> registers -> (+bias) -> activation -> 16-bit -> global.
// bias_main / bias_up point at the bias entries of these columns (null: no bias).
template <int W>
__device__ __forceinline__ void epilogue_chunk(uint32_t t_main, uint32_t t_up, bool swiglu, int act, float scale,
                                               bool valid, uint16_t* dst_h, const uint16_t* bias_main,
                                               const uint16_t* bias_up, bool bf16) {
  float v[W];
  tmem_ld<W>(t_main, v);
  if (bias_main != nullptr) {
#pragma unroll
    for (int i = 0; i < W; ++i) v[i] += load16(bias_main + i, bf16);
  }
  if (swiglu) {
    float u[W];
    tmem_ld<W>(t_up, u);
    if (bias_up != nullptr) {
#pragma unroll
      for (int i = 0; i < W; ++i) u[i] += load16(bias_up + i, bf16);
    }
#pragma unroll
    for (int i = 0; i < W; ++i) v[i] = silu(v[i]) * u[i];
  } else if (act == MOE_ACT_GELU) {
#pragma unroll
    for (int i = 0; i < W; ++i) v[i] = gelu_erf(v[i]);
  } else if (act == MOE_ACT_SILU) {
#pragma unroll
    for (int i = 0; i < W; ++i) v[i] = silu(v[i]);
  }
  if (valid) {
    uint4* dst = reinterpret_cast<uint4*>(dst_h);
#pragma unroll
    for (int i = 0; i < W / 8; ++i) {
      uint4 o;
      o.x = pack16x2(v[8 * i + 0] * scale, v[8 * i + 1] * scale, bf16);
      o.y = pack16x2(v[8 * i + 2] * scale, v[8 * i + 3] * scale, bf16);
      o.z = pack16x2(v[8 * i + 4] * scale, v[8 * i + 5] * scale, bf16);
      o.w = pack16x2(v[8 * i + 6] * scale, v[8 * i + 7] * scale, bf16);
      dst[i] = o;
    }
  }
}

// Store 32 staged rows x 64 columns (one epilogue warp's staging area, filled by epilogue_chunk with
// dst_h pointing into it) to the rows' own base addresses: lane l handles the 16-byte piece l%8 of
// row 4*i + l/8 in pass i.  `my_row` / `my_valid` describe the row this lane owns (row == lane).
__device__ __forceinline__ void store_staged_rows(const uint8_t* stage, uint16_t* my_row, bool my_valid, int col0,
                                                  int lane) {
  const unsigned long long mine = my_valid ? reinterpret_cast<unsigned long long>(my_row) : 0ull;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = 4 * i + (lane >> 3);
    const unsigned long long base = __shfl_sync(0xffffffffu, mine, r);
    const uint4 v = *reinterpret_cast<const uint4*>(stage + r * kStageRowBytes + (lane & 7) * 16);
    if (base != 0ull) *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(base) + col0 + (lane & 7) * 8) = v;
  }
}

// What an epilogue warp needs to know about itself.  Warp w of the eight reads TMEM lanes
// 32*(w%4)..; the two warps of a lane quarter split the tile's columns (dense output, >= 64 columns),
// otherwise the second warp of a quarter only takes part in the barriers.
struct EpiCtx {
  int q, lane, col_half, out_bn;
  bool split, swiglu;
  uint8_t* s_stage;
};
__device__ __forceinline__ EpiCtx make_epi_ctx(const GParams& p, int warp, int lane, uint8_t* s_stage) {
  EpiCtx c;
  c.q = warp & 3;
  c.lane = lane;
  c.col_half = (warp - 2) >> 2;  // 0: warps 2..5, 1: warps 6..9
  c.swiglu = p.act == MOE_ACT_SWIGLU;
  c.out_bn = c.swiglu ? p.bn / 2 : p.bn;  // output columns per tile
  c.split = p.c_rows == nullptr && c.out_bn >= 64;
  c.s_stage = s_stage;
  return c;
}

// Which rows and columns of a tile a TMEM lane holds.
enum : int {
  kAccM128 = 0,    // UMMA M=128 (or one CTA's half of a two-CTA M=256): lane = row, all columns
  kAccM64 = 1,     // as kAccM128, but a tile that holds at most 64 rows was issued as UMMA M=64: 16 rows in each
                   // 32-lane quarter (lanes 0..15 of the quarter)
  kAccPairM128 = 2 // one CTA's half (64 rows) of a two-CTA M=128: lanes 0..63 hold the rows' columns 0..N/2-1,
                   // lanes 64..127 the same rows' columns N/2..N-1, both at accumulator columns 0..N/2-1
};

// One accumulator (`tmem_acc`: TMEM address of its first column, lane 0) -> output rows row0.. of
// expert e, columns of n tile nt; rows at or past seg_end are masked.
__device__ __forceinline__ void epilogue_tile(const GParams& p, const EpiCtx& c, uint32_t tmem_acc, int e, int nt,
                                              int row0, int seg_end, int acc_layout) {
  const int out_bn = c.out_bn, lane = c.lane, q = c.q;
  const bool swiglu = c.swiglu;
  // accumulator columns this lane holds, and the output column (inside the n tile) of the first
  const int cols = acc_layout == kAccPairM128 ? out_bn / 2 : out_bn;
  const int col_off = acc_layout == kAccPairM128 ? (q >> 1) * (out_bn / 2) : 0;
  const int c_lo = c.split ? c.col_half * (cols / 2) : 0;
  const int c_hi = c.split ? c_lo + cols / 2 : (c.col_half == 0 ? cols : 0);
  if (c_lo >= c_hi) return;
  // bias of expert e: main columns at nt*out_bn, SwiGLU up columns n_out further
  const int n_w = swiglu ? 2 * p.n_out : p.n_out;
  const uint16_t* brow = p.bias ? p.bias + (size_t)e * n_w + (size_t)nt * out_bn + col_off : nullptr;
  int trow = q * 32 + lane;  // row of the tile held by this thread's TMEM lane
  bool lane_used = true;
  if (acc_layout == kAccM64 && seg_end - row0 <= 64) {
    trow = q * 16 + lane;
    lane_used = lane < 16;
  } else if (acc_layout == kAccPairM128) {
    trow = (q & 1) * 32 + lane;
  }
  const int grow = row0 + trow;
  const bool valid = lane_used && grow < seg_end && grow >= 0;
  const uint32_t acc = tmem_acc + ((uint32_t)(q * 32) << 16);
  const float scale = (valid && p.row_scale != nullptr) ? p.row_scale[grow] : 1.f;
  uint16_t* crow;
  if (p.c_rows == nullptr) crow = p.c + (size_t)(valid ? grow : 0) * p.n_out + (size_t)nt * out_bn + col_off;
  else crow = (valid ? p.c_rows[grow] : nullptr) + (size_t)nt * out_bn + col_off;
  if (p.c_rows != nullptr && out_bn % 64 == 0) {
    uint8_t* stage = c.s_stage + q * kStageWarpBytes;
    uint16_t* mine = reinterpret_cast<uint16_t*>(stage + lane * kStageRowBytes);
    for (int c0 = c_lo; c0 < c_hi; c0 += 64) {
#pragma unroll
      for (int hh = 0; hh < 64; hh += 32)
        epilogue_chunk<32>(acc + (uint32_t)(c0 + hh), acc + (uint32_t)(out_bn + c0 + hh), swiglu, p.act, scale, true,
                           mine + hh, brow ? brow + c0 + hh : nullptr,
                           (brow && swiglu) ? brow + p.n_out + c0 + hh : nullptr, p.bf16 != 0);
      __syncwarp();
      store_staged_rows(stage, crow, valid, c0, lane);
      __syncwarp();
    }
  } else if (out_bn % 64 == 0 || (!c.split && out_bn % 32 == 0)) {
    for (int c0 = c_lo; c0 < c_hi; c0 += 32)
      epilogue_chunk<32>(acc + (uint32_t)c0, acc + (uint32_t)(out_bn + c0), swiglu, p.act, scale, valid, crow + c0,
                         brow ? brow + c0 : nullptr, (brow && swiglu) ? brow + p.n_out + c0 : nullptr, p.bf16 != 0);
  } else {
    for (int c0 = c_lo; c0 < c_hi; c0 += 16)
      epilogue_chunk<16>(acc + (uint32_t)c0, acc + (uint32_t)(out_bn + c0), swiglu, p.act, scale, valid, crow + c0,
                         brow ? brow + c0 : nullptr, (brow && swiglu) ? brow + p.n_out + c0 : nullptr, p.bf16 != 0);
  }
}

// The weight boxes of one stage: f(byte offset inside the stage's B area, tensor-map coordinates).
template <typename F>
__device__ __forceinline__ void for_each_weight_box(const GParams& p, int BN, bool swiglu, int kb, int nt, int e, F&& f) {
  const int half = BN / 2;
  if (!p.w_kn) {
    // weights [E, Nw, K]: K-major B, one box of BN rows (SwiGLU: gate rows and up rows)
    if (!swiglu) {
      f(0u, kb * kBK, nt * BN, e);
    } else {
      f(0u, kb * kBK, nt * half, e);
      f((uint32_t)half * kBK * 2, kb * kBK, p.n_out + nt * half, e);
    }
  } else {
    // weights [E, K, Nw]: MN-major B, boxes of 64 (N) x 64 (K), one per 64 output columns
    for (int j = 0; j < BN / 64; ++j) {
      int ncol = nt * BN + j * 64;
      if (swiglu) ncol = (j < BN / 128) ? nt * half + j * 64 : p.n_out + nt * half + (j - BN / 128) * 64;
      f((uint32_t)j * 8192u, ncol, kb * kBK, e);
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                    const GParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {
    record_error(p.status, kErrBadIndex | 0xfe);
    return;
  }
  const int BN = p.bn;                    // accumulator columns per tile (256 / 128 / 64)
  const int b_bytes = BN * kBK * 2;
  // Pair mode is chosen here, from the number of rows actually routed (the host only knows the
  // capacity of the row buffer): every thread reads the same total and takes the same branch.
  const int routed = routed_rows(p);
  if (cta2_mode(p, routed)) return;  // grouped_gemm_cta2_kernel, launched next, does this call's work
  const int pair = (p.pair_min_avg > 0 && (long long)routed >= (long long)p.pair_min_avg * p.experts) ? 1 : 0;
  const int n_stages = pair ? p.stages_pair : p.stages;
  const int PM = pair ? 2 : 1;            // 128-row tiles per work unit
  const int a_stage = kABytes * PM;       // A bytes per stage
  uint8_t* sA = smem;
  uint8_t* sB = sA + (size_t)n_stages * a_stage;
  // the barriers sit behind the larger of the two stage layouts, at the same place in both modes
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + p.stage_area);
  // full[kMaxStages], empty[kMaxStages], tmem_full[2], tmem_empty[2]
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_bar + 2 * kMaxStages + 4);
  int32_t* s_mt = reinterpret_cast<int32_t*>(s_tmem + 4);  // [experts + 1] class A units before each expert
  int32_t* s_mb = s_mt + p.experts + 1;                    // [experts + 1] class B units before each expert
  // staging for scattered output rows: 4 epilogue warps x 32 rows x 144 B, 16-byte aligned
  uint8_t* s_stage = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(s_mb + p.experts + 1) + 15) & ~static_cast<uintptr_t>(15));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t full0 = smem_u32(s_bar);
  const uint32_t empty0 = smem_u32(s_bar + kMaxStages);
  const uint32_t tfull0 = smem_u32(s_bar + 2 * kMaxStages);
  const uint32_t tempty0 = smem_u32(s_bar + 2 * kMaxStages + 2);
  const uint32_t tmem_cols = (uint32_t)(2 * BN < 32 ? 32 : 2 * BN);

  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull0 + 8 * b, 1);
      mbar_init(tempty0 + 8 * b, kEpiThreads);  // every epilogue thread arrives
    }
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(s_tmem), tmem_cols);
    tmem_relinquish();
  }
  // class A / class B units before each expert (serial prefix by one warp; experts <= 1024)
  if (warp == 2) {
    int carry_a = 0, carry_b = 0;
    for (int eb = 0; eb < p.experts; eb += 32) {
      const int e = eb + lane;
      int ca = 0, cb = 0;
      if (e < p.experts) {
        const int lo = seg_lo(p, e), hi = seg_hi(p, e);
        const int tiles = hi > lo ? (hi - lo + kBM - 1) / kBM : 0;
        ca = pair ? tiles / 2 : tiles;
        cb = pair ? tiles & 1 : 0;
      }
      int ia = ca, ib = cb;
#pragma unroll
      for (int ofs = 1; ofs < 32; ofs <<= 1) {
        const int na = __shfl_up_sync(0xffffffffu, ia, ofs);
        const int nb = __shfl_up_sync(0xffffffffu, ib, ofs);
        if (lane >= ofs) { ia += na; ib += nb; }
      }
      if (e < p.experts) { s_mt[e] = carry_a + ia - ca; s_mb[e] = carry_b + ib - cb; }
      carry_a += __shfl_sync(0xffffffffu, ia, 31);
      carry_b += __shfl_sync(0xffffffffu, ib, 31);
    }
    if (lane == 0) { s_mt[p.experts] = carry_a; s_mb[p.experts] = carry_b; }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  const int total_tiles = (s_mt[p.experts] + s_mb[p.experts]) * p.n_tiles;
  const bool swiglu = p.act == MOE_ACT_SWIGLU;

  if (warp == 0 || warp >= 10) {
    // ------------------------------ TMA producers ------------------------------
    // The bulk tensor copies of ONE thread are served one after another (about 0.35 us each on B200).
    // With single-tile units (two boxes per 48 KiB stage, four stages) a second issuing warp measured
    // 5-6 % faster (32 x 256 rows: 1228 -> 1163 us, 64 x 128: 1539 -> 1454 us); pair-mode units are not
    // issue-bound and measured 0-3 % slower with it, so they keep one.  Producer j owns the stages s
    // with s % producers == j and fills them in order (a stage's barrier parity is never ambiguous).
    const int pw = warp == 0 ? 0 : warp - 9;
    const int producers = pair ? 1 : min(p.producers, n_stages);
    if (lane == 0 && pw < producers) {
      int s = 0;        // stage and the parity of its use, advanced without divisions (this thread is
      uint32_t ph = 0;  // on the critical path of its stages)
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const Unit u = decode_unit(s_mt, s_mb, p, pair, t);
        const int e = u.e, nt = u.nt, row0 = u.row0;
        const bool two = u.two;  // the unit has a second tile
        for (int kb = 0; kb < p.kblocks; ++kb) {
          const int s_now = s;
          const uint32_t ph_now = ph;
          if (++s == n_stages) { s = 0; ph ^= 1u; }
          if (producers == 2 && (s_now & 1) != pw) continue;
          if (!mbar_wait(empty0 + 8 * s_now, ph_now ^ 1u, p.status, 1)) { ok = false; break; }
          mbar_expect_tx(full0 + 8 * s_now, (uint32_t)(kABytes * (two ? 2 : 1) + b_bytes));
          tma_load_2d(smem_u32(sA + (size_t)s_now * a_stage), &tmap_a, full0 + 8 * s_now, kb * kBK, row0);
          if (two) tma_load_2d(smem_u32(sA + (size_t)s_now * a_stage + kABytes), &tmap_a, full0 + 8 * s_now, kb * kBK, row0 + kBM);
          const uint32_t sb = smem_u32(sB + (size_t)s_now * b_bytes);
          for_each_weight_box(p, BN, swiglu, kb, nt, e, [&](uint32_t ofs, int c0, int c1, int c2) {
            tma_load_3d(sb + ofs, &tmap_w, full0 + 8 * s_now, c0, c1, c2);
          });
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc128 = make_idesc_f16(kBM, BN, p.bf16, 0, p.w_kn);
      const uint32_t idesc64 = make_idesc_f16(64, BN, p.bf16, 0, p.w_kn);
      int s = 0;
      uint32_t ph = 0;
      int local = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
        const Unit u = decode_unit(s_mt, s_mb, p, pair, t);
        const int seg_end = seg_hi(p, u.e);
        const int row0 = u.row0;
        const bool two = u.two;
        // a last tile that holds at most 64 rows of its expert costs half the tensor time as M=64
        const uint32_t idesc_h0 = (p.m64 && seg_end - row0 <= 64) ? idesc64 : idesc128;
        const uint32_t idesc_h1 = (p.m64 && seg_end - (row0 + kBM) <= 64) ? idesc64 : idesc128;
        // accumulators: single-tile units alternate between the two; a pair unit owns both
        const int ab = pair ? 0 : (local & 1);
        const uint32_t par = pair ? ((uint32_t)local & 1u) : (((uint32_t)local >> 1) & 1u);
        if (!mbar_wait(tempty0 + 8 * ab, par ^ 1u, p.status, 4)) break;
        if (pair && !mbar_wait(tempty0 + 8, par ^ 1u, p.status, 4)) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + (uint32_t)(ab * BN);
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait(full0 + 8 * s, ph, p.status, 2)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + (size_t)s * a_stage);
          const uint32_t b_addr = smem_u32(sB + (size_t)s * b_bytes);
          const uint64_t adesc = make_desc_kmajor_sw128(a_addr);
#pragma unroll
          for (int k = 0; k < kBK / kUK; ++k) {
            uint64_t bdesc;
            if (!p.w_kn) bdesc = make_desc_kmajor_sw128(b_addr) + 2 * k;          // +32 B along K
            else bdesc = make_desc_mnmajor_sw128(b_addr + (uint32_t)k * 2048u, 8192u);  // +16 K rows of 128 B
            umma_f16(acc, adesc + 2 * k, bdesc, idesc_h0, (uint32_t)((kb | k) != 0));
          }
          if (two) {
            const uint64_t adesc1 = make_desc_kmajor_sw128(a_addr + (uint32_t)kABytes);
#pragma unroll
            for (int k = 0; k < kBK / kUK; ++k) {
              uint64_t bdesc;
              if (!p.w_kn) bdesc = make_desc_kmajor_sw128(b_addr) + 2 * k;
              else bdesc = make_desc_mnmajor_sw128(b_addr + (uint32_t)k * 2048u, 8192u);
              umma_f16(acc + (uint32_t)BN, adesc1 + 2 * k, bdesc, idesc_h1, (uint32_t)((kb | k) != 0));
            }
          }
          umma_commit(empty0 + 8 * s);
          if (++s == n_stages) { s = 0; ph ^= 1u; }
        }
        umma_commit(tfull0 + 8 * ab);
        if (pair) umma_commit(tfull0 + 8);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue -----------------------------------
    const EpiCtx ec = make_epi_ctx(p, warp, lane, s_stage);
    int local = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
      const Unit u = decode_unit(s_mt, s_mb, p, pair, t);
      const int e = u.e, nt = u.nt;
      const int seg_end = seg_hi(p, e);
      for (int h = 0; h < PM; ++h) {
        const int ab = pair ? h : (local & 1);
        const uint32_t par = pair ? ((uint32_t)local & 1u) : (((uint32_t)local >> 1) & 1u);
        const int row0 = u.row0 + h * kBM;
        if (!mbar_wait(tfull0 + 8 * ab, par, p.status, 3)) { ok = false; break; }
        tc_fence_after();
        // (the second accumulator of a single-tile unit holds nothing)
        if (h == 0 || u.two)
          epilogue_tile(p, ec, tmem_base + (uint32_t)(ab * BN), e, nt, row0, seg_end, p.m64 ? kAccM64 : kAccM128);
        tc_fence_before();
        mbar_arrive(tempty0 + 8 * ab);  // this thread is done reading the accumulator
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}


// ---------------------------------------------------------------------------------------------------
// Two-CTA kernel (experts with many rows, 256 accumulator columns).  A cluster of two CTAs works on a
// unit of 256 rows x one n tile of one expert with `tcgen05.mma.cta_group::2`: D = 256 x 256 per
// instruction, rows 0..127 in the even CTA's TMEM and rows 128..255 in the odd CTA's.  CTA r loads its
// own 128 rows of A and ITS HALF of the weight tile (128 of the 256 accumulator columns; the tensor
// core reads the other half from the other CTA's shared memory), so the operand bytes per FLOP are
// those of a 256 x 256 tile while every CTA keeps two 256-column accumulators: the epilogue of unit
// i (GELU costs about 9,000 cycles per 128 x 256 tile, more than a quarter of the tile's tensor time)
// runs entirely under the main loop of unit i+1, which two-tile units of one CTA cannot do (their two
// accumulators belong to one unit; the MMA thread then idles a fifth of the time).
// The copies are ordinary TMA loads of this GPU's memory into the issuing CTA's own shared memory;
// only their completion is signalled to the even CTA's barrier.  The even CTA's thread issues the
// MMAs; its commits arrive on the barriers of both CTAs.
// Warp roles (448 threads): warps 0, 10, 11, 12 issue the TMA copies (copies of one thread are served
// one after another, so the operand boxes are spread over four), warp 1 owns TMEM, warps 1 and 13 of
// the even CTA issue the MMAs, warps 2..9 are the epilogue of the CTA's own 128 rows.
// An expert with an odd number of 128-row tiles ends with a unit of one tile, issued as a two-CTA
// M=128 (64 rows per CTA, half the tensor time; the accumulator then holds each row's two column
// halves on lanes l and l+64).  SwiGLU pairs a row's gate and up columns inside one lane, so there the
// last unit stays M=256 with its second half past the expert's rows, computed and masked.  The
// one-tile units are listed after all full ones, so the round-robin hands every cluster the same mix.
constexpr int kCThreads = 448;
// A stage holds two 64-wide k blocks of each operand (A block 0 | A block 1 | weight-half block 0 |
// weight-half block 1, 16 KiB each): the commit that frees a stage costs the issuing thread about as
// much as four MMAs, and with one k block per stage (six 32 KiB stages) the kernel measured 20 %
// slower, bound by that thread.
constexpr int kCKH = 2;
constexpr int kCStageBytes = kCKH * 2 * kABytes;
constexpr int kCRows = 2 * kBM;            // rows per unit

struct CUnit {
  int e, nt, row0;
  bool one;  // the expert's odd last tile
};
// Inside a class, units are ordered by expert, then n tile, then row group, so clusters that run at
// the same time share weight tiles through L2.  s_a[e] / s_b[e] = full / one-tile units (per n tile)
// of experts < e.
__device__ __forceinline__ CUnit decode_cta2(const int32_t* s_a, const int32_t* s_b, const GParams& p, int t) {
  CUnit u;
  const int total_a = s_a[p.experts] * p.n_tiles;
  if (t < total_a) {
    u.e = last_not_above(s_a, p.experts, p.n_tiles, t);
    const int per = s_a[u.e + 1] - s_a[u.e];
    const int local = t - s_a[u.e] * p.n_tiles;
    u.nt = local / per;
    u.row0 = seg_lo(p, u.e) + (local % per) * kCRows;
    u.one = false;
  } else {
    const int tb = t - total_a;
    u.e = last_not_above(s_b, p.experts, p.n_tiles, tb);
    u.nt = tb - s_b[u.e] * p.n_tiles;
    u.row0 = seg_lo(p, u.e) + (s_a[u.e + 1] - s_a[u.e]) * kCRows;  // after the expert's full units
    u.one = true;
  }
  return u;
}

__global__ void __launch_bounds__(kCThreads, 1)
grouped_gemm_cta2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_a64,
                         const __grid_constant__ CUtensorMap tmap_w, const GParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  // every CTA reads the same total and takes the same branch (no barrier has been touched yet)
  if (!cta2_mode(p, routed_rows(p))) return;
  if ((smem_u32(smem) & 1023u) != 0u) {  // the same in both CTAs of a pair
    record_error(p.status, kErrBadIndex | 0xfd);
    return;
  }
  constexpr int BN = 256;
  constexpr int KH = kCKH;
  const int n_stages = p.stages_cta2;
  const int kblocks = (p.kblocks + KH - 1) / KH;  // stages per unit
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + (size_t)n_stages * kCStageBytes);
  // full[kMaxStages] (used in the even CTA), empty[kMaxStages], tmem_full[2], tmem_empty[2] (even CTA)
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_bar + 2 * kMaxStages + 4);
  uint32_t* s_seq = s_tmem + 1;                            // stages issued so far (two MMA-issuing threads)
  int32_t* s_mt = reinterpret_cast<int32_t*>(s_tmem + 4);  // [experts + 1] full units before each expert
  int32_t* s_mb = s_mt + p.experts + 1;                    // [experts + 1] one-tile units before each expert
  uint8_t* s_stage = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(s_mb + p.experts + 1) + 15) & ~static_cast<uintptr_t>(15));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: the CTA that issues the MMAs
  const int cluster = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const uint32_t full0 = smem_u32(s_bar);
  const uint32_t empty0 = smem_u32(s_bar + kMaxStages);
  const uint32_t tfull0 = smem_u32(s_bar + 2 * kMaxStages);
  const uint32_t tempty0 = smem_u32(s_bar + 2 * kMaxStages + 2);
  constexpr uint32_t kTmemCols = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(full0 + 8 * s, 1);   // the even CTA's producer arrives with the byte count of both CTAs
      mbar_init(empty0 + 8 * s, 1);  // one commit per use
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull0 + 8 * b, (uint32_t)p.cta2_issuers);  // one commit per MMA-issuing thread
      mbar_init(tempty0 + 8 * b, 2 * kEpiThreads);          // every epilogue thread of both CTAs arrives
    }
    *s_seq = 0;
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_a64);
    prefetch_tensormap(&tmap_w);
  }
  if (warp == 1) {
    // each CTA allocates all of its own TMEM, so both get the same base address
    tmem_alloc(smem_u32(s_tmem), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 2) {
    int carry_a = 0, carry_b = 0;
    for (int eb = 0; eb < p.experts; eb += 32) {
      const int e = eb + lane;
      int ca = 0, cb = 0;
      if (e < p.experts) {
        const int lo = seg_lo(p, e), hi = seg_hi(p, e);
        const int tiles = hi > lo ? (hi - lo + kBM - 1) / kBM : 0;
        ca = tiles / 2;
        cb = tiles & 1;
      }
      int ia = ca, ib = cb;
#pragma unroll
      for (int ofs = 1; ofs < 32; ofs <<= 1) {
        const int na = __shfl_up_sync(0xffffffffu, ia, ofs);
        const int nb = __shfl_up_sync(0xffffffffu, ib, ofs);
        if (lane >= ofs) { ia += na; ib += nb; }
      }
      if (e < p.experts) { s_mt[e] = carry_a + ia - ca; s_mb[e] = carry_b + ib - cb; }
      carry_a += __shfl_sync(0xffffffffu, ia, 31);
      carry_b += __shfl_sync(0xffffffffu, ib, 31);
    }
    if (lane == 0) { s_mt[p.experts] = carry_a; s_mb[p.experts] = carry_b; }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before any copy or arrival names them
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  const int total_units = (s_mt[p.experts] + s_mb[p.experts]) * p.n_tiles;
  const bool swiglu = p.act == MOE_ACT_SWIGLU;

  if (warp == 0 || (warp >= 10 && warp <= 12)) {
    // ------------------------------ TMA producers ------------------------------
    // Producers 0/1 copy the two k blocks of this CTA's rows of A, producers 2/3 those of its half of
    // the weight tile.  Every producer waits for the stage to be free in its own CTA; the bytes of both CTAs complete on the
    // even CTA's `full` barrier, armed by the even CTA's producer of the stage's first A block.
    const int op = warp == 0 ? 0 : warp - 9;
    const int which = op >> 1, sub = op & 1;
    if (lane == 0) {
      int s = 0;         // stage and the parity of its use, advanced without divisions
      uint32_t ph = 0;
      bool ok = true;
      for (int t = cluster; t < total_units && ok; t += n_clusters) {
        const CUnit u = decode_cta2(s_mt, s_mb, p, t);
        const bool m128 = u.one && !swiglu;  // one tile as a two-CTA M=128: 64 rows of A per CTA
        // first weight row (column, for [K, N] weights) of this CTA's half: SwiGLU tiles hold the gate
        // columns in the even CTA's half and the up columns in the odd CTA's
        const int n0 = swiglu ? (int)rank * p.n_out + u.nt * (BN / 2) : u.nt * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, 1)) { ok = false; break; }
          const uint32_t full_even = map_to_cta(full0 + 8 * s, 0);
          const int h = sub;  // k block of the stage
          const uint32_t st = smem_u32(smem + (size_t)s * kCStageBytes) + (uint32_t)((which * KH + h) * kABytes);
          const int k0 = (kb * KH + h) * kBK;
          if (which == 0 && h == 0 && rank == 0)
            mbar_expect_tx(full0 + 8 * s, (uint32_t)(m128 ? 2 * KH * (kABytes / 2 + kABytes) : 2 * kCStageBytes));
          if (which == 0) {
            if (m128) tma_load_2d_pair(st, &tmap_a64, full_even, k0, u.row0 + (int)rank * (kBM / 2));
            else tma_load_2d_pair(st, &tmap_a, full_even, k0, u.row0 + (int)rank * kBM);
          } else if (!p.w_kn) {
            tma_load_3d_pair(st, &tmap_w, full_even, k0, n0, u.e);  // 128 rows of the K-major tile
          } else {
            // weights [E, K, Nw]: two boxes of 64 (N) x 64 (K)
            tma_load_3d_pair(st, &tmap_w, full_even, n0, k0, u.e);
            tma_load_3d_pair(st + 8192u, &tmap_w, full_even, n0 + 64, k0, u.e);
          }
          if (++s == n_stages) { s = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1 || warp == 13) {
    // ------------------------------ MMA issuers (even CTA) ---------------------
    // Issuing a stage's eight MMAs and the commit that frees the stage takes one thread about as long
    // as the tensor pipe needs to run them, so two threads take the stages alternately: while one sits
    // in its commit the other issues.  They issue strictly in stage order (`s_seq` counts the stages
    // issued; warps 1 and 13 share a scheduler), so the accumulation order, and with it every result
    // bit, is the same as with one thread.  Each thread commits its own MMAs: a stage's `empty`
    // barrier by the thread that issued the stage, the unit's `tmem_full` barrier by both.
    const int issuers = p.cta2_issuers;
    const int me = warp == 1 ? 0 : 1;
    if (lane == 0 && rank == 0 && me < issuers) {
      const uint32_t idesc256 = make_idesc_f16(2 * kBM, BN, p.bf16, 0, p.w_kn);
      const uint32_t idesc128 = make_idesc_f16(kBM, BN, p.bf16, 0, p.w_kn);
      const int total_a = s_mt[p.experts] * p.n_tiles;
      volatile uint32_t* seq = s_seq;
      int s = 0;
      uint32_t ph = 0;
      uint32_t g = 0;  // stages since the start of the kernel
      int local = 0;
      bool ok = true;
      for (int t = cluster; t < total_units && ok; t += n_clusters, ++local) {
        const uint32_t idesc = (t >= total_a && !swiglu) ? idesc128 : idesc256;
        const int ab = local & 1;  // units alternate between the two accumulators
        const uint32_t par = ((uint32_t)local >> 1) & 1u;
        const uint32_t acc = tmem_base + (uint32_t)(ab * BN);
        // The epilogue must have drained the accumulator before the unit's first MMA overwrites it.
        // Both threads wait, also the one that issues later stages or none: its commit on `tmem_full`
        // below must not fall into the barrier phase of the accumulator's previous unit.
        if (!mbar_wait(tempty0 + 8 * ab, par ^ 1u, p.status, 4)) break;
        for (int kb = 0; kb < kblocks; ++kb, ++g) {
          const int s_now = s;
          const uint32_t ph_now = ph;
          if (++s == n_stages) { s = 0; ph ^= 1u; }
          if (issuers == 2 && (int)(g & 1u) != me) continue;
          if (!mbar_wait(full0 + 8 * s_now, ph_now, p.status, 2)) { ok = false; break; }
          if (issuers == 2) {
            // my turn: every earlier stage has been issued (bounded like every other wait)
            bool turn = false;
            for (int spin = 0; spin < (1 << 26); ++spin)
              if (*seq == g) { turn = true; break; }
            if (!turn) { record_error(p.status, kErrMbarTimeout | 5); ok = false; break; }
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s_now * kCStageBytes);
          const uint32_t b_addr = a_addr + KH * kABytes;
#pragma unroll
          for (int h = 0; h < KH; ++h) {
            const uint64_t adesc = make_desc_kmajor_sw128(a_addr + (uint32_t)(h * kABytes));
#pragma unroll
            for (int k = 0; k < kBK / kUK; ++k) {
              uint64_t bdesc;
              if (!p.w_kn) bdesc = make_desc_kmajor_sw128(b_addr + (uint32_t)(h * kABytes)) + 2 * k;  // +32 B along K
              else bdesc = make_desc_mnmajor_sw128(b_addr + (uint32_t)(h * kABytes) + (uint32_t)k * 2048u, 8192u);
              umma_f16_pair(acc, adesc + 2 * k, bdesc, idesc, (uint32_t)((kb | h | k) != 0));
            }
          }
          if (issuers == 2) {
            tc_fence_before();
            *seq = g + 1;  // the other thread may issue the next stage
          }
          umma_commit_pair(empty0 + 8 * s_now, 3);  // the stage is free in both CTAs
        }
        if (ok) umma_commit_pair(tfull0 + 8 * ab, 3);  // (a thread without a stage in this unit arrives at once)
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (both CTAs) -----------------------
    const EpiCtx ec = make_epi_ctx(p, warp, lane, s_stage);
    const uint32_t tempty_even = map_to_cta(tempty0, 0);
    int local = 0;
    for (int t = cluster; t < total_units; t += n_clusters, ++local) {
      const CUnit u = decode_cta2(s_mt, s_mb, p, t);
      const int seg_end = seg_hi(p, u.e);
      const int ab = local & 1;
      if (!mbar_wait(tfull0 + 8 * ab, ((uint32_t)local >> 1) & 1u, p.status, 3)) break;
      tc_fence_after();
      if (u.one && !swiglu)
        epilogue_tile(p, ec, tmem_base + (uint32_t)(ab * BN), u.e, u.nt, u.row0 + (int)rank * (kBM / 2), seg_end, kAccPairM128);
      else
        epilogue_tile(p, ec, tmem_base + (uint32_t)(ab * BN), u.e, u.nt, u.row0 + (int)rank * kBM, seg_end, kAccM128);
      tc_fence_before();
      mbar_arrive_cluster(tempty_even + 8 * ab);  // this thread is done reading the accumulator
    }
    __syncwarp();
  }

  // no CTA leaves (or frees TMEM) while the other may still read its shared memory or signal its barriers
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace
}  // namespace moe

namespace moe {
namespace {
// Which variants the grouped GEMM may use (MOE_GEMM_* bits).  Set from the environment at first use,
// changed by moe_set_gemm_mode; every variant computes the same bits, the fastest set is the default.
std::atomic<int> g_gemm_mode{-1};
int gemm_mode() {
  int m = g_gemm_mode.load(std::memory_order_relaxed);
  if (m >= 0) return m;
  auto off = [](const char* name) { const char* v = getenv(name); return v && v[0] == '0'; };
  m = MOE_GEMM_ALL;
  if (off("MOE_B200_CTA2")) m &= ~MOE_GEMM_TWO_CTA;
  if (off("MOE_B200_PAIR")) m &= ~MOE_GEMM_TILE_PAIRS;
  if (off("MOE_B200_M64")) m &= ~MOE_GEMM_M64;
  { const char* v = getenv("MOE_B200_CTA2_ISSUERS"); if (v && v[0] == '1') m &= ~MOE_GEMM_TWO_ISSUERS; }
  { const char* v = getenv("MOE_B200_GEMM_PRODUCERS"); if (v && v[0] == '1') m &= ~MOE_GEMM_TWO_PRODUCERS; }
  g_gemm_mode.store(m, std::memory_order_relaxed);
  return m;
}

int grouped_gemm_launch(const void* a, const void* w, void* c, void* const* c_rows, const int32_t* offsets,
                        int experts, int rows, int K, int N, int w_layout, int64_t stride_w, int activation,
                        const float* row_scale, const void* bias, int dtype, int sm_margin, void* workspace,
                        size_t workspace_bytes, void* stream) {
  if (experts <= 0 || rows < 0 || K <= 0 || N <= 0) return fail(MOE_ERR_ARG, "moe_grouped_gemm: bad shape");
  if (experts > kMaxExperts) return fail(MOE_ERR_UNSUPPORTED, "moe_grouped_gemm: experts must be <= %d", kMaxExperts);
  if (K % 8 != 0) return fail(MOE_ERR_UNSUPPORTED, "moe_grouped_gemm: K must be a multiple of 8, got %d", K);
  if (N % 16 != 0) return fail(MOE_ERR_UNSUPPORTED, "moe_grouped_gemm: N must be a multiple of 16, got %d", N);
  if (w_layout == MOE_W_KN && N % 64 != 0)
    return fail(MOE_ERR_UNSUPPORTED, "moe_grouped_gemm: N must be a multiple of 64 for [K,N] weights, got %d", N);
  if (activation < MOE_ACT_NONE || activation > MOE_ACT_SWIGLU) return fail(MOE_ERR_ARG, "moe_grouped_gemm: bad activation");
  if (w_layout != MOE_W_KN && w_layout != MOE_W_NK) return fail(MOE_ERR_ARG, "moe_grouped_gemm: bad weight layout");
  if (dtype != MOE_F16 && dtype != MOE_BF16) return fail(MOE_ERR_ARG, "moe_grouped_gemm: dtype must be fp16 or bf16");
  if (rows == 0) return MOE_OK;
  if (!a || !w || (!c && !c_rows) || !offsets) return fail(MOE_ERR_ARG, "moe_grouped_gemm: null pointer");
  if (!workspace || workspace_bytes < (size_t)kStatusBytes) return fail(MOE_ERR_WORKSPACE, "moe_grouped_gemm: workspace missing");
  // the epilogue stores 128-bit pieces; bias is read with 128-bit loads
  if (c != nullptr && (reinterpret_cast<uintptr_t>(c) & 15) != 0)
    return fail(MOE_ERR_ARG, "moe_grouped_gemm: c must be 16-byte aligned");
  if (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 15) != 0)
    return fail(MOE_ERR_ARG, "moe_grouped_gemm: bias must be 16-byte aligned");
  const bool swiglu = activation == MOE_ACT_SWIGLU;
  const int n_w = swiglu ? 2 * N : N;  // output features held by one weight matrix

  GParams p;
  p.offsets = offsets; p.experts = experts; p.rows = rows; p.K = K; p.n_out = N;
  // accumulator columns per tile; SwiGLU tiles hold `bn/2` gate and `bn/2` up columns
  int out_bn = N % 256 == 0 ? 256 : (N % 128 == 0 ? 128 : (N % 64 == 0 ? 64 : (N % 32 == 0 ? 32 : 16)));
  if (swiglu && out_bn > 128) out_bn = 128;
  p.bn = swiglu ? 2 * out_bn : out_bn;
  p.n_tiles = N / out_bn;
  p.kblocks = (K + kBK - 1) / kBK;
  p.w_kn = w_layout == MOE_W_KN;
  p.act = activation;
  p.row_scale = row_scale;
  p.c = static_cast<uint16_t*>(c);
  p.c_rows = reinterpret_cast<uint16_t* const*>(c_rows);
  const int mode = gemm_mode();
  // an expert's last tile runs as UMMA M=64 when it holds at most 64 rows: half the tensor time for it
  p.m64 = (mode & MOE_GEMM_M64) ? 1 : 0;
  p.producers = (mode & MOE_GEMM_TWO_PRODUCERS) ? kProducerWarps : 1;
  p.bias = static_cast<const uint16_t*>(bias);
  p.bf16 = dtype == MOE_BF16;
  p.status = static_cast<int32_t*>(workspace);

  CUtensorMap tmap_a, tmap_w;
  int rc = encode_tmap_2d(&tmap_a, a, (uint64_t)rows, (uint64_t)K, (uint64_t)K * 2, kBK, kBM);
  if (rc != MOE_OK) return rc;
  if (!p.w_kn) {
    const uint32_t box_rows = swiglu ? (uint32_t)out_bn : (uint32_t)p.bn;
    rc = encode_tmap_3d(&tmap_w, w, (uint64_t)experts, (uint64_t)n_w, (uint64_t)K, (uint64_t)K * 2,
                        (uint64_t)stride_w * 2, kBK, box_rows);
  } else {
    rc = encode_tmap_3d(&tmap_w, w, (uint64_t)experts, (uint64_t)K, (uint64_t)n_w, (uint64_t)n_w * 2,
                        (uint64_t)stride_w * 2, 64, kBK);
  }
  if (rc != MOE_OK) return rc;

  const int stage_single = kABytes + p.bn * kBK * 2;
  const int stage_pair = 2 * kABytes + p.bn * kBK * 2;
  const int fixed = (2 * kMaxStages + 4) * 8 + 16 + 2 * (experts + 1) * 4 + 64 + (c_rows ? 4 * kStageWarpBytes + 16 : 0);
  int stages = (227 * 1024 - fixed) / stage_single;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return fail(MOE_ERR_UNSUPPORTED, "moe_grouped_gemm: shared memory budget exceeded");
  p.stages = stages;
  {
    // Pair mode (see the top of the file) pays when experts hold several full tiles: measured +10 %
    // at 8 x 1024 rows, +3 % at 8 x ~1030 and 16 x ~515, -7 % at 32 x ~260 rows (the epilogue of a
    // pair is not hidden behind the next main loop).
    const int pair_on = (mode & MOE_GEMM_TILE_PAIRS) ? 1 : 0;
    int stages_pair = (227 * 1024 - fixed) / stage_pair;
    if (stages_pair > kMaxStages) stages_pair = kMaxStages;
    p.stages_pair = stages_pair;
    p.pair_min_avg = (pair_on && p.bn == 256 && stages_pair >= 2) ? 4 * kBM : 0;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  if (sm_margin > 0 && sm_margin < sms) sms -= sm_margin;
  {
    // The two-CTA kernel takes the calls whose experts hold 512 rows or more on average (it replaces
    // the two-tile units of one CTA there).
    const int cta2_on = (mode & MOE_GEMM_TWO_CTA) ? 1 : 0;
    int stages_cta2 = (227 * 1024 - fixed) / kCStageBytes;
    if (stages_cta2 > kMaxStages) stages_cta2 = kMaxStages;
    p.stages_cta2 = stages_cta2;
    p.cta2_issuers = (mode & MOE_GEMM_TWO_ISSUERS) ? 2 : 1;
    // Below 512 rows per expert the odd last tiles weigh too much: a one-tile unit costs the two-CTA
    // kernel almost a full unit's time (24 x 384 rows: 1390-1410 us against 1170-1180 on the one-CTA
    // kernel; 32 x 256 rows, no odd tiles: 1060 against 1120).
    p.cta2_min_avg = (cta2_on && p.bn == 256 && stages_cta2 >= 2 && sms >= 2) ? 4 * kBM : 0;
  }
  size_t stage_area = (size_t)stages * stage_single;
  if (p.pair_min_avg && (size_t)p.stages_pair * stage_pair > stage_area) stage_area = (size_t)p.stages_pair * stage_pair;
  p.stage_area = (int)stage_area;
  const size_t smem = stage_area + fixed;

  // upper bound of the tile count known on the host: every expert may add one partial m tile
  const long long max_tiles = ((long long)rows / kBM + experts) * p.n_tiles;
  const int grid = (int)(max_tiles < sms ? max_tiles : sms);

  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "moe_grouped_gemm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  grouped_gemm_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(tmap_a, tmap_w, p);
  rc = check_launch("grouped_gemm_kernel");
  if (rc != MOE_OK || p.cta2_min_avg == 0) return rc;

  // The two-CTA kernel: whichever of the two kernels the routed row count selects does the work, the
  // other returns at once (the choice needs the offsets, which only the device has).
  CUtensorMap tmap_wq = tmap_w, tmap_a64;
  rc = encode_tmap_2d(&tmap_a64, a, (uint64_t)rows, (uint64_t)K, (uint64_t)K * 2, kBK, kBM / 2);
  if (rc != MOE_OK) return rc;
  if (!p.w_kn && !swiglu) {
    rc = encode_tmap_3d(&tmap_wq, w, (uint64_t)experts, (uint64_t)n_w, (uint64_t)K, (uint64_t)K * 2,
                        (uint64_t)stride_w * 2, kBK, 128);
    if (rc != MOE_OK) return rc;
  }
  const size_t smem_q = (size_t)p.stages_cta2 * kCStageBytes + fixed;
  const long long max_units = ((long long)rows / kCRows + experts) * p.n_tiles;
  const int clusters = (int)(max_units < sms / 2 ? max_units : sms / 2);
  e = cudaFuncSetAttribute(grouped_gemm_cta2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "moe_grouped_gemm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(kCThreads, 1, 1);
  cfg.dynamicSmemBytes = smem_q;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, grouped_gemm_cta2_kernel, tmap_a, tmap_a64, tmap_wq, p);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "moe_grouped_gemm: cluster launch: %s", cudaGetErrorString(e));
  return check_launch("grouped_gemm_cta2_kernel");
}
}  // namespace
}  // namespace moe

extern "C" int moe_grouped_gemm(const void* a, const void* w, void* c, const int32_t* offsets, int experts, int rows,
                                int K, int N, int w_layout, int64_t stride_w, int activation,
                                const float* row_scale, const void* bias, int dtype, int sm_margin,
                                void* workspace, size_t workspace_bytes, void* stream) {
  return moe::grouped_gemm_launch(a, w, c, nullptr, offsets, experts, rows, K, N, w_layout, stride_w, activation,
                                  row_scale, bias, dtype, sm_margin, workspace, workspace_bytes, stream);
}

extern "C" int moe_grouped_gemm_rows(const void* a, const void* w, void* const* c_rows, const int32_t* offsets,
                                     int experts, int rows, int K, int N, int w_layout, int64_t stride_w,
                                     int activation, const float* row_scale, const void* bias, int dtype,
                                     int sm_margin, void* workspace, size_t workspace_bytes, void* stream) {
  if (!c_rows) return moe::fail(MOE_ERR_ARG, "moe_grouped_gemm_rows: null row table");
  return moe::grouped_gemm_launch(a, w, nullptr, c_rows, offsets, experts, rows, K, N, w_layout, stride_w, activation,
                                  row_scale, bias, dtype, sm_margin, workspace, workspace_bytes, stream);
}

extern "C" int moe_set_gemm_mode(int mode) {
  const int before = moe::gemm_mode();
  if (mode >= 0) moe::g_gemm_mode.store(mode & MOE_GEMM_ALL, std::memory_order_relaxed);
  return before;
}
