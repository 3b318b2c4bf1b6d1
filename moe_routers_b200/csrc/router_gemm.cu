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
#include "sm100.cuh"

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
  int kblocks, splitk, stages, tmem_cols, num_tiles;
  int32_t* idx;
  float* gates;
  float* logits_out;
  int32_t* tile_hist;
  int32_t* status;
};

// A logit that has been rounded to fp16 and its column pack into one 32-bit key whose unsigned
// order is "larger value first, then lower column": high half = the fp16 bits mapped to an
// order-preserving unsigned code (-0 folded onto +0), low half = 0xFFFF - column.
__device__ __forceinline__ uint32_t make_key(__half h, int col) {
  uint32_t hb = __half_as_ushort(h);
  if (hb == 0x8000u) hb = 0u;
  const uint32_t code = (hb & 0x8000u) ? (~hb & 0xFFFFu) : (hb | 0x8000u);
  return (code << 16) | (0xFFFFu - (uint32_t)col);
}
__device__ __forceinline__ float key_value(uint32_t key) {
  const uint32_t code = key >> 16;
  const uint32_t hb = (code & 0x8000u) ? (code & 0x7FFFu) : (~code & 0xFFFFu);
  return __half2float(__ushort_as_half((unsigned short)hb));
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
template <int KMAX, int S>
__device__ __forceinline__ void scan_columns(const float* __restrict__ prow, int E, int EP, int wq,
                                             int skew_experts, float skew_bias, float* __restrict__ logits_row,
                                             uint32_t (&keys)[KMAX]) {
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
      __half h = __float2half_rn(acc[u]);
      if (c < skew_experts) h = __float2half_rn(__half2float(h) + skew_bias);
      if (logits_row != nullptr) logits_row[c] = __half2float(h);
      key_insert<KMAX>(keys, make_key(h, c));
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

template <int KMAX>
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

  const int E = p.experts;
  const int b_bytes = E * kBlockK * 2;
  uint8_t* sA = smem;
  uint8_t* sB = sA + (size_t)p.stages * kABytes;
  const int EP = E + 4;  // padded row of a partial tile: conflict-free 128-bit accesses, thread = row
  float* s_partial = reinterpret_cast<float*>(sB + (size_t)p.stages * b_bytes);  // [4][32][EP]
  int32_t* s_hist = reinterpret_cast<int32_t*>(s_partial + 4 * 32 * EP);        // [4][E]
  uint32_t* s_cand = reinterpret_cast<uint32_t*>(s_hist + 4 * E);               // [4][4][KMAX][32]
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_cand + 16 * KMAX * 32);       // full[], empty[], tmem_full
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_bar + 2 * kMaxStages + 1);

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
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(kBlockM, E, 0, 0, 0);
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
    // -------------- epilogue phase B: reduce, round, bias, top-k, gates, histogram --------------
    // Warp wq scans a quarter of the expert columns for all 32 rows of a block (thread = row),
    // keeps its local top-k as sortable 32-bit keys, and one warp merges the four lists of a row.
    const int wq = warp - 2;
    const int nslots = 4 / S;
    for (int s = 0; s < nslots; ++s) {
      const int rb = s * S + krank;
      const int row = m_tile * kBlockM + rb * 32 + lane;
      float* lo = (MOE_LOGITS_OUT != nullptr && row < p.tokens) ? MOE_LOGITS_OUT + (size_t)row * E : nullptr;
      const float* prow = s_partial + (size_t)((s * S) * 32 + lane) * EP;
      uint32_t keys[KMAX];
      if (S == 4) scan_columns<KMAX, 4>(prow, E, EP, wq, p.skew_experts, p.skew_bias, lo, keys);
      else if (S == 2) scan_columns<KMAX, 2>(prow, E, EP, wq, p.skew_experts, p.skew_bias, lo, keys);
      else scan_columns<KMAX, 1>(prow, E, EP, wq, p.skew_experts, p.skew_bias, lo, keys);
#pragma unroll
      for (int j = 0; j < KMAX; ++j) s_cand[((s * 4 + wq) * KMAX + j) * 32 + lane] = keys[j];
    }
    MOE_TRACE(8, threadIdx.x == 64);
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
    if (wq < nslots) {
      const int s = wq;
      const int rb = s * S + krank;
      const int row = m_tile * kBlockM + rb * 32 + lane;
      uint32_t keys[KMAX];
#pragma unroll
      for (int j = 0; j < KMAX; ++j) keys[j] = s_cand[((s * 4 + 0) * KMAX + j) * 32 + lane];
#pragma unroll
      for (int w4 = 1; w4 < 4; ++w4)
#pragma unroll
        for (int j = 0; j < KMAX; ++j) key_insert<KMAX>(keys, s_cand[((s * 4 + w4) * KMAX + j) * 32 + lane]);
      if (row < p.tokens) {
        float e[KMAX];
        float sum = 0.f;
        const float v0 = key_value(keys[0]);
#pragma unroll
        for (int j = 0; j < KMAX; ++j)
          if (j < p.top_k) { e[j] = expf(key_value(keys[j]) - v0); sum += e[j]; }
        const float inv = 1.f / fmaxf(sum, 1e-9f);
#pragma unroll
        for (int j = 0; j < KMAX; ++j)
          if (j < p.top_k) {
            const int pick = keys[j] == 0u ? 0 : key_column(keys[j]);
            p.idx[(size_t)row * p.top_k + j] = pick;
            p.gates[(size_t)row * p.top_k + j] = e[j] * inv;
            atomicAdd(&s_hist[s * E + pick], 1);
          }
      }
      __syncwarp();
      const int tile = m_tile * (kBlockM / kTileTokens) + rb;
      if (p.tile_hist != nullptr && tile < p.num_tiles)
        for (int e2 = lane; e2 < E; e2 += 32) p.tile_hist[(size_t)tile * E + e2] = s_hist[s * E + e2];
    }
  }

  MOE_TRACE(9, threadIdx.x == 64);
  MOE_TRACE_G(14, threadIdx.x == 64);
  tc_fence_before();
  __syncthreads();
  MOE_TRACE(10, threadIdx.x == 0);
  MOE_TRACE_G(13, threadIdx.x == 0);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

int launch_router(const void* x, const void* w, int tokens, int d, int experts, int top_k, int skew_experts,
                  float skew_bias, int32_t* idx, float* gates, float* logits_out, const Workspace& ws,
                  cudaStream_t stream) {
  CUtensorMap tmap_x, tmap_w;
  int rc = encode_tmap_2d(&tmap_x, x, (uint64_t)tokens, (uint64_t)d, (uint64_t)d * 2, kBlockK, kBlockM);
  if (rc != MOE_OK) return rc;
  rc = encode_tmap_2d(&tmap_w, w, (uint64_t)experts, (uint64_t)d, (uint64_t)d * 2, kBlockK, (uint32_t)experts);
  if (rc != MOE_OK) return rc;

  RouterParams p;
  p.tokens = tokens; p.d = d; p.experts = experts; p.top_k = top_k;
  p.skew_experts = skew_experts < 0 ? 0 : (skew_experts > experts ? experts : skew_experts);
  p.skew_bias = skew_bias;
  if (skew_bias == 0.0f) p.skew_experts = 0;
  p.kblocks = (d + kBlockK - 1) / kBlockK;
  p.splitk = p.kblocks >= 16 ? 4 : (p.kblocks >= 4 ? 2 : 1);
  int cols = 32;
  while (cols < experts) cols *= 2;
  p.tmem_cols = cols;
  p.num_tiles = ws.num_tiles;
  const int stage_bytes = kABytes + experts * kBlockK * 2;
  const int kmax = top_k <= 1 ? 1 : (top_k <= 2 ? 2 : (top_k <= 4 ? 4 : 8));
  const int fixed = 4 * 32 * (experts + 4) * 4 + 4 * experts * 4 + 16 * kmax * 32 * 4 + (2 * kMaxStages + 1) * 8 + 16;
  int stages = (kSmemLimit - 1024 - fixed) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  const int max_nkb = (p.kblocks + p.splitk - 1) / p.splitk;
  if (stages > max_nkb) stages = max_nkb;
  if (stages < 1) return fail(MOE_ERR_UNSUPPORTED, "router GEMM: shared memory budget exceeded for experts=%d", experts);
  p.stages = stages;
  p.idx = idx; p.gates = gates; p.logits_out = logits_out;
  p.tile_hist = ws.tile_hist; p.status = ws.status;
  const size_t smem = 1024 + (size_t)stages * stage_bytes + fixed;

  auto kernel = kmax == 1 ? router_gemm_select_kernel<1>
                : kmax == 2 ? router_gemm_select_kernel<2>
                : kmax == 4 ? router_gemm_select_kernel<4>
                            : router_gemm_select_kernel<8>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "router GEMM: cudaFuncSetAttribute: %s", cudaGetErrorString(e));

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((tokens + kBlockM - 1) / kBlockM, p.splitk, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = p.splitk;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kernel, tmap_x, tmap_w, p);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "router_gemm_select_kernel: %s", cudaGetErrorString(e));
  return MOE_OK;
}

int check_router_args(const char* who, const void* x, const void* w, int tokens, int d, int experts, int top_k,
                      const void* idx, const void* gates, const void* workspace, size_t workspace_bytes) {
  if (tokens < 0 || d <= 0 || experts <= 0) return fail(MOE_ERR_ARG, "%s: bad shape", who);
  if (top_k < 1 || top_k > 8) return fail(MOE_ERR_UNSUPPORTED, "%s: top_k must be in [1,8], got %d", who, top_k);
  if (top_k > experts) return fail(MOE_ERR_ARG, "%s: top_k must be <= n_experts", who);
  if (experts % 16 != 0 || experts < 16 || experts > 256)
    return fail(MOE_ERR_UNSUPPORTED, "%s: experts must be a multiple of 16 in [16,256], got %d", who, experts);
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
                        int32_t* route_row, const Workspace& ws, cudaStream_t s);

}  // namespace moe

extern "C" int moe_router_gemm_select(const void* x, const void* w_router, int tokens, int d, int experts,
                                      int top_k, int skew_experts, float skew_bias, int32_t* idx, float* gates,
                                      float* logits_out, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace moe;
  int rc = check_router_args("moe_router_gemm_select", x, w_router, tokens, d, experts, top_k, idx, gates,
                             workspace, workspace_bytes);
  if (rc != MOE_OK || tokens == 0) return rc;
  Workspace ws = carve(workspace, tokens, experts);
  return launch_router(x, w_router, tokens, d, experts, top_k, skew_experts, skew_bias, idx, gates, logits_out, ws,
                       static_cast<cudaStream_t>(stream));
}

extern "C" int moe_route_fused(const void* x, const void* w_router, int tokens, int d, int experts, int top_k,
                               int skew_experts, float skew_bias, int32_t* idx, float* gates, int32_t* counts,
                               int32_t* offsets, void* packed, int32_t* row_route, int32_t* route_row,
                               float* logits_out, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace moe;
  int rc = check_router_args("moe_route_fused", x, w_router, tokens, d, experts, top_k, idx, gates, workspace,
                             workspace_bytes);
  if (rc != MOE_OK) return rc;
  if (!counts || !offsets || (tokens > 0 && !row_route)) return fail(MOE_ERR_ARG, "moe_route_fused: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Workspace ws = carve(workspace, tokens, experts);
  if (tokens > 0) {
    rc = launch_router(x, w_router, tokens, d, experts, top_k, skew_experts, skew_bias, idx, gates, logits_out, ws, s);
    if (rc != MOE_OK) return rc;
  }
  return launch_scan_scatter(x, 2, idx, tokens, d, experts, top_k, counts, offsets, packed, row_route, route_row,
                             ws, s);
}
