// Sinkhorn-balanced routing in one kernel.
//
// Replaces SinkhornRouter.forward (models/decoder_moe.py:92-123: 2 + 4*iters elementwise and
// reduction launches over a [T,E] fp32 matrix) and the unbuilt kernels of
// kernels/fused_sinkhorn.cu:56-209 (6 launches per iteration, global float atomics).
//
// The reference iterates on the matrix q itself:
//     q = exp(s - rowmax);  iters x { q /= rowsum(q) + eps ;  q = q / (colsum(q) + eps) * T/E };
//     q /= rowsum(q) + eps ;  top-k of q ;  w = vals / (sum(vals) + eps)
// Every step scales whole rows or whole columns, so q_ij = a_i * K_ij * b_j with K = exp(s - rowmax)
// fixed: only the vectors a (rows) and b (columns) change.  K stays in shared memory for the whole
// run (each CTA owns a block of rows), a row step is local to a CTA, and a column step needs one
// sum over all CTAs: per-CTA partial sums go to a double-buffered global scratch, a grid barrier
// follows, and every CTA adds the partials in the same fixed order (bit-identical b everywhere,
// run-to-run deterministic).  One grid barrier per iteration; the grid is launched cooperatively so
// that all CTAs are co-resident, and the barrier spin is bounded in time.
#include <cstdlib>

#include "sm100.cuh"

namespace moe {
namespace {

constexpr int kThreads = 256;

struct SParams {
  const void* logits;
  int tokens, experts, top_k, iters;
  float eps, temperature;
  int rows_per_cta;
  int32_t* idx;
  float* gates;
  float* scratch;    // [2][gridDim.x][experts]
  int32_t* control;  // [0] arrival count, [1] generation
  int32_t* status;
};

// CLUSTER = false: any number of co-resident CTAs (cooperative launch), column partials through a
// global scratch and a grid barrier.  CLUSTER = true: the whole matrix fits the shared memory of
// ONE thread-block cluster (16 or 8 CTAs x 1024 threads); column partials are pushed into every CTA's
// shared memory (st.shared::cluster) and a hardware cluster barrier replaces the grid barrier, which
// takes the global-memory round trips out of every iteration.
// One thread per row: scan q_ij = a_i K_ij b_j over the columns keeping the best KMAX entries under
// "larger value, then lower index" (the first slot a candidate beats takes it, the rest shifts down).
template <int KMAX>
__device__ __forceinline__ void topk_rows(const SParams& p, const float* s_k, const float* s_a, const float* s_b,
                                          int SK, int row0, int nrows) {
  for (int r = threadIdx.x; r < nrows; r += (int)blockDim.x) {
    const float* kr = s_k + r * SK;
    const float a = s_a[r];
    float tv[KMAX];
    int ti[KMAX];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) { tv[j] = -INFINITY; ti[j] = 0x7fffffff; }
    for (int c = 0; c < p.experts; ++c) {
      float cv = a * kr[c] * s_b[c];
      int ci = c;
      bool placed = false;
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        if (placed || better(cv, ci, tv[j], ti[j])) {
          const float fv = tv[j];
          const int fi = ti[j];
          tv[j] = cv; ti[j] = ci;
          cv = fv; ci = fi;
          placed = true;
        }
      }
    }
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < KMAX; ++j)
      if (j < p.top_k) sum += tv[j];
    const float inv = 1.f / (sum + p.eps);
#pragma unroll
    for (int j = 0; j < KMAX; ++j)
      if (j < p.top_k) {
        p.idx[(size_t)(row0 + r) * p.top_k + j] = ti[j] == 0x7fffffff ? 0 : ti[j];
        p.gates[(size_t)(row0 + r) * p.top_k + j] = tv[j] * inv;
      }
  }
}

template <typename T, bool CLUSTER>
__global__ void __launch_bounds__(CLUSTER ? 1024 : kThreads)
sinkhorn_kernel(const SParams p) {
  extern __shared__ __align__(16) float s_f[];
  const int E = p.experts;
  const int R = p.rows_per_cta;
  const int nthreads = (int)blockDim.x;
  const int nblk = (int)gridDim.x;
  const int cw = min(E, nthreads);       // columns handled side by side
  const int groups = nthreads / cw;      // row groups working on the same column
  const int SK = E + 1;                  // row stride of K in shared memory
  float* s_k = s_f;                      // [R][SK]  K = exp(s - rowmax)
  float* s_a = s_k + (size_t)R * SK;     // [R]      row scale
  float* s_b = s_a + R;                  // [E]      column scale
  float* s_part = s_b + E;               // [groups][E] partial column sums of this CTA
  float* s_all = s_part + (size_t)groups * E;  // [2][nblk][E] partials of all CTAs (CLUSTER only)
  __shared__ int s_flag;

  const int row0 = blockIdx.x * R;
  const int nrows = max(0, min(R, p.tokens - row0));
  const T* logits = static_cast<const T*>(p.logits);
  const float ct = (float)p.tokens / (float)max(E, 1);
  // Remote shared-memory stores below need every CTA of the cluster to be running: arrive now, wait
  // just before the first store (by then the others have long started, so the wait costs nothing).
  if constexpr (CLUSTER) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

  // ---- K = exp(s - rowmax), s = (logits / temperature) rounded to the logits dtype ----
  // coalesced load of the CTA's rows, then one thread per row (rows are SK = E+1 floats apart, so
  // threads of a warp working on consecutive rows hit different banks)
  for (int i = threadIdx.x; i < nrows * E; i += nthreads) {
    const int r = i / E, j = i - r * E;
    float v = to_float(logits[(size_t)row0 * E + i]);
    if (p.temperature != 1.0f) v = to_float(from_float<T>(v / p.temperature));
    s_k[r * SK + j] = v;
  }
  __syncthreads();
  for (int r = threadIdx.x; r < nrows; r += nthreads) {
    float* kr = s_k + r * SK;
    float m = -INFINITY;
    for (int j = 0; j < E; ++j) m = fmaxf(m, kr[j]);
    for (int j = 0; j < E; ++j) kr[j] = expf(kr[j] - m);
    s_a[r] = 1.f;
  }
  for (int j = threadIdx.x; j < E; j += nthreads) s_b[j] = 1.f;
  __syncthreads();

  const int g = threadIdx.x / cw;
  const int jc = threadIdx.x % cw;

  bool ok = true;
  for (int it = 0; it <= p.iters && ok; ++it) {
    // ---- row step: a_i <- a_i / (a_i * sum_j K_ij b_j + eps), one thread per row ----
    for (int r = threadIdx.x; r < nrows; r += nthreads) {
      const float* kr = s_k + r * SK;
      float s0 = 0.f, s1 = 0.f;
      int j = 0;
      for (; j + 1 < E; j += 2) {
        s0 = fmaf(kr[j], s_b[j], s0);
        s1 = fmaf(kr[j + 1], s_b[j + 1], s1);
      }
      if (j < E) s0 = fmaf(kr[j], s_b[j], s0);
      const float a = s_a[r];
      s_a[r] = a / (a * (s0 + s1) + p.eps);
    }
    __syncthreads();
    if (it == p.iters) break;  // the last pass is the final row normalisation only

    // ---- column step: b_j <- b_j * (T/E) / (b_j * sum_i a_i K_ij + eps) ----
    if (g < groups) {
      for (int j = jc; j < E; j += cw) {
        float s = 0.f;
        for (int r = g; r < nrows; r += groups) s = fmaf(s_a[r], s_k[r * SK + j], s);
        s_part[(size_t)g * E + j] = s;
      }
    }
    __syncthreads();
    if constexpr (CLUSTER) {
      // this CTA's column sums go into slot [it & 1][my rank] of every CTA of the cluster
      const uint32_t me = sm100::cluster_ctarank();
      if (it == 0) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
      float* slot = s_all + ((size_t)(it & 1) * nblk + me) * E;
      for (int j = threadIdx.x; j < E; j += nthreads) {
        float s = 0.f;
        for (int gg = 0; gg < groups; ++gg) s += s_part[(size_t)gg * E + j];
        const uint32_t local = sm100::smem_u32(slot + j);
        for (int c = 0; c < nblk; ++c) sm100::st_cluster_f32(sm100::map_to_cta(local, (uint32_t)c), s);
      }
      sm100::cluster_sync_all();
      const float* all = s_all + (size_t)(it & 1) * nblk * E;
      for (int j = threadIdx.x; j < E; j += nthreads) {
        float s = 0.f;
        for (int c = 0; c < nblk; ++c) s += all[(size_t)c * E + j];  // same order in every CTA
        const float b = s_b[j];
        s_b[j] = b / (b * s + p.eps) * ct;
      }
      __syncthreads();
    } else {
      float* mine = p.scratch + ((size_t)(it & 1) * nblk + blockIdx.x) * E;
      for (int j = threadIdx.x; j < E; j += nthreads) {
        float s = 0.f;
        for (int gg = 0; gg < groups; ++gg) s += s_part[(size_t)gg * E + j];
        mine[j] = s;
      }
      ok = grid_barrier(p.control, nblk, p.status, &s_flag);
      if (!ok) break;
      // every CTA adds the partials of all CTAs in the same fixed order: `groups` threads per column
      // each take a contiguous range of CTAs (loads in flight together), then the ranges are added
      // in order
      const float* all = p.scratch + (size_t)(it & 1) * nblk * E;
      const int per = (nblk + groups - 1) / groups;
      if (g < groups) {
        for (int j = jc; j < E; j += cw) {
          const int c0 = g * per, c1 = min(nblk, c0 + per);
          float s = 0.f;
          int c = c0;
          for (; c + 7 < c1; c += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldcg(all + (size_t)(c + u) * E + j);
#pragma unroll
            for (int u = 0; u < 8; ++u) s += v[u];
          }
          for (; c < c1; ++c) s += __ldcg(all + (size_t)c * E + j);
          s_part[(size_t)g * E + j] = s;
        }
      }
      __syncthreads();
      for (int j = threadIdx.x; j < E; j += nthreads) {
        float s = 0.f;
        for (int gg = 0; gg < groups; ++gg) s += s_part[(size_t)gg * E + j];
        const float b = s_b[j];
        s_b[j] = b / (b * s + p.eps) * ct;
      }
      __syncthreads();
    }
  }
  if (!ok) return;

  // ---- top-k of q_ij = a_i K_ij b_j (lowest index wins ties), w = vals / (sum(vals) + eps) ----
  if (p.top_k <= 1) topk_rows<1>(p, s_k, s_a, s_b, SK, row0, nrows);
  else if (p.top_k <= 2) topk_rows<2>(p, s_k, s_a, s_b, SK, row0, nrows);
  else if (p.top_k <= 4) topk_rows<4>(p, s_k, s_a, s_b, SK, row0, nrows);
  else topk_rows<8>(p, s_k, s_a, s_b, SK, row0, nrows);
}

constexpr int kClusterCtas = 8;        // portable cluster size
constexpr int kClusterCtasWide = 16;   // needs cudaFuncAttributeNonPortableClusterSizeAllowed
constexpr int kClusterThreads = 1024;

// Shared memory (bytes) of a launch with `rows` rows per CTA.
size_t sinkhorn_smem(int rows, int experts, int threads, int nblk, bool cluster) {
  const int cw = experts < threads ? experts : threads;
  const int groups = threads / cw;
  size_t floats = (size_t)rows * (experts + 1) + rows + experts + (size_t)groups * experts;
  if (cluster) floats += (size_t)2 * nblk * experts;
  return floats * sizeof(float);
}

// Launch as ONE cluster of `ctas` CTAs.  Returns MOE_ERR_UNSUPPORTED (nothing launched, no error text
// kept) when `probe` is set and the device cannot place such a cluster, so that the caller can fall
// back to the portable size.
template <typename T>
int launch_sinkhorn_cluster(SParams& p, int ctas, size_t smem, cudaStream_t s, bool probe) {
  cudaError_t e = cudaFuncSetAttribute(sinkhorn_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "moe_sinkhorn: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  if (ctas > kClusterCtas) {
    e = cudaFuncSetAttribute(sinkhorn_kernel<T, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return MOE_ERR_UNSUPPORTED;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas, 1, 1);
  cfg.blockDim = dim3(kClusterThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ctas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (probe) {
    int clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&clusters, sinkhorn_kernel<T, true>, &cfg);
    if (e != cudaSuccess || clusters < 1) {
      (void)cudaGetLastError();
      return MOE_ERR_UNSUPPORTED;
    }
  }
  e = cudaLaunchKernelEx(&cfg, sinkhorn_kernel<T, true>, p);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "sinkhorn_kernel (cluster): %s", cudaGetErrorString(e));
  note_launch();
  return MOE_OK;
}

template <typename T>
int launch_sinkhorn(SParams& p, int grid, size_t smem, cudaStream_t s) {
  cudaError_t e = cudaFuncSetAttribute(sinkhorn_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "moe_sinkhorn: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sinkhorn_kernel<T, false>, kThreads, smem);
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess || per_sm * sms < grid)
    return fail(MOE_ERR_UNSUPPORTED, "moe_sinkhorn: a grid of %d CTAs cannot be co-resident on this device", grid);
  void* args[] = {&p};
  e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(sinkhorn_kernel<T, false>), dim3(grid), dim3(kThreads), args, smem, s);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "sinkhorn_kernel: %s", cudaGetErrorString(e));
  note_launch();
  return MOE_OK;
}

}  // namespace
}  // namespace moe

extern "C" int moe_sinkhorn(const void* logits, int logits_dtype, int tokens, int experts, int top_k, int iters,
                            float epsilon, float temperature, int32_t* idx, float* gates, void* workspace,
                            size_t workspace_bytes, void* stream) {
  using namespace moe;
  if (tokens < 0 || experts <= 0) return fail(MOE_ERR_ARG, "moe_sinkhorn: bad shape");
  if (iters <= 0) return fail(MOE_ERR_ARG, "SinkhornRouter.iters must be > 0");
  if (!(epsilon > 0.f)) return fail(MOE_ERR_ARG, "SinkhornRouter.epsilon must be > 0");
  if (!(temperature > 0.f)) return fail(MOE_ERR_ARG, "SinkhornRouter.temperature must be > 0");
  if (top_k <= 0) return fail(MOE_ERR_ARG, "top_k must be > 0");
  if (top_k > experts) return fail(MOE_ERR_ARG, "top_k must be <= n_experts");
  if (top_k > 8) return fail(MOE_ERR_UNSUPPORTED, "moe_sinkhorn: top_k must be <= 8, got %d", top_k);
  if (experts > 1024) return fail(MOE_ERR_UNSUPPORTED, "moe_sinkhorn: experts must be <= 1024");
  if (tokens == 0) return MOE_OK;
  if (!logits || !idx || !gates) return fail(MOE_ERR_ARG, "moe_sinkhorn: null pointer");
  if (!workspace || workspace_bytes < workspace_bytes_for(tokens, experts, top_k))
    return fail(MOE_ERR_WORKSPACE, "moe_sinkhorn: workspace too small (need %zu bytes)",
                workspace_bytes_for(tokens, experts, top_k));
  Workspace ws = carve(workspace, tokens, experts);

  SParams p;
  p.logits = logits; p.tokens = tokens; p.experts = experts; p.top_k = top_k; p.iters = iters;
  p.eps = epsilon; p.temperature = temperature;
  p.idx = idx; p.gates = gates; p.scratch = ws.fscratch; p.control = ws.control; p.status = ws.status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  // One cluster when the matrix fits its shared memory (T=4096, E=64 does): no global round trips
  // inside the iterations.  16 CTAs where the device can place such a cluster (half the rows per CTA:
  // every pass of the iteration is shorter), else the portable 8.  MOE_B200_SINKHORN_CLUSTER=8 in the
  // environment keeps the portable size.
  static const int wide_ok = [] { const char* v = getenv("MOE_B200_SINKHORN_CLUSTER"); return !(v && atoi(v) == 8); }();
  for (int ctas : {kClusterCtasWide, kClusterCtas}) {
    if (ctas == kClusterCtasWide && (!wide_ok || tokens < 1024)) continue;
    const int rows = (tokens + ctas - 1) / ctas;
    const size_t smem = sinkhorn_smem(rows, experts, kClusterThreads, ctas, true);
    if (smem <= 200 * 1024 && tokens >= 256) {
      p.rows_per_cta = rows;
      const bool probe = ctas == kClusterCtasWide;
      int rc;
      switch (logits_dtype) {
        case MOE_F16: rc = launch_sinkhorn_cluster<__half>(p, ctas, smem, s, probe); break;
        case MOE_BF16: rc = launch_sinkhorn_cluster<__nv_bfloat16>(p, ctas, smem, s, probe); break;
        case MOE_F32: rc = launch_sinkhorn_cluster<float>(p, ctas, smem, s, probe); break;
        default: return fail(MOE_ERR_ARG, "moe_sinkhorn: logits must be fp16/bf16/fp32");
      }
      if (!(probe && rc == MOE_ERR_UNSUPPORTED)) return rc;
    }
  }

  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  int grid = (tokens + 127) / 128;  // about 128 rows per CTA: few partials to add after each barrier
  if (grid > sms) grid = sms;
  if (grid > kMaxGridBlocks) grid = kMaxGridBlocks;
  const int rows_per_cta = (tokens + grid - 1) / grid;
  grid = (tokens + rows_per_cta - 1) / rows_per_cta;
  const size_t smem = sinkhorn_smem(rows_per_cta, experts, kThreads, grid, false);
  if (smem > 200 * 1024)
    return fail(MOE_ERR_UNSUPPORTED, "moe_sinkhorn: tokens*experts too large for the resident kernel (%d x %d)", tokens, experts);
  p.rows_per_cta = rows_per_cta;
  switch (logits_dtype) {
    case MOE_F16: return launch_sinkhorn<__half>(p, grid, smem, s);
    case MOE_BF16: return launch_sinkhorn<__nv_bfloat16>(p, grid, smem, s);
    case MOE_F32: return launch_sinkhorn<float>(p, grid, smem, s);
    default: return fail(MOE_ERR_ARG, "moe_sinkhorn: logits must be fp16/bf16/fp32");
  }
}
