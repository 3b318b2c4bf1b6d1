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
#include "sm100.cuh"

namespace moe {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

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

template <typename T>
__global__ void __launch_bounds__(kThreads)
sinkhorn_kernel(const SParams p) {
  extern __shared__ __align__(16) float s_f[];
  const int E = p.experts;
  const int R = p.rows_per_cta;
  float* s_k = s_f;                    // [R][E]   K = exp(s - rowmax)
  float* s_a = s_k + (size_t)R * E;    // [R]      row scale
  float* s_b = s_a + R;                // [E]      column scale
  float* s_part = s_b + E;             // [groups][E] partial column sums of this CTA
  __shared__ int s_flag;

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row0 = blockIdx.x * R;
  const int nrows = max(0, min(R, p.tokens - row0));
  const T* logits = static_cast<const T*>(p.logits);
  const float ct = (float)p.tokens / (float)max(E, 1);

  // ---- K = exp(s - rowmax), s = (logits / temperature) rounded to the logits dtype ----
  for (int r = warp; r < nrows; r += kWarps) {
    const T* src = logits + (size_t)(row0 + r) * E;
    float m = -INFINITY;
    for (int j = lane; j < E; j += 32) {
      float v = to_float(src[j]);
      if (p.temperature != 1.0f) v = to_float(from_float<T>(v / p.temperature));
      s_k[(size_t)r * E + j] = v;
      m = fmaxf(m, v);
    }
#pragma unroll
    for (int ofs = 16; ofs > 0; ofs >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, ofs));
    for (int j = lane; j < E; j += 32) s_k[(size_t)r * E + j] = expf(s_k[(size_t)r * E + j] - m);
    if (lane == 0) s_a[r] = 1.f;
  }
  for (int j = threadIdx.x; j < E; j += kThreads) s_b[j] = 1.f;
  __syncthreads();

  const int cw = min(E, kThreads);       // columns handled side by side
  const int groups = kThreads / cw;      // row groups working on the same column
  const int g = threadIdx.x / cw;
  const int jc = threadIdx.x % cw;

  bool ok = true;
  for (int it = 0; it <= p.iters && ok; ++it) {
    // ---- row step: a_i <- a_i / (a_i * sum_j K_ij b_j + eps) ----
    for (int r = warp; r < nrows; r += kWarps) {
      float s = 0.f;
      for (int j = lane; j < E; j += 32) s = fmaf(s_k[(size_t)r * E + j], s_b[j], s);
#pragma unroll
      for (int ofs = 16; ofs > 0; ofs >>= 1) s += __shfl_xor_sync(0xffffffffu, s, ofs);
      if (lane == 0) {
        const float a = s_a[r];
        s_a[r] = a / (a * s + p.eps);
      }
    }
    __syncthreads();
    if (it == p.iters) break;  // the last pass is the final row normalisation only

    // ---- column step: b_j <- b_j * (T/E) / (b_j * sum_i a_i K_ij + eps) ----
    if (g < groups) {
      for (int j = jc; j < E; j += cw) {
        float s = 0.f;
        for (int r = g; r < nrows; r += groups) s = fmaf(s_a[r], s_k[(size_t)r * E + j], s);
        s_part[(size_t)g * E + j] = s;
      }
    }
    __syncthreads();
    float* mine = p.scratch + ((size_t)(it & 1) * gridDim.x + blockIdx.x) * E;
    for (int j = threadIdx.x; j < E; j += kThreads) {
      float s = 0.f;
      for (int gg = 0; gg < groups; ++gg) s += s_part[(size_t)gg * E + j];
      mine[j] = s;
    }
    ok = grid_barrier(p.control, (int)gridDim.x, p.status, &s_flag);
    if (!ok) break;
    // every CTA adds the partials of all CTAs in the same fixed order: `groups` threads per column
    // each take a contiguous range of CTAs (loads in flight together), then the ranges are added
    // in order
    const float* all = p.scratch + (size_t)(it & 1) * gridDim.x * E;
    const int nblk = (int)gridDim.x;
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
    for (int j = threadIdx.x; j < E; j += kThreads) {
      float s = 0.f;
      for (int gg = 0; gg < groups; ++gg) s += s_part[(size_t)gg * E + j];
      const float b = s_b[j];
      s_b[j] = b / (b * s + p.eps) * ct;
    }
    __syncthreads();
  }
  if (!ok) return;

  // ---- top-k of q_ij = a_i K_ij b_j (lowest index wins ties), w = vals / (sum(vals) + eps) ----
  for (int r = warp; r < nrows; r += kWarps) {
    const float a = s_a[r];
    uint32_t taken = 0;  // bit m: column lane + 32*m already picked (experts <= 1024)
    float pv[8];
    int pi[8];
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      if (jj < p.top_k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int m = 0, j = lane; j < E; ++m, j += 32) {
          if ((taken >> m) & 1u) continue;
          const float q = a * s_k[(size_t)r * E + j] * s_b[j];
          if (better(q, j, bv, bi)) { bv = q; bi = j; }
        }
#pragma unroll
        for (int ofs = 16; ofs > 0; ofs >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, bv, ofs);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, ofs);
          if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (bi != 0x7fffffff && (bi & 31) == lane) taken |= 1u << (bi >> 5);
        pv[jj] = bv;
        pi[jj] = bi == 0x7fffffff ? 0 : bi;
      }
    }
    if (lane == 0) {
      float sum = 0.f;
#pragma unroll
      for (int jj = 0; jj < 8; ++jj)
        if (jj < p.top_k) sum += pv[jj];
      const float inv = 1.f / (sum + p.eps);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj)
        if (jj < p.top_k) {
          p.idx[(size_t)(row0 + r) * p.top_k + jj] = pi[jj];
          p.gates[(size_t)(row0 + r) * p.top_k + jj] = pv[jj] * inv;
        }
    }
  }
}

template <typename T>
int launch_sinkhorn(SParams& p, int grid, size_t smem, cudaStream_t s) {
  cudaError_t e = cudaFuncSetAttribute(sinkhorn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "moe_sinkhorn: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sinkhorn_kernel<T>, kThreads, smem);
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess || per_sm * sms < grid)
    return fail(MOE_ERR_UNSUPPORTED, "moe_sinkhorn: a grid of %d CTAs cannot be co-resident on this device", grid);
  void* args[] = {&p};
  e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(sinkhorn_kernel<T>), dim3(grid), dim3(kThreads), args, smem, s);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "sinkhorn_kernel: %s", cudaGetErrorString(e));
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

  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  int grid = (tokens + 127) / 128;  // about 128 rows per CTA: few partials to add after each barrier
  if (grid > sms) grid = sms;
  if (grid > kMaxGridBlocks) grid = kMaxGridBlocks;
  const int rows_per_cta = (tokens + grid - 1) / grid;
  grid = (tokens + rows_per_cta - 1) / rows_per_cta;
  const int cw = experts < kThreads ? experts : kThreads;
  const int groups = kThreads / cw;
  const size_t smem = ((size_t)rows_per_cta * experts + rows_per_cta + experts + (size_t)groups * experts) * sizeof(float);
  if (smem > 200 * 1024)
    return fail(MOE_ERR_UNSUPPORTED, "moe_sinkhorn: tokens*experts too large for the resident kernel (%d x %d)", tokens, experts);

  SParams p;
  p.logits = logits; p.tokens = tokens; p.experts = experts; p.top_k = top_k; p.iters = iters;
  p.eps = epsilon; p.temperature = temperature; p.rows_per_cta = rows_per_cta;
  p.idx = idx; p.gates = gates; p.scratch = ws.fscratch; p.control = ws.control; p.status = ws.status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (logits_dtype) {
    case MOE_F16: return launch_sinkhorn<__half>(p, grid, smem, s);
    case MOE_BF16: return launch_sinkhorn<__nv_bfloat16>(p, grid, smem, s);
    case MOE_F32: return launch_sinkhorn<float>(p, grid, smem, s);
    default: return fail(MOE_ERR_ARG, "moe_sinkhorn: logits must be fp16/bf16/fp32");
  }
}
