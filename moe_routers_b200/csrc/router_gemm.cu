// Router logit GEMM with a fused select epilogue (tcgen05 / TMEM / TMA).
//
// Replaces `logits = x @ w.t(); logits[:, :n] += bias` (bench_router.py:512-516,
// bench_2gpu_pcie.py:426-428, models/decoder_moe.py:201) followed by the
// top-k selection (kernels/fused_select.cu:47-113, models/decoder_moe.py:58-62)
// and the per-expert count (kernels/fused_select.cu:116-143).  The logits stay
// on chip: TMEM accumulators -> distributed shared memory -> registers.
//
// Work split: one cluster of SPLITK CTAs per block of 128 tokens; CTA r of the cluster multiplies
// its slice of the K dimension (d / SPLITK) on the tensor core (UMMA 128 x E x 16, fp32 accumulators
// in TMEM).  The kernel is bound by the stream of x from HBM, and two per-thread costs would keep it
// from reaching that bound if one thread did each job:
//   * the bulk tensor copies of ONE thread are served one after another (about 0.35 us each on
//     B200 whatever their size): four producer warps issue, each owning every fourth pipeline stage;
//   * issuing one short MMA (E = 64 columns: 32 tensor cycles of work) costs its thread ~85 cycles
//     and a commit ~220: two warps issue, each owning every second stage and accumulating into its
//     own TMEM accumulator; the epilogue adds the two.
// The four row quarters of the partial accumulator (TMEM lane quarter q) go to their owner CTA
// (q % SPLITK) through distributed shared memory: each epilogue warp transposes its quarter through
// local shared memory so that every remote store instruction writes two contiguous 256-byte row
// pieces, and tells the owner by remote mbarrier arrivals (no cluster-wide barrier on the critical
// path).  The owner adds the SPLITK partials in a fixed order, rounds to the 16-bit logit type (the
// dtype the reference holds its logits in), adds the skew bias, and keeps the top-k under the
// ordering "larger value, then lower index" (eight warps, several threads per row).  Every owner
// holds whole 32-token groups and writes their per-expert histograms, which the pack consumes.
//
// Warp roles (320 threads): warps 0..3 = TMA producers (lane 0), then select; warps 4..5 = MMA
// issuers (warp 4 owns the TMEM allocation); warps 6..9 = epilogue (warp w reads TMEM lanes
// 32*(w%4)...), then select.
#include <cstdlib>

#include "sm100.cuh"

namespace moe {
namespace {

using namespace sm100;

constexpr int kBlockTokens = 128;  // tokens per cluster = UMMA M
constexpr int kBlockK = 64;        // 64 16-bit elements = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kProducers = 4;      // warps whose lane 0 issues TMA copies
constexpr int kMmaWarps = 2;       // warps whose lane 0 issues MMAs (one TMEM accumulator each)
constexpr int kEpiWarps = 4;       // one per TMEM lane quarter
constexpr int kThreads = 32 * (kProducers + kMmaWarps + kEpiWarps);
constexpr int kEpiThreads = 32 * kEpiWarps;
constexpr int kSelThreads = 32 * (kProducers + kEpiWarps);  // threads that run the select
constexpr int kMaxStages = 12;
constexpr int kChunk = 64;         // columns moved per transpose step of the partial exchange
constexpr int kSmemLimit = 227 * 1024;

struct RouterParams {
  int tokens, d, experts, top_k;
  int skew_experts;
  float skew_bias;
  int bf16;  // 0: fp16 tokens / weights / logits, 1: bf16
  int epad;  // experts rounded up to the UMMA N granule (16); padded logit columns are never selected
  int kblocks, splitk, stages, tmem_cols, num_tiles;
  int stage_in_ring;  // the exchange's transpose tiles reuse the pipeline stages
  int bulk_push;      // the exchange moves a warp's 32 x (E + 4) quarter with one bulk copy (E == 64 only)
  int prefetch_x;     // request this CTA's token boxes into L2 before the dependency wait
  int nacc;  // MMA-issuing warps = TMEM accumulators (1 or 2; at most the stage count)
  // bit (2 * k-slice rank + m): issuing warp m gets at least one k-block of that k slice, i.e.
  // accumulator m holds a partial sum (the other was never written)
  uint32_t acc_mask;
  int32_t* idx;
  float* gates;
  float* logits_out;
  int32_t* tile_hist;
  int32_t* status;
};

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

// ---- cluster-scope mbarrier operations (the exchange of partial tiles) -----------------------------
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int32_t* status, int code) {
#pragma unroll 1
  for (int i = 0; i < 2048; ++i)
    if (mbar_try_wait_cluster(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  const unsigned long long limit = wait_limit_ns(status);
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait_cluster(bar, parity)) return true;
    if (globaltimer_ns() - t0 > limit) {
      record_error(status, kErrMbarTimeout | code);
      return false;
    }
  }
}
// Shared memory of this CTA -> shared memory of a CTA of the cluster, completion counted in bytes on an
// mbarrier of the destination CTA (both given as shared::cluster addresses); 16-byte granularity.
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes,
                                                     uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   dst_cluster),
               "r"(src_cta), "r"(bytes), "r"(bar_cluster)
               : "memory");
}
// Start-of-kernel arrival: the barrier initialisations were released to the cluster by
// fence.mbarrier_init, nothing else has to be visible to the other CTAs yet.
__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// 32 lanes x 16 consecutive fp32 columns without the trailing wait (several loads in flight).
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void st_cluster_v4u(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

// Select for the rows this CTA owns: kSelThreads threads split every owned row between
// TPR = kSelThreads / rows threads (consecutive lanes of a warp), each summing the S split-K partials
// of its 4-column chunks in a fixed order, rounding, biasing and keeping the best KMAX keys; the TPR
// lists of a row are merged with warp shuffles and lane 0 of the row's group writes the result.
// Partials of quarter slot s, source CTA c, row r: s_part[((s * S + c) * 32 + r) * EP + column].
template <int KMAX, int S>
__device__ __forceinline__ void select_rows(const RouterParams& p, const float* __restrict__ s_part,
                                            int32_t* __restrict__ s_hist, int st, int block, int krank) {
  constexpr int ROWS = kBlockTokens / S;   // rows this CTA owns
  constexpr int TPR = kSelThreads / ROWS;  // threads per row (2, 4 or 8)
  const int E = p.epad, EL = p.experts, EP = p.epad + 4;
  const bool bf16 = p.bf16 != 0;
  const int ro = st / TPR, cg = st % TPR;
  const int slot = ro >> 5, r = ro & 31;
  const int q = slot * S + krank;  // TMEM lane quarter == 32-token group of the block
  const int row = block * kBlockTokens + q * 32 + r;
  const float* prow = s_part + (size_t)((slot * S) * 32 + r) * EP;
  float* lrow = (p.logits_out != nullptr && row < p.tokens) ? p.logits_out + (size_t)row * EL : nullptr;

  uint32_t keys[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j) keys[j] = 0u;
  for (int ch = cg; ch < E / 4; ch += TPR) {
    const int c0 = ch * 4;
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
      const uint32_t h1 = round16(widen16(h0, bf16) + p.skew_bias, bf16);
      const uint32_t hv = c < p.skew_experts ? h1 : h0;
      if (lrow != nullptr && c < EL) lrow[c] = widen16(hv, bf16);
      key_insert<KMAX>(keys, c < EL ? make_key(hv, c) : 0u);  // padding columns can never be picked
    }
  }
#pragma unroll
  for (int ofs = 1; ofs < TPR; ofs <<= 1) {
    uint32_t other[KMAX];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) other[j] = __shfl_xor_sync(0xffffffffu, keys[j], ofs);
#pragma unroll
    for (int j = 0; j < KMAX; ++j) key_insert<KMAX>(keys, other[j]);
  }
  if (cg == 0 && row < p.tokens) {
    float e[KMAX];
    float sum = 0.f;
    const float v0 = key_value(keys[0], bf16);
#pragma unroll
    for (int j = 0; j < KMAX; ++j)
      if (j < p.top_k) { e[j] = expf(key_value(keys[j], bf16) - v0); sum += e[j]; }
    const float inv = 1.f / fmaxf(sum, 1e-9f);
#pragma unroll
    for (int j = 0; j < KMAX; ++j)
      if (j < p.top_k) {
        const int pick = keys[j] == 0u ? 0 : min(key_column(keys[j]), EL - 1);  // never index past the experts
        p.idx[(size_t)row * p.top_k + j] = pick;
        p.gates[(size_t)row * p.top_k + j] = e[j] * inv;
        atomicAdd(&s_hist[slot * E + pick], 1);
      }
  }
}

// After the exchange: wait until all partials of the rows this CTA owns have arrived, select, and
// write the histogram of every 32-token group the CTA owns.  Run by the kSelThreads threads of the
// producer and epilogue warps (st = index among them).
template <int KMAX>
__device__ __forceinline__ void select_phase(const RouterParams& p, const float* s_partial, int32_t* s_hist,
                                             uint32_t part_full, int st, int block, int krank) {
  const int S = p.splitk;
  const bool arrived = mbar_wait_cluster(part_full, 0, p.status, 4);
  // bulk exchange: every copy into this CTA has landed; the matching wait is at the end of the kernel
  if (p.bulk_push) {
    __syncwarp();
    cluster_arrive_relaxed();
  }
  if (__all_sync(0xffffffffu, arrived)) {  // warp-uniform: select_rows shuffles
    if (S == 4) select_rows<KMAX, 4>(p, s_partial, s_hist, st, block, krank);
    else if (S == 2) select_rows<KMAX, 2>(p, s_partial, s_hist, st, block, krank);
    else select_rows<KMAX, 1>(p, s_partial, s_hist, st, block, krank);
  }
  asm volatile("bar.sync 1, 256;" ::: "memory");  // the kSelThreads threads only
  if (p.tile_hist != nullptr) {
    const int E = p.epad, EL = p.experts;
    for (int i = st; i < (4 / S) * EL; i += kSelThreads) {
      const int sl = i / EL, e2 = i - sl * EL;
      const int tile = block * 4 + sl * S + krank;
      if (tile < p.num_tiles) p.tile_hist[(size_t)tile * EL + e2] = s_hist[sl * E + e2];
    }
  }
}

template <int KMAX>
__global__ void __launch_bounds__(kThreads, 1)
router_gemm_select_kernel(const __grid_constant__ CUtensorMap tmap_x,
                          const __grid_constant__ CUtensorMap tmap_w, const RouterParams p) {
  constexpr int kABytes = kBlockTokens * kBlockK * 2;
  static_assert(kSelThreads == 256, "bar.sync 1 counts the select threads");
  // 128-byte-swizzled TMA tiles need a 1024-byte aligned base; the pointers are derived from the
  // array itself so that the compiler keeps them in the shared address space.
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {  // uniform over the grid: every CTA would see the same offset
    record_error(p.status, kErrBadIndex | 0xff);
    return;
  }

  const int E = p.epad;  // accumulator / shared-memory width
  const int b_bytes = E * kBlockK * 2;
  const int EP = E + 4;  // padded row of a partial tile: conflict-free 128-bit accesses
  uint8_t* sA = smem;
  uint8_t* sB = sA + (size_t)p.stages * kABytes;
  float* s_partial = reinterpret_cast<float*>(sB + (size_t)p.stages * b_bytes);  // [4][32][EP]
  // transpose tiles of the exchange [4 warps][32][kChunk + 4]: the pipeline stages themselves once the
  // last MMA has read them (the usual case), else a region of their own behind the partial tiles
  float* s_own_stage = s_partial + (size_t)4 * 32 * EP;
  float* s_stage = p.stage_in_ring ? reinterpret_cast<float*>(smem) : s_own_stage;
  int32_t* s_hist = reinterpret_cast<int32_t*>(s_own_stage + (p.stage_in_ring ? 0 : kEpiWarps * 32 * (kChunk + 4)));  // [4][E]
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_hist + 4 * E);  // full[], empty[], tmem_full, part_full
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_bar + 2 * kMaxStages + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int block = blockIdx.x;
  const int krank = (int)cluster_ctarank();
  const int S = p.splitk;
  // this CTA's k blocks: kblocks * krank / S with S = 1, 2 or 4 (shifts: the prologue is on the
  // critical path of the first copy)
  const int sh = S == 4 ? 2 : (S == 2 ? 1 : 0);
  const int kb0 = (int)(((unsigned)p.kblocks * (unsigned)krank) >> sh);
  const int kb1 = (int)(((unsigned)p.kblocks * (unsigned)(krank + 1)) >> sh);
  const int nkb = kb1 - kb0;

  const uint32_t full0 = smem_u32(s_bar);
  const uint32_t empty0 = smem_u32(s_bar + kMaxStages);
  const uint32_t tmem_full = smem_u32(s_bar + 2 * kMaxStages);
  const uint32_t part_full = smem_u32(s_bar + 2 * kMaxStages + 1);

  // One barrier per thread (the prologue is on the critical path of the first copy); the descriptor
  // fetches start at once, from a warp that initialises nothing.
  if (threadIdx.x == kThreads - 32) {
    prefetch_tensormap(&tmap_x);
    prefetch_tensormap(&tmap_w);
    // The tokens are an input of the whole route: nothing this library launches writes them.  Their
    // boxes are requested into L2 here, ahead of the dependency wait below, so that with programmatic
    // dependent launch the HBM reads of this route start under the tail of the kernel before it
    // (in a sequence of routes: under the previous scatter's stores).  Only a hint: the copies into
    // shared memory are issued after the wait and read whatever L2 then holds.
    if (p.prefetch_x)
      for (int it = 0; it < nkb; ++it) tma_prefetch_l2_2d(&tmap_x, (kb0 + it) * kBlockK, block * kBlockTokens);
  }
  if ((int)threadIdx.x < 2 * p.stages + 2) {
    const int t = (int)threadIdx.x;
    if (t < p.stages) mbar_init(full0 + 8 * t, 1);
    else if (t < 2 * p.stages) mbar_init(empty0 + 8 * (t - p.stages), 1);
    else if (t == 2 * p.stages) mbar_init(tmem_full, (uint32_t)p.nacc);  // one commit per issuing warp
    else if (!p.bulk_push) mbar_init(part_full, kEpiThreads);  // S source CTAs x (4 / S) warps x 32 lanes
    else {
      // bulk exchange: the four quarters this CTA owns arrive as byte counts on the barrier
      mbar_init(part_full, 1);
      fence_barrier_init();
      mbar_expect_tx(part_full, (uint32_t)(4 * 32 * (kChunk + 4) * sizeof(float)));
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  for (int i = threadIdx.x; i < 4 * E; i += kThreads) s_hist[i] = 0;
  __syncthreads();
  // Remote shared-memory traffic below needs every CTA of the cluster to be running with its
  // barriers initialised: arrive now, wait just before the first remote access.
  cluster_arrive_relaxed();
  // Let a dependent kernel (launched with programmatic stream serialisation) start its own input
  // prefetch as soon as it finds room; it still waits for this grid to finish before reading what
  // we write.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp < kProducers) {
    // ------------------------------ TMA producers ------------------------------
    // Producer warp j owns the pipeline stages s with s % producers == j and fills them in order,
    // so the parity of a stage's barrier is never ambiguous.
    const int producers = min(kProducers, p.stages);
    // With programmatic dependent launch this grid may start while its predecessor in the stream is
    // still running: everything above overlaps it; global memory is first touched after this wait.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (lane == 0 && warp < producers) {
      // stage, its owner and the parity of its use advance without divisions: this thread is on the
      // critical path of its fills
      int s = 0, owner = 0;
      uint32_t ph = 0;
      for (int it = 0; it < nkb; ++it) {
        const int s_now = s, owner_now = owner;
        const uint32_t ph_now = ph;
        if (++owner == producers) owner = 0;
        if (++s == p.stages) { s = 0; owner = 0; ph ^= 1u; }
        if (owner_now != warp) continue;
        if (!mbar_wait(empty0 + 8 * s_now, ph_now ^ 1u, p.status, 1)) break;
        mbar_expect_tx(full0 + 8 * s_now, (uint32_t)(kABytes + b_bytes));
        const int kb = kb0 + it;
        tma_load_2d(smem_u32(sA + (size_t)s_now * kABytes), &tmap_x, full0 + 8 * s_now, kb * kBlockK, block * kBlockTokens);
        tma_load_2d(smem_u32(sB + (size_t)s_now * b_bytes), &tmap_w, full0 + 8 * s_now, kb * kBlockK, 0);
      }
    }
    __syncwarp();
    cluster_wait_acquire();
    select_phase<KMAX>(p, s_partial, s_hist, part_full, warp * 32 + lane, block, krank);
  } else if (warp < kProducers + kMmaWarps) {
    // ------------------------------ MMA issuers (the first also owns the TMEM allocation) ---------------
    // Issuing warp m owns the stages s with s % nacc == m, consumes their fills in order and
    // accumulates all of them into its own TMEM accumulator m.
    const int m = warp - kProducers;
    if (m == 0) {
      tmem_alloc(smem_u32(s_tmem), (uint32_t)p.tmem_cols);
      tmem_relinquish();
    }
    tc_fence_before();
    asm volatile("bar.sync 2, 192;" ::: "memory");  // MMA + epilogue warps: the TMEM address is published
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    if (lane == 0 && m < p.nacc) {
      const uint32_t idesc = make_idesc_f16(kBlockTokens, E, p.bf16, 0, 0);
      bool fresh = true;  // accumulator m holds nothing yet
      int s_next = 0, owner = 0;
      uint32_t ph_next = 0;
      for (int it = 0; it < nkb; ++it) {
        const int s = s_next, owner_now = owner;
        const uint32_t ph = ph_next;
        if (++owner == p.nacc) owner = 0;
        if (++s_next == p.stages) { s_next = 0; owner = 0; ph_next ^= 1u; }
        if (owner_now != m) continue;
        if (!mbar_wait(full0 + 8 * s, ph, p.status, 2)) break;
        tc_fence_after();
        const uint64_t adesc = make_desc_kmajor_sw128(smem_u32(sA + (size_t)s * kABytes));
        const uint64_t bdesc = make_desc_kmajor_sw128(smem_u32(sB + (size_t)s * b_bytes));
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
          // +32 bytes per K step inside the 128-byte swizzle row (address field is in 16-byte units)
          umma_f16(tmem_base + (uint32_t)(m * E), adesc + 2 * k, bdesc + 2 * k, idesc, (uint32_t)(!fresh || k != 0));
        }
        fresh = false;
        umma_commit(empty0 + 8 * s);  // stage may be refilled once these MMAs have read it
      }
      umma_commit(tmem_full);  // this warp's accumulator is complete (or abandoned: the epilogue must not hang)
    }
    __syncwarp();
    cluster_wait_acquire();
    if (p.bulk_push) cluster_arrive_relaxed();  // see the end of the kernel
  } else {
    // ------------------------------ epilogue warps ------------------------------
    asm volatile("bar.sync 2, 192;" ::: "memory");
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int ew = warp - kProducers - kMmaWarps;
    const int dest = q % S;
    const int slot = q / S;
    asm volatile("griddepcontrol.wait;" ::: "memory");  // before the first global write (PDL)
    cluster_wait_acquire();  // every CTA of the cluster has initialised its barriers
    // ---- this warp's quarter of the partial accumulator -> its owner's shared memory ----
    const bool ok = mbar_wait(tmem_full, 0, p.status, 3);
    tc_fence_after();
    const unsigned mask = (p.acc_mask >> (2 * krank)) & 3u;
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
    float* stage = s_stage + (size_t)ew * 32 * (kChunk + 4);
    // row (slot * S + krank) * 32 + r of the owner's partial buffer
    const uint32_t owner_part = map_to_cta(smem_u32(s_partial), (uint32_t)dest) + (uint32_t)((slot * S + krank) * 32 * EP) * 4u;
    for (int c0 = 0; c0 < E; c0 += kChunk) {
      const int width = min(kChunk, E - c0);  // 16, 32, 48 or 64 columns
      // (1) sum the accumulators of this chunk: thread = row, registers = columns; all loads of the
      // chunk are in flight together
      float v[kChunk];
      {
        uint32_t r[kMmaWarps][kChunk];
#pragma unroll
        for (int a = 0; a < kMmaWarps; ++a)
#pragma unroll
          for (int i = 0; i < kChunk; ++i) r[a][i] = 0u;
        if (ok) {
#pragma unroll
          for (int a = 0; a < kMmaWarps; ++a) {
            if (a < p.nacc && ((mask >> a) & 1u)) {
#pragma unroll
              for (int g = 0; g < kChunk / 16; ++g)
                if (g * 16 < width)
                  tmem_ld16_nowait(taddr + (uint32_t)(a * E + c0 + g * 16), reinterpret_cast<uint32_t(&)[16]>(r[a][g * 16]));
            }
          }
          tmem_ld_wait();
        }
#pragma unroll
        for (int i = 0; i < kChunk; ++i) {
          float acc = __uint_as_float(r[0][i]);
#pragma unroll
          for (int a = 1; a < kMmaWarps; ++a) acc += __uint_as_float(r[a][i]);
          v[i] = acc;
        }
      }
      // (2) transpose through this warp's staging tile so that a store instruction covers whole rows
      __syncwarp();  // the previous chunk has been read out of the staging tile
#pragma unroll
      for (int i = 0; i < kChunk; i += 4)
        *reinterpret_cast<float4*>(stage + lane * (kChunk + 4) + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
      __syncwarp();
      if (p.bulk_push) {
        // (3a) E == 64: the staging tile has the layout of the owner's block (32 rows of E + 4 floats),
        // so one bulk copy moves the quarter and counts its bytes on the owner's barrier: no remote
        // store instructions and no release-arrive behind them
        fence_proxy_async();  // this lane's staging writes, for the async proxy
        __syncwarp();
        if (lane == 0)
          bulk_copy_to_cluster(owner_part, smem_u32(stage), (uint32_t)(32 * (kChunk + 4) * sizeof(float)),
                               map_to_cta(part_full, (uint32_t)dest));
        break;
      }
      // (3) 16 lanes x 16 bytes cover the (up to) 64 columns of one row: two rows per instruction
      const int cl = (lane & 15) * 4;
      if (cl < width) {
#pragma unroll 4
        for (int r2 = 0; r2 < 32; r2 += 2) {
          const int r = r2 + (lane >> 4);
          const float4 t = *reinterpret_cast<const float4*>(stage + r * (kChunk + 4) + cl);
          st_cluster_v4u(owner_part + (uint32_t)(r * EP + c0 + cl) * 4u, __float_as_uint(t.x), __float_as_uint(t.y),
                         __float_as_uint(t.z), __float_as_uint(t.w));
        }
      }
    }
    if (!p.bulk_push) mbar_arrive_remote(map_to_cta(part_full, (uint32_t)dest));  // releases this thread's stores
    select_phase<KMAX>(p, s_partial, s_hist, part_full, (kProducers + ew) * 32 + lane, block, krank);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kProducers) {
    tc_fence_after();
    tmem_dealloc(*s_tmem, (uint32_t)p.tmem_cols);
  }
  // A bulk copy reads its source asynchronously and reports only to its destination.  The select
  // threads of every CTA arrived at the cluster barrier once their own `part_full` had completed (the
  // MMA warps on their way here), so when it completes every copy of the cluster has landed and no
  // CTA's shared memory is still being read.
  if (p.bulk_push) cluster_wait_acquire();
}

int launch_router(const void* x, const void* w, int tokens, int d, int experts, int top_k, int skew_experts,
                  float skew_bias, int dtype, int32_t* idx, float* gates, float* logits_out, const Workspace& ws,
                  cudaStream_t stream) {
  const int epad = (experts + 15) / 16 * 16;  // W rows past `experts` are zero-filled by the TMA unit
  CUtensorMap tmap_x, tmap_w;
  int rc = encode_tmap_2d(&tmap_x, x, (uint64_t)tokens, (uint64_t)d, (uint64_t)d * 2, kBlockK, kBlockTokens);
  if (rc != MOE_OK) return rc;
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
  p.num_tiles = ws.num_tiles;
  const int stage_bytes = kBlockTokens * kBlockK * 2 + epad * kBlockK * 2;
  int fixed = 128 * (epad + 4) * 4 + 4 * epad * 4 + (2 * kMaxStages + 2) * 8 + 16;
  const int transpose_bytes = kEpiWarps * 32 * (kChunk + 4) * 4;
  int stages = (kSmemLimit - 1024 - fixed) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  const int max_fills = (p.kblocks + p.splitk - 1) / p.splitk;
  if (stages > max_fills) stages = max_fills;
  if (stages < 1) return fail(MOE_ERR_UNSUPPORTED, "router GEMM: shared memory budget exceeded for experts=%d", experts);
  p.stages = stages;
  p.stage_in_ring = stages * stage_bytes >= transpose_bytes;
  {
    static const int bulk_on = [] { const char* v = getenv("MOE_B200_ROUTER_BULK"); return (v && v[0] == '0') ? 0 : 1; }();
    p.bulk_push = (bulk_on && epad == kChunk) ? 1 : 0;
    static const int pf_on = [] { const char* v = getenv("MOE_B200_ROUTER_PREFETCH"); return (v && v[0] == '0') ? 0 : 1; }();
    p.prefetch_x = pf_on;
  }
  if (!p.stage_in_ring) fixed += transpose_bytes;  // few small stages (tiny d_model): the tiles get room of their own
  // every issuing warp needs a stage of its own; both accumulators must fit the 512 TMEM columns
  p.nacc = kMmaWarps;
  while (p.nacc > 1 && (p.nacc > stages || p.nacc * epad > 512)) p.nacc /= 2;
  int cols = 32;
  while (cols < p.nacc * epad) cols *= 2;
  p.tmem_cols = cols;
  p.acc_mask = 0;
  for (int r = 0; r < p.splitk; ++r) {
    const int k0 = (int)(((long long)p.kblocks * r) / p.splitk), k1 = (int)(((long long)p.kblocks * (r + 1)) / p.splitk);
    unsigned mask = 0;
    for (int it = 0; it < k1 - k0; ++it) mask |= 1u << ((it % stages) % p.nacc);
    p.acc_mask |= mask << (2 * r);
  }
  p.idx = idx; p.gates = gates; p.logits_out = logits_out;
  p.tile_hist = ws.tile_hist; p.status = ws.status;
  const size_t smem = 1024 + (size_t)stages * stage_bytes + fixed;
  const int kmax = top_k <= 1 ? 1 : (top_k <= 2 ? 2 : (top_k <= 4 ? 4 : 8));
  auto kernel = kmax == 1 ? router_gemm_select_kernel<1>
                : kmax == 2 ? router_gemm_select_kernel<2>
                : kmax == 4 ? router_gemm_select_kernel<4>
                            : router_gemm_select_kernel<8>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((tokens + kBlockTokens - 1) / kBlockTokens, p.splitk, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = p.splitk;
  attr[0].val.clusterDim.z = 1;
  // the prologue (barrier set-up, TMEM allocation, tensor-map prefetch) may run under the tail of the
  // preceding kernel of the stream; the kernel waits for that kernel before it touches global memory
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "router GEMM: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  e = cudaLaunchKernelEx(&cfg, kernel, tmap_x, tmap_w, p);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "router_gemm_select_kernel: %s", cudaGetErrorString(e));
  note_launch();
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
    rc = launch_router(x, w_router, tokens, d, experts, top_k, skew_experts, skew_bias, dtype, idx, gates, logits_out,
                       ws, s);
    if (rc != MOE_OK) return rc;
  }
  return launch_scan_scatter(x, 2, idx, tokens, d, experts, top_k, counts, offsets, packed, row_route, route_row,
                             ws, s);
}
