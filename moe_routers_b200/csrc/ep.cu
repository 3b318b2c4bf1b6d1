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
#include <cstring>

#include "sm100.cuh"

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

// ---------------------------------------------------------------------------
// Device-initiated dispatch / combine over peer memory (NVLink): no staging, no re-bucketing.
//
// Every rank holds the all-gathered counts, so it can compute where each of its expert segments
// belongs in the OWNER's expert-major inbox and stores the rows there directly with plain 128-bit
// peer stores (`push`); after the expert FFN the owner stores every result row straight into the
// packed slot of the rank it came from (`push back`).  The ranks synchronise between the phases
// on the host side of the stream (a tiny NCCL collective): the kernels themselves never wait on a
// peer.  No multicast, no TMA on peer memory.
namespace moe {
namespace {

// dir 0 (dispatch): segment = (dest rank p, local expert e of p): rows packed[off_me[pE+e] ..] of this
//   rank -> inbox of p at row B_p(me, e).
// dir 1 (combine):  segment = (source rank s, local expert e of me): rows yb[B_me(s, e) ..] of this
//   rank -> y_home of s at row off_s[meE + e].
// off_r[g] = rows of rank r routed to experts < g; B_p(s, e) = rows in p's inbox before (s, e) in
// expert-major order.
__global__ void __launch_bounds__(kThreads)
ep_push_kernel(const char* __restrict__ local, char* const* __restrict__ peer_bufs,
               const int32_t* __restrict__ counts_all, int experts, int world, int rank, int dir,
               size_t row_bytes, int32_t* __restrict__ local_offsets) {
  __shared__ long long s_from, s_to;
  __shared__ int s_len;
  const int el = experts / world;
  const int peer = blockIdx.x / el;  // dest rank (dispatch) or source rank (combine)
  const int e = blockIdx.x % el;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    const int owner = dir == 0 ? peer : rank;    // whose inbox the expert-major offset refers to
    const int sender = dir == 0 ? rank : peer;   // whose packed order the packed offset refers to
    const int ge = owner * el + e;               // global expert of this segment
    // packed offset of (sender, ge): rows of `sender` routed to experts < ge
    int off = 0;
    for (int g = lane; g < ge; g += 32) off += counts_all[(size_t)sender * experts + g];
    // expert-major offset of (sender, e) in owner's inbox
    int b = 0, total = 0;
    for (int i = lane; i < world * el; i += 32) {
      const int ss = i / el, ee = i % el;
      const int l = counts_all[(size_t)ss * experts + owner * el + ee];
      if (ee < e || (ee == e && ss < sender)) b += l;
      total += l;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      off += __shfl_xor_sync(0xffffffffu, off, o);
      b += __shfl_xor_sync(0xffffffffu, b, o);
      total += __shfl_xor_sync(0xffffffffu, total, o);
    }
    if (lane == 0) {
      s_len = counts_all[(size_t)sender * experts + ge];
      s_from = (long long)(dir == 0 ? off : b);
      s_to = (long long)(dir == 0 ? b : off);
    }
    // the owner's own expert-major offsets, for its grouped GEMM (dispatch only, one CTA per expert)
    if (dir == 0 && local_offsets != nullptr && peer == rank && blockIdx.y == 0) {
      int first = 0, tot_mine = 0;  // rows before expert e / all rows in MY inbox
      for (int i = lane; i < world * el; i += 32) {
        const int ss = i / el, ee = i % el;
        const int l = counts_all[(size_t)ss * experts + rank * el + ee];
        if (ee < e) first += l;
        tot_mine += l;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        first += __shfl_xor_sync(0xffffffffu, first, o);
        tot_mine += __shfl_xor_sync(0xffffffffu, tot_mine, o);
      }
      if (lane == 0) {
        local_offsets[e] = first;
        if (e == el - 1) local_offsets[el] = tot_mine;
      }
    }
  }
  __syncthreads();
  const size_t bytes = (size_t)s_len * row_bytes;
  if (bytes == 0) return;
  const char* src = local + (size_t)s_from * row_bytes;
  char* dst = peer_bufs[peer] + (size_t)s_to * row_bytes;
  const size_t chunk = ((bytes / gridDim.y + 15) / 16 + 1) * 16;
  const size_t lo = (size_t)blockIdx.y * chunk;
  const size_t hi = lo + chunk < bytes ? lo + chunk : bytes;
  if (lo >= hi) return;
  const uint4* s4 = reinterpret_cast<const uint4*>(src + lo);
  uint4* d4 = reinterpret_cast<uint4*>(dst + lo);
  const size_t n = (hi - lo) / 16;
  size_t i = threadIdx.x;
  for (; i + 3 * kThreads < n; i += 4 * kThreads) {
    const uint4 r0 = __ldg(s4 + i), r1 = __ldg(s4 + i + kThreads), r2 = __ldg(s4 + i + 2 * kThreads),
                r3 = __ldg(s4 + i + 3 * kThreads);
    d4[i] = r0; d4[i + kThreads] = r1; d4[i + 2 * kThreads] = r2; d4[i + 3 * kThreads] = r3;
  }
  for (; i < n; i += kThreads) d4[i] = __ldg(s4 + i);
}


// Row targets for the combine direction: for every row of this rank's expert-major inbox, the address
// of the packed slot it came from (in the memory of the rank that sent it).  One CTA per (source rank
// s, local expert e) segment: inbox rows B_me(s, e) + j  ->  home[s] + (off_s[me*E_local + e] + j) rows.
// moe_grouped_gemm_rows takes this table so that the second expert GEMM stores its result rows there.
__global__ void __launch_bounds__(kThreads)
ep_row_targets_kernel(char* const* __restrict__ home_bufs, const int32_t* __restrict__ counts_all, int experts,
                      int world, int rank, size_t row_bytes, char** __restrict__ row_ptrs) {
  __shared__ int s_off, s_b, s_len;
  const int el = experts / world;
  const int src = blockIdx.x / el;
  const int e = blockIdx.x % el;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    const int ge = rank * el + e;
    int off = 0, b = 0;
    for (int g = lane; g < ge; g += 32) off += counts_all[(size_t)src * experts + g];
    for (int i = lane; i < world * el; i += 32) {
      const int ss = i / el, ee = i % el;
      if (ee < e || (ee == e && ss < src)) b += counts_all[(size_t)ss * experts + rank * el + ee];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      off += __shfl_xor_sync(0xffffffffu, off, o);
      b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    if (lane == 0) {
      s_off = off; s_b = b;
      s_len = counts_all[(size_t)src * experts + ge];
    }
  }
  __syncthreads();
  char* base = home_bufs[src] + (size_t)s_off * row_bytes;
  for (int j = threadIdx.x; j < s_len; j += kThreads) row_ptrs[s_b + j] = base + (size_t)j * row_bytes;
}

// Dispatch destinations for moe_pack_scatter_to: the rows this rank routes to global expert g =
// p * E_local + e start at row B_p(me, e) of rank p's expert-major inbox.  One CTA per expert; the
// CTAs of this rank's own experts also write its local_offsets (as the dispatch push does).
__global__ void __launch_bounds__(32)
ep_segment_bases_kernel(char* const* __restrict__ inbox_bufs, const int32_t* __restrict__ counts_all, int experts,
                        int world, int rank, size_t row_bytes, char** __restrict__ seg_base,
                        int32_t* __restrict__ local_offsets) {
  const int el = experts / world;
  const int owner = blockIdx.x / el;
  const int e = blockIdx.x % el;
  const int lane = threadIdx.x;
  int b = 0, first = 0, total = 0;
  for (int i = lane; i < world * el; i += 32) {
    const int ss = i / el, ee = i % el;
    const int l = counts_all[(size_t)ss * experts + owner * el + ee];
    if (ee < e || (ee == e && ss < rank)) b += l;
    if (ee < e) first += l;
    total += l;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    b += __shfl_xor_sync(0xffffffffu, b, o);
    first += __shfl_xor_sync(0xffffffffu, first, o);
    total += __shfl_xor_sync(0xffffffffu, total, o);
  }
  if (lane == 0) {
    seg_base[blockIdx.x] = inbox_bufs[owner] + (size_t)b * row_bytes;
    if (owner == rank && local_offsets != nullptr) {
      local_offsets[e] = first;
      if (e == el - 1) local_offsets[el] = total;
    }
  }
}
}  // namespace
}  // namespace moe

extern "C" int moe_ep_push(const void* local, void* const* peer_bufs, const int32_t* counts_all, int experts,
                           int world, int rank, int combine, int d, int elem_bytes, int32_t* local_offsets,
                           void* stream) {
  using namespace moe;
  if (experts <= 0 || world <= 0 || experts % world != 0)
    return fail(MOE_ERR_ARG, "experts must be divisible by world_size");
  if (rank < 0 || rank >= world) return fail(MOE_ERR_ARG, "moe_ep_push: bad rank");
  if (d <= 0 || (elem_bytes != 2 && elem_bytes != 4) || ((size_t)d * elem_bytes) % 16 != 0)
    return fail(MOE_ERR_ARG, "moe_ep_push: rows must be a multiple of 16 bytes");
  if (!local || !peer_bufs || !counts_all) return fail(MOE_ERR_ARG, "moe_ep_push: null pointer");
  if ((reinterpret_cast<uintptr_t>(local) & 15) != 0) return fail(MOE_ERR_ARG, "moe_ep_push: local must be 16-byte aligned");
  dim3 grid(experts, 8, 1);  // world * (experts / world) segments, 8 CTAs each
  ep_push_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const char*>(local), reinterpret_cast<char* const*>(peer_bufs), counts_all, experts, world, rank,
      combine ? 1 : 0, (size_t)d * elem_bytes, local_offsets);
  return check_launch("ep_push_kernel");
}

extern "C" int moe_ep_row_targets(void* const* home_bufs, const int32_t* counts_all, int experts, int world, int rank,
                                  int d, int elem_bytes, void** row_ptrs, void* stream) {
  using namespace moe;
  if (experts <= 0 || world <= 0 || experts % world != 0)
    return fail(MOE_ERR_ARG, "experts must be divisible by world_size");
  if (rank < 0 || rank >= world) return fail(MOE_ERR_ARG, "moe_ep_row_targets: bad rank");
  if (d <= 0 || (elem_bytes != 2 && elem_bytes != 4) || ((size_t)d * elem_bytes) % 16 != 0)
    return fail(MOE_ERR_ARG, "moe_ep_row_targets: rows must be a multiple of 16 bytes");
  if (!home_bufs || !counts_all || !row_ptrs) return fail(MOE_ERR_ARG, "moe_ep_row_targets: null pointer");
  ep_row_targets_kernel<<<experts, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<char* const*>(home_bufs), counts_all, experts, world, rank, (size_t)d * elem_bytes,
      reinterpret_cast<char**>(row_ptrs));
  return check_launch("ep_row_targets_kernel");
}

extern "C" int moe_ep_segment_bases(void* const* inbox_bufs, const int32_t* counts_all, int experts, int world,
                                    int rank, int d, int elem_bytes, void** seg_base, int32_t* local_offsets,
                                    void* stream) {
  using namespace moe;
  if (experts <= 0 || world <= 0 || experts % world != 0)
    return fail(MOE_ERR_ARG, "experts must be divisible by world_size");
  if (rank < 0 || rank >= world) return fail(MOE_ERR_ARG, "moe_ep_segment_bases: bad rank");
  if (d <= 0 || (elem_bytes != 2 && elem_bytes != 4) || ((size_t)d * elem_bytes) % 16 != 0)
    return fail(MOE_ERR_ARG, "moe_ep_segment_bases: rows must be a multiple of 16 bytes");
  if (!inbox_bufs || !counts_all || !seg_base) return fail(MOE_ERR_ARG, "moe_ep_segment_bases: null pointer");
  ep_segment_bases_kernel<<<experts, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<char* const*>(inbox_bufs), counts_all, experts, world, rank, (size_t)d * elem_bytes,
      reinterpret_cast<char**>(seg_base), local_offsets);
  return check_launch("ep_segment_bases_kernel");
}

// ---------------------------------------------------------------------------
// Rank-to-rank signals over the peer mappings: the phase ordering of the expert-parallel layer
// without a collective.  Every rank owns a flag table int32 [slots][world] in memory its peers have
// mapped; `signal` stores `value` into entry [slot][my rank] of every rank's table (after an optional
// small payload, e.g. the per-expert counts, into every rank's payload buffer), `wait` polls the
// rank's OWN table until all entries of the slot have reached `value`.  Values only grow (the
// caller passes its call counter), so a table never has to be cleared.  The wait is bounded in
// time like every other device-side wait of the library.
namespace moe {
namespace {

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kThreads)
ep_signal_kernel(int32_t* const* __restrict__ peer_flags, int world, int rank, int slot, int32_t value,
                 const int32_t* __restrict__ payload, int32_t* const* __restrict__ peer_payload,
                 size_t payload_offset_words, int payload_words) {
  if (payload != nullptr) {
    for (int i = threadIdx.x; i < payload_words * world; i += kThreads) {
      const int p = i / payload_words, j = i - p * payload_words;
      peer_payload[p][payload_offset_words + j] = payload[j];
    }
  }
  // everything this rank stored before (earlier kernels of the stream included) becomes visible to
  // the peers before the flag does
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < world) st_release_sys(peer_flags[threadIdx.x] + (size_t)slot * world + rank, value);
}

__global__ void __launch_bounds__(32)
ep_wait_kernel(const int32_t* __restrict__ flags, int world, int slot, int32_t value, int32_t* status) {
  const int32_t* mine = flags + (size_t)slot * world;
  for (int p = threadIdx.x; p < world; p += 32) {
    bool seen = false;
#pragma unroll 1
    for (int i = 0; i < 4096 && !seen; ++i) seen = ld_acquire_sys(mine + p) - value >= 0;
    if (!seen) {
      const unsigned long long t0 = sm100::globaltimer_ns();
      const unsigned long long limit = sm100::wait_limit_ns(status);
      while (!seen) {
#pragma unroll 1
        for (int i = 0; i < 256 && !seen; ++i) seen = ld_acquire_sys(mine + p) - value >= 0;
        if (!seen && sm100::globaltimer_ns() - t0 > limit) {
          record_error(status, kErrPeerWait | (p & 0xff));
          break;
        }
      }
    }
  }
  __threadfence_system();
}

}  // namespace
}  // namespace moe

namespace moe {
namespace {
// signal + wait in one launch (one CTA): the layer's phase boundary costs one kernel, not two
__global__ void __launch_bounds__(kThreads)
ep_sync_kernel(int32_t* const* __restrict__ peer_flags, const int32_t* __restrict__ flags, int world, int rank, int slot,
               int32_t value, const int32_t* __restrict__ payload, int32_t* const* __restrict__ peer_payload,
               size_t payload_offset_words, int payload_words, int32_t* status) {
  if (payload != nullptr) {
    for (int i = threadIdx.x; i < payload_words * world; i += kThreads) {
      const int p = i / payload_words, j = i - p * payload_words;
      peer_payload[p][payload_offset_words + j] = payload[j];
    }
  }
  __threadfence_system();
  __syncthreads();
  const int32_t* mine = flags + (size_t)slot * world;
  for (int p = threadIdx.x; p < world; p += kThreads) {
    st_release_sys(peer_flags[p] + (size_t)slot * world + rank, value);
    bool seen = false;
#pragma unroll 1
    for (int i = 0; i < 4096 && !seen; ++i) seen = ld_acquire_sys(mine + p) - value >= 0;
    if (!seen) {
      const unsigned long long t0 = sm100::globaltimer_ns();
      const unsigned long long limit = sm100::wait_limit_ns(status);
      while (!seen) {
#pragma unroll 1
        for (int i = 0; i < 256 && !seen; ++i) seen = ld_acquire_sys(mine + p) - value >= 0;
        if (!seen && sm100::globaltimer_ns() - t0 > limit) {
          record_error(status, kErrPeerWait | (p & 0xff));
          break;
        }
      }
    }
  }
  __threadfence_system();
}
}  // namespace
}  // namespace moe

extern "C" int moe_ep_sync(void* const* peer_flags, const int32_t* flags, int world, int rank, int slot, int value,
                           const int32_t* payload, void* const* peer_payload, size_t payload_offset_words,
                           int payload_words, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace moe;
  if (world <= 0 || world > kThreads || rank < 0 || rank >= world || slot < 0)
    return fail(MOE_ERR_ARG, "moe_ep_sync: bad world / rank / slot");
  if (!peer_flags || !flags) return fail(MOE_ERR_ARG, "moe_ep_sync: null flag table");
  if (payload != nullptr && (!peer_payload || payload_words <= 0)) return fail(MOE_ERR_ARG, "moe_ep_sync: bad payload");
  if (!workspace || workspace_bytes < (size_t)kStatusBytes) return fail(MOE_ERR_WORKSPACE, "moe_ep_sync: workspace missing");
  ep_sync_kernel<<<1, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<int32_t* const*>(peer_flags), flags, world, rank, slot, value, payload,
      reinterpret_cast<int32_t* const*>(peer_payload), payload_offset_words, payload ? payload_words : 0,
      static_cast<int32_t*>(workspace));
  return check_launch("ep_sync_kernel");
}

extern "C" int moe_ep_signal(void* const* peer_flags, int world, int rank, int slot, int value, const int32_t* payload,
                             void* const* peer_payload, size_t payload_offset_words, int payload_words, void* stream) {
  using namespace moe;
  if (world <= 0 || world > kThreads || rank < 0 || rank >= world || slot < 0)
    return fail(MOE_ERR_ARG, "moe_ep_signal: bad world / rank / slot");
  if (!peer_flags) return fail(MOE_ERR_ARG, "moe_ep_signal: null flag table");
  if (payload != nullptr && (!peer_payload || payload_words <= 0)) return fail(MOE_ERR_ARG, "moe_ep_signal: bad payload");
  ep_signal_kernel<<<1, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<int32_t* const*>(peer_flags), world, rank, slot, value, payload,
      reinterpret_cast<int32_t* const*>(peer_payload), payload_offset_words, payload ? payload_words : 0);
  return check_launch("ep_signal_kernel");
}

extern "C" int moe_ep_wait(const int32_t* flags, int world, int slot, int value, void* workspace, size_t workspace_bytes,
                           void* stream) {
  using namespace moe;
  if (world <= 0 || slot < 0 || !flags) return fail(MOE_ERR_ARG, "moe_ep_wait: bad argument");
  if (!workspace || workspace_bytes < (size_t)kStatusBytes) return fail(MOE_ERR_WORKSPACE, "moe_ep_wait: workspace missing");
  ep_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, world, slot, value,
                                                                   static_cast<int32_t*>(workspace));
  return check_launch("ep_wait_kernel");
}

extern "C" int moe_enable_peer_access(int peer_device) {
  using namespace moe;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "moe_enable_peer_access: %s", cudaGetErrorString(e));
  if (peer_device == dev) return MOE_OK;
  int can = 0;
  e = cudaDeviceCanAccessPeer(&can, dev, peer_device);
  if (e != cudaSuccess || !can)
    return fail(MOE_ERR_UNSUPPORTED, "moe_enable_peer_access: device %d cannot access device %d", dev, peer_device);
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();
    return MOE_OK;
  }
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "moe_enable_peer_access: %s", cudaGetErrorString(e));
  return MOE_OK;
}

// Map a peer process's device allocation into this process for access from the CURRENT device.
// `handle64` is the 64-byte cudaIpcMemHandle_t of the allocation's base (as exported by the owner);
// the handle is opened with the calling rank's own device current, which is what makes the mapping
// usable by kernels on this device (lazy peer access).  Setup helper, not on the data path.
extern "C" int moe_ipc_open(const void* handle64, void** base_out) {
  using namespace moe;
  if (!handle64 || !base_out) return fail(MOE_ERR_ARG, "moe_ipc_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* base = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(MOE_ERR_LAUNCH, "moe_ipc_open: %s", cudaGetErrorString(e));
  }
  *base_out = base;
  return MOE_OK;
}

// Export side of moe_ipc_open: the 64-byte IPC handle of the allocation that contains `ptr` and the
// offset of `ptr` inside it (a tensor of a caching allocator usually sits inside a larger block).
extern "C" int moe_ipc_export(const void* ptr, void* handle64_out, size_t* offset_out) {
  using namespace moe;
  if (!ptr || !handle64_out || !offset_out) return fail(MOE_ERR_ARG, "moe_ipc_export: null pointer");
  using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn range = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<RangeFn>(fn);
  }();
  if (!range) return fail(MOE_ERR_LAUNCH, "moe_ipc_export: cuMemGetAddressRange is not available from this driver");
  CUdeviceptr base = 0;
  size_t size = 0;
  if (range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS || base == 0)
    return fail(MOE_ERR_ARG, "moe_ipc_export: not a device allocation");
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(MOE_ERR_UNSUPPORTED, "moe_ipc_export: %s (the buffer must come from cudaMalloc, not a virtual-memory pool)",
                cudaGetErrorString(e));
  }
  memcpy(handle64_out, &h, sizeof(h));
  *offset_out = reinterpret_cast<uintptr_t>(ptr) - static_cast<uintptr_t>(base);
  return MOE_OK;
}

extern "C" int moe_ipc_close(void* base) {
  using namespace moe;
  if (!base) return MOE_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(base);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(MOE_ERR_LAUNCH, "moe_ipc_close: %s", cudaGetErrorString(e));
  }
  return MOE_OK;
}
