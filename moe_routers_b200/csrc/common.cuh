// Shared host/device helpers for libmoe_b200 (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "../../include/moe_b200.h"

namespace moe {

// ---- workspace layout -------------------------------------------------------
// [0, 256)            status block: int32 words, word 0 = first recorded error; words 2..3 = limit of
//                     every bounded device-side wait in nanoseconds as one uint64 (0 = the default)
// [256, 512)          control block: tickets / barrier counters (self-resetting)
// [512, ...)          tile histograms  int32 [num_tiles][experts]
//                     tile bases       int32 [num_tiles][experts]
//                     float scratch    float [2][kMaxGridBlocks][experts]  (Sinkhorn column partials)
constexpr int kStatusBytes = 256;
constexpr int kControlBytes = 256;
constexpr int kTileTokens = 32;  // tokens per histogram tile (router GEMM epilogue and pack agree)
constexpr int kMaxGridBlocks = 256;  // upper bound of the co-resident grid of the Sinkhorn kernel

// Device-side error codes written to status word 0 (first error wins).
constexpr int kErrMbarTimeout = 0x100;   // | role id
constexpr int kErrGridBarrier = 0x200;
constexpr int kErrBadIndex = 0x300;
constexpr int kErrPeerWait = 0x400;      // | rank that never signalled

struct Workspace {
  int32_t* status;
  int32_t* control;
  int32_t* tile_hist;
  int32_t* tile_base;
  float* fscratch;
  int num_tiles;
};

inline int num_tiles_for(int tokens) { return (tokens + kTileTokens - 1) / kTileTokens; }

inline size_t workspace_bytes_for(int tokens, int experts, int /*top_k*/) {
  size_t tiles = (size_t)num_tiles_for(tokens > 0 ? tokens : 1);
  size_t hist = tiles * (size_t)experts * sizeof(int32_t);
  hist = (hist + 255) & ~(size_t)255;
  return (size_t)kStatusBytes + kControlBytes + 2 * hist + 2 * (size_t)kMaxGridBlocks * experts * sizeof(float);
}

inline Workspace carve(void* ws, int tokens, int experts) {
  Workspace w;
  char* p = static_cast<char*>(ws);
  w.status = reinterpret_cast<int32_t*>(p);
  w.control = reinterpret_cast<int32_t*>(p + kStatusBytes);
  w.num_tiles = num_tiles_for(tokens > 0 ? tokens : 1);
  size_t hist = (size_t)w.num_tiles * (size_t)experts * sizeof(int32_t);
  hist = (hist + 255) & ~(size_t)255;
  w.tile_hist = reinterpret_cast<int32_t*>(p + kStatusBytes + kControlBytes);
  w.tile_base = reinterpret_cast<int32_t*>(p + kStatusBytes + kControlBytes + hist);
  w.fscratch = reinterpret_cast<float*>(p + kStatusBytes + kControlBytes + 2 * hist);
  return w;
}

// ---- error text (thread local, host) ---------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);  // counts the launch when it succeeded
void note_launch();                  // for launches checked by hand (cudaLaunchKernelEx)
bool pdl_enabled();                  // programmatic dependent launch between the route kernels

__device__ __forceinline__ void record_error(int32_t* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// ---- dtype helpers ----------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Ordering used by every selection in the library: larger value first, on
// equal values the lower index first.
__device__ __forceinline__ bool better(float av, int ai, float bv, int bi) {
  return (av > bv) || (av == bv && ai < bi);
}

__device__ __forceinline__ uint32_t lanemask_lt() {
  uint32_t m;
  asm volatile("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

}  // namespace moe
