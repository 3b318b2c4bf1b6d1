// Host side of TMA: tensor-map encoding through the driver entry point
// cuTensorMapEncodeTiled, resolved at run time (the library does not link
// libcuda, so it builds and loads on machines without a driver).
#include <mutex>

#include "sm100.cuh"

namespace moe {
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

}  // namespace

int encode_tmap_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                   uint32_t box_cols, uint32_t box_rows) {
  EncodeFn fn = get_encode();
  if (!fn) return fail(MOE_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15))
    return fail(MOE_ERR_ARG, "TMA needs a 16-byte aligned base and row stride");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MOE_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return MOE_OK;
}

int encode_tmap_3d(CUtensorMap* map, const void* base, uint64_t d2, uint64_t rows, uint64_t cols,
                   uint64_t row_stride_bytes, uint64_t d2_stride_bytes, uint32_t box_cols, uint32_t box_rows) {
  EncodeFn fn = get_encode();
  if (!fn) return fail(MOE_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15) || (d2_stride_bytes & 15))
    return fail(MOE_ERR_ARG, "TMA needs a 16-byte aligned base and strides");
  cuuint64_t dims[3] = {cols, rows, d2};
  cuuint64_t strides[2] = {row_stride_bytes, d2_stride_bytes};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MOE_ERR_LAUNCH, "cuTensorMapEncodeTiled (3d) failed with CUresult %d", (int)r);
  return MOE_OK;
}

// 4-D view {d0 (contiguous), d1, d2, d3} with byte strides s1, s2, s3 and a box b0 x b1 x b2 x b3.
int encode_tmap_4d(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1,
                   uint64_t s2, uint64_t s3, uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
  EncodeFn fn = get_encode();
  if (!fn) return fail(MOE_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1 & 15) || (s2 & 15) || (s3 & 15))
    return fail(MOE_ERR_ARG, "TMA needs a 16-byte aligned base and strides");
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1, s2, s3};
  cuuint32_t box[4] = {b0, b1, b2, b3};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MOE_ERR_LAUNCH, "cuTensorMapEncodeTiled (4d) failed with CUresult %d", (int)r);
  return MOE_OK;
}

}  // namespace moe
