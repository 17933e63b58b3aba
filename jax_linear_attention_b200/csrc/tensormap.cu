// Host side of tma.cuh: cuTensorMapEncodeTiled resolved through the runtime's driver entry point (the library
// does not link libcuda directly).
#include <mutex>

#include "tma.cuh"

namespace jla {
namespace tma {
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      return static_cast<EncodeFn>(nullptr);
    }
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

}  // namespace

bool encode_3d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t mid, uint64_t outer, uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  if (outer == 0) outer = 1;
  const cuuint64_t dims[3] = {inner, mid, outer};
  const cuuint64_t strides[2] = {inner * 2, inner * mid * 2};  // bytes, dims 1 and 2
  const cuuint32_t box[3] = {64, 1, box_rows};
  const cuuint32_t estr[3] = {1, 1, 1};
  auto encode = [&] {
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult rc = encode();
  if (rc == CUDA_ERROR_INVALID_CONTEXT || rc == CUDA_ERROR_NOT_INITIALIZED) {
    // A host thread that has made no runtime call yet (an autograd worker, say) has no current context for a driver
    // call: a no-op runtime call binds the device's primary context to it.
    cudaFree(nullptr);
    rc = encode();
  }
  if (rc != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed (%d) for dims {%llu, %llu, %llu}", (int)rc, (unsigned long long)inner,
              (unsigned long long)mid, (unsigned long long)outer);
    return false;
  }
  return true;
}

}  // namespace tma
}  // namespace jla
