#include "kernels.h"
#include <cudaTypedefs.h>

namespace ghb {

static int g_last_encode_error = 0;
int last_encode_error() { return g_last_encode_error; }

// The encode call is a driver-API entry: a thread that has made no runtime call yet (an autograd worker running its
// first backward node) has no current context, and the driver answers CUDA_ERROR_INVALID_CONTEXT. One runtime call
// per thread binds the primary context of the current device.
static void bind_context_once() {
  thread_local bool bound = false;
  if (!bound) { cudaFree(nullptr); bound = true; }
}

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  bind_context_once();
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

bool encode_tensor_map_2d(CUtensorMap* map, const void* ptr, int elem_bytes, const uint64_t dims[2], const uint64_t strides[1],
                          const uint32_t box[2], bool swizzle128) {
  auto fn = encode_fn();
  if (!fn) { g_last_encode_error = -1; return false; }
  const cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
  CUresult r = fn(map, dt, 2, const_cast<void*>(ptr), reinterpret_cast<const cuuint64_t*>(dims),
                  reinterpret_cast<const cuuint64_t*>(strides), reinterpret_cast<const cuuint32_t*>(box), estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  g_last_encode_error = static_cast<int>(r);
  return r == CUDA_SUCCESS;
}

bool encode_tensor_map_3d(CUtensorMap* map, const void* ptr, int elem_bytes, const uint64_t dims[3], const uint64_t strides[2],
                          const uint32_t box[3], bool swizzle128) {
  auto fn = encode_fn();
  if (!fn) return false;
  const cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
  CUresult r = fn(map, dt, 3, const_cast<void*>(ptr), reinterpret_cast<const cuuint64_t*>(dims),
                  reinterpret_cast<const cuuint64_t*>(strides), reinterpret_cast<const cuuint32_t*>(box), estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace ghb
