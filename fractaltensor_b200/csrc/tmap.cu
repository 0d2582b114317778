#include "tmap.h"

#include <atomic>
#include <mutex>

#include "ptx.cuh"

namespace ftb {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

CUtensorMapDataType tmap_dtype(int dt) {
  switch (dt) {
    case FTB_F32: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    case FTB_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  }
}
}  // namespace

int make_tmap_2d(CUtensorMap* out, const void* base, int dtype, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return FTB_ERR_DRIVER;
  const size_t es = dtype_size(dtype);
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * es) & 15)) return FTB_ERR_ALIGN;
  if (box_rows > 256 || box_cols > 256 || (swizzle128 && box_cols * es > 128)) return FTB_ERR_ARG;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * es};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, tmap_dtype(dtype), 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FTB_OK : FTB_ERR_DRIVER;
}

int make_tmap_3d(CUtensorMap* out, const void* base, int dtype, uint64_t cols, uint64_t rows, uint64_t planes,
                 uint64_t row_stride_bytes, uint64_t plane_stride_bytes, uint32_t box_cols, uint32_t box_rows,
                 uint32_t box_planes, bool swizzle128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return FTB_ERR_DRIVER;
  const size_t es = dtype_size(dtype);
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15) || (plane_stride_bytes & 15))
    return FTB_ERR_ALIGN;
  if (box_rows > 256 || box_cols > 256 || box_planes > 256 || (swizzle128 && box_cols * es > 128))
    return FTB_ERR_ARG;
  cuuint64_t dims[3] = {cols, rows, planes};
  cuuint64_t strides[2] = {row_stride_bytes, plane_stride_bytes};
  cuuint32_t box[3] = {box_cols, box_rows, box_planes};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, tmap_dtype(dtype), 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FTB_OK : FTB_ERR_DRIVER;
}

int check_device_sm100() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return FTB_ERR_ARCH;
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return FTB_ERR_ARCH;
  return major == 10 ? FTB_OK : FTB_ERR_ARCH;
}

namespace {
std::atomic<long long> g_launches{0};
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches_so_far() { return g_launches.load(std::memory_order_relaxed); }

int current_sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return n;
}

}  // namespace ftb
