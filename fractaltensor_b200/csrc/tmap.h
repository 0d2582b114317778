// Host-side helpers shared by the C-ABI entry points: TMA tensor-map encoding
// (through a driver entry point looked up at run time, so the library links
// against the CUDA runtime only and still loads on a machine without a GPU
// driver), device checks and small argument checks.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>

namespace ftb {

enum DType : int { FTB_F32 = 0, FTB_F16 = 1, FTB_BF16 = 2 };

inline size_t dtype_size(int dt) { return dt == FTB_F32 ? 4 : 2; }

// Encodes a row-major [rows, cols] matrix (row stride `ld` elements) as a 2-D
// tiled tensor map with box [box_rows, box_cols] and 128-byte swizzle; box_cols
// times the element size must be 128 bytes or less.  Returns 0 on success.
int make_tmap_2d(CUtensorMap* out, const void* base, int dtype, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols, bool swizzle128 = true);

// 3-D variant: dims (cols, rows, planes) with byte strides for rows and planes.
int make_tmap_3d(CUtensorMap* out, const void* base, int dtype, uint64_t cols, uint64_t rows, uint64_t planes,
                 uint64_t row_stride_bytes, uint64_t plane_stride_bytes, uint32_t box_cols, uint32_t box_rows,
                 uint32_t box_planes, bool swizzle128 = true);

// 0 when the current device is compute capability 10.x, else FTB_ERR_ARCH.
int check_device_sm100();

int current_sm_count();

// Opt-in to more than 48 KB of dynamic shared memory for kernel `kfn` on the CURRENT device.
// The attribute belongs to each device's copy of the kernel, so `configured` (one static per
// kernel instantiation) keeps one bit per device ordinal; devices past 63 are set up on every call.
// Safe to call from several host threads.  Returns false when the runtime refuses.
template <typename Kernel>
inline bool ensure_dynamic_smem(Kernel kfn, int bytes, std::atomic<unsigned long long>& configured) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return false;
  const unsigned long long bit = dev < 64 ? (1ull << dev) : 0ull;
  if (bit != 0 && (configured.load(std::memory_order_acquire) & bit) != 0) return true;
  if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  configured.fetch_or(bit, std::memory_order_release);
  return true;
}

// Launches `kfn` so that it may start while the kernel before it in the stream is still draining
// (programmatic dependent launch): its CTAs are scheduled as SMs free up and run their set-up
// (barriers, tensor memory, descriptor prefetch) early.  The kernel must execute
// `griddepcontrol.wait` before its first access to global memory; that instruction returns once
// the kernel before it has completed and its writes are visible.  Behind a kernel that never
// signals, or as the first kernel of a stream, this is an ordinary launch.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kfn)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kfn, static_cast<KArgs>(args)...);
}

#ifndef FTB_LIGHT_DEPENDENT
#define FTB_LIGHT_DEPENDENT 1
#endif
// The same for kernels with next to no set-up (row-wise kernels).  Measured against plain launches:
// attention RNN 1.16 against 1.22 ms, online softmax 88 against 91 us, embedding lookup equal,
// projection + softmax 65 against 62 us; -DFTB_LIGHT_DEPENDENT=0 builds them as plain launches.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_light(void (*kfn)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = FTB_LIGHT_DEPENDENT;
  return cudaLaunchKernelEx(&cfg, kfn, static_cast<KArgs>(args)...);
}

// Process-wide count of kernels this library has launched (reported by ftb_launch_count()).
void count_launch(int n = 1);
long long launches_so_far();

}  // namespace ftb
