// Row-wise softmax of an fp32 matrix with the online (maximum, normaliser) reduction.
//
// Stands in for KeOnlineNormalizedSoftMax / OnlineNormalizedSoftmaxOp
// (kaleido/core/device/kernels/online_softmax.h:15-183,
// kaleido/core/operators/online_softmax_op.cu:13-38): every row keeps a running
// pair (m, d) = (maximum so far, sum of e^(x - m) so far); two pairs merge as
// d = d1 e^(m1 - m) + d2 e^(m2 - m) with m = max(m1, m2); the output is
// e^(max(x - m, -64)) / d, the reference's clamp included.
//
// The op is HBM-bound (8 bytes per element when the input is read once), so the
// kernel is organised around one global read and one global write per element:
// a CTA owns a row at a time, keeps it in shared memory between the reduction
// and the rescale when it fits, moves 16 bytes per thread per access, and the
// grid is a whole number of CTAs per SM looping over rows.  Rows that do not fit
// in shared memory are read a second time (from L2 when the row is smaller than it).
#include <cfloat>

#include "../../include/ftb200.h"
#include "ptx.cuh"
#include "tmap.h"

namespace ftb {
namespace {

constexpr int kSoftmaxThreads = 256;
constexpr float kClamp = -64.f;
constexpr float kLog2e = 1.4426950408889634f;

struct MD {
  float m, d;
};

__device__ __forceinline__ float exp_fast(float x) { return exp2_fast(x * kLog2e); }

// (m, d) of the union of two sets of elements.
__device__ __forceinline__ MD merge(MD a, MD b) {
  const float m = fmaxf(a.m, b.m);
  MD r;
  r.m = m;
  r.d = a.d * exp_fast(a.m - m) + b.d * exp_fast(b.m - m);
  return r;
}

__device__ __forceinline__ void push(MD& s, float v) {
  // One exponential per element whichever way the maximum moves.
  const float m = fmaxf(s.m, v);
  const float e = exp_fast(fminf(s.m, v) - m);
  s.d = v > s.m ? fmaf(s.d, e, 1.f) : s.d + e;
  s.m = m;
}

__global__ void __launch_bounds__(kSoftmaxThreads)
online_softmax_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int width, int cache_floats) {
  extern __shared__ float4 row_cache4[];
  float* row_cache = reinterpret_cast<float*>(row_cache4);
  __shared__ float red_m[kSoftmaxThreads / 32], red_d[kSoftmaxThreads / 32];
  __shared__ float final_m, final_d;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool cached = width <= cache_floats;
  // 16-byte accesses need rows that start on a 16-byte boundary.
  const bool vec = (width & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;

  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* xr = x + static_cast<size_t>(r) * width;
    float* yr = y + static_cast<size_t>(r) * width;
    MD s;
    s.m = -FLT_MAX;
    s.d = 0.f;
    if (vec) {
      const float4* x4 = reinterpret_cast<const float4*>(xr);
      for (int i = tid; i < width / 4; i += kSoftmaxThreads) {
        const float4 v = __ldcs(x4 + i);  // streamed: read once
        if (cached) row_cache4[i] = v;
        push(s, v.x);
        push(s, v.y);
        push(s, v.z);
        push(s, v.w);
      }
    } else {
      for (int i = tid; i < width; i += kSoftmaxThreads) {
        const float v = xr[i];
        if (cached) row_cache[i] = v;
        push(s, v);
      }
    }
    // Threads that saw no element hold (-FLT_MAX, 0): neutral in a merge.
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MD t;
      t.m = __shfl_xor_sync(0xffffffffu, s.m, o);
      t.d = __shfl_xor_sync(0xffffffffu, s.d, o);
      s = merge(s, t);
    }
    if (lane == 0) {
      red_m[warp] = s.m;
      red_d[warp] = s.d;
    }
    __syncthreads();
    if (warp == 0) {
      MD t;
      t.m = lane < kSoftmaxThreads / 32 ? red_m[lane] : -FLT_MAX;
      t.d = lane < kSoftmaxThreads / 32 ? red_d[lane] : 0.f;
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {
        MD u;
        u.m = __shfl_xor_sync(0xffffffffu, t.m, o);
        u.d = __shfl_xor_sync(0xffffffffu, t.d, o);
        t = merge(t, u);
      }
      if (lane == 0) {
        final_m = t.m;
        final_d = t.d;
      }
    }
    __syncthreads();
    const float m = final_m;
    const float inv_d = 1.f / final_d;
    if (vec) {
      const float4* src = cached ? row_cache4 : reinterpret_cast<const float4*>(xr);
      float4* y4 = reinterpret_cast<float4*>(yr);
      for (int i = tid; i < width / 4; i += kSoftmaxThreads) {
        float4 v = src[i];
        v.x = exp_fast(fmaxf(v.x - m, kClamp)) * inv_d;
        v.y = exp_fast(fmaxf(v.y - m, kClamp)) * inv_d;
        v.z = exp_fast(fmaxf(v.z - m, kClamp)) * inv_d;
        v.w = exp_fast(fmaxf(v.w - m, kClamp)) * inv_d;
        __stcs(y4 + i, v);
      }
    } else {
      const float* src = cached ? row_cache : xr;
      for (int i = tid; i < width; i += kSoftmaxThreads) yr[i] = exp_fast(fmaxf(src[i] - m, kClamp)) * inv_d;
    }
    __syncthreads();  // the cache and the reduction slots are reused by the next row
  }
}

}  // namespace
}  // namespace ftb

using namespace ftb;

extern "C" int ftb_online_softmax(const float* x, float* y, int rows, int width, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!x || !y || rows <= 0 || width <= 0) return FTB_ERR_ARG;
  if (static_cast<int64_t>(rows) * width > 0x7fffffffffLL) return FTB_ERR_ARG;
  int rc = check_device_sm100();
  if (rc) return rc;
  // Row cache: the whole row when it fits in 192 KB of shared memory, else none.
  constexpr int kMaxCacheFloats = 48 * 1024;
  const int cache_floats = width <= kMaxCacheFloats ? ((width + 3) & ~3) : 0;
  const size_t smem = static_cast<size_t>(cache_floats) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(online_softmax_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kMaxCacheFloats * static_cast<int>(sizeof(float))) != cudaSuccess)
      return FTB_ERR_LAUNCH;
    configured = true;
  }
  // A whole number of CTAs per SM: as many as the row cache lets be resident (at most 8).
  int per_sm = smem == 0 ? 8 : static_cast<int>((200 * 1024) / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
  const int64_t want = static_cast<int64_t>(current_sm_count()) * per_sm;
  const int grid = static_cast<int>(rows < want ? rows : want);
  online_softmax_kernel<<<grid, kSoftmaxThreads, smem, stream>>>(x, y, rows, width, cache_floats);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
}
