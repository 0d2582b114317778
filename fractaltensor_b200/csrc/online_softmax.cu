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
// and the rescale (the first 48 K floats of it when it is longer: only the rest is
// read a second time), moves 16 bytes per thread per access, and the grid is a whole
// number of CTAs per SM looping over rows.  Rows of up to 2048 floats take a warp each
// and stay in registers: no block-wide synchronisation at all.
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

template <int THREADS>
__global__ void __launch_bounds__(THREADS)
online_softmax_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int width, int ld,
                      int cache_floats) {
  extern __shared__ float4 row_cache4[];
  float* row_cache = reinterpret_cast<float*>(row_cache4);
  __shared__ float red_m[32], red_d[32];
  __shared__ float final_m, final_d;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cached_floats = width < cache_floats ? width : cache_floats;  // prefix of the row kept on chip
  grid_launch_dependents();
  grid_dependency_wait();  // the kernel before this one (the projection GEMM, say) wrote x
  // 16-byte accesses need rows that start on a 16-byte boundary.
  const bool vec = ((width | ld) & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;

  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* xr = x + static_cast<size_t>(r) * ld;
    float* yr = y + static_cast<size_t>(r) * ld;
    MD s;
    s.m = -FLT_MAX;
    s.d = 0.f;
    if (vec) {
      const float4* x4 = reinterpret_cast<const float4*>(xr);
#pragma unroll 4
      for (int i = tid; i < width / 4; i += THREADS) {
        // The cached part is read once (streamed); the tail is read again by the rescale.
        const bool keep = 4 * i < cached_floats;
        const float4 v = keep ? __ldcs(x4 + i) : x4[i];
        if (keep) row_cache4[i] = v;
        push(s, v.x);
        push(s, v.y);
        push(s, v.z);
        push(s, v.w);
      }
    } else {
      for (int i = tid; i < width; i += THREADS) {
        const float v = xr[i];
        if (i < cached_floats) row_cache[i] = v;
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
      t.m = lane < THREADS / 32 ? red_m[lane] : -FLT_MAX;
      t.d = lane < THREADS / 32 ? red_d[lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
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
      const float4* x4 = reinterpret_cast<const float4*>(xr);
      float4* y4 = reinterpret_cast<float4*>(yr);
#pragma unroll 4
      for (int i = tid; i < width / 4; i += THREADS) {
        float4 v = 4 * i < cached_floats ? row_cache4[i] : __ldcs(x4 + i);
        v.x = exp_fast(fmaxf(v.x - m, kClamp)) * inv_d;
        v.y = exp_fast(fmaxf(v.y - m, kClamp)) * inv_d;
        v.z = exp_fast(fmaxf(v.z - m, kClamp)) * inv_d;
        v.w = exp_fast(fmaxf(v.w - m, kClamp)) * inv_d;
        __stcs(y4 + i, v);
      }
    } else {
      for (int i = tid; i < width; i += THREADS) {
        const float v = i < cached_floats ? row_cache[i] : xr[i];
        yr[i] = exp_fast(fmaxf(v - m, kClamp)) * inv_d;
      }
    }
    __syncthreads();  // the cache and the reduction slots are reused by the next row
  }
}

// Short rows (width % 4 == 0, up to 32 * 4 * kMaxV floats): one warp per row, the row in registers.
constexpr int kMaxV = 16;
__global__ void __launch_bounds__(kSoftmaxThreads)
online_softmax_warp_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int width, int ld) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = kSoftmaxThreads / 32;
  const int n4 = width / 4;
  grid_launch_dependents();
  grid_dependency_wait();
  for (int r = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); r < rows; r += gridDim.x * warps_per_cta) {
    const float4* x4 = reinterpret_cast<const float4*>(x + static_cast<size_t>(r) * ld);
    float4* y4 = reinterpret_cast<float4*>(y + static_cast<size_t>(r) * ld);
    float4 v[kMaxV];
#pragma unroll
    for (int j = 0; j < kMaxV; ++j)
      if (j * 32 + lane < n4) v[j] = __ldcs(x4 + j * 32 + lane);
    MD s;
    s.m = -FLT_MAX;
    s.d = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxV; ++j)
      if (j * 32 + lane < n4) {
        push(s, v[j].x);
        push(s, v[j].y);
        push(s, v[j].z);
        push(s, v[j].w);
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MD t;
      t.m = __shfl_xor_sync(0xffffffffu, s.m, o);
      t.d = __shfl_xor_sync(0xffffffffu, s.d, o);
      s = merge(s, t);
    }
    const float m = s.m, inv_d = 1.f / s.d;
#pragma unroll
    for (int j = 0; j < kMaxV; ++j)
      if (j * 32 + lane < n4) {
        float4 o4;
        o4.x = exp_fast(fmaxf(v[j].x - m, kClamp)) * inv_d;
        o4.y = exp_fast(fmaxf(v[j].y - m, kClamp)) * inv_d;
        o4.z = exp_fast(fmaxf(v[j].z - m, kClamp)) * inv_d;
        o4.w = exp_fast(fmaxf(v[j].w - m, kClamp)) * inv_d;
        __stcs(y4 + j * 32 + lane, o4);
      }
  }
}

}  // namespace
}  // namespace ftb

using namespace ftb;

namespace ftb {
// Softmax over the first `width` floats of each row of x (rows `ld` floats apart), written to the
// same positions of y; x == y is allowed when a row fits the on-chip cache (width <= 48 K floats).
int online_softmax_rows(const float* x, float* y, int rows, int width, int ld, cudaStream_t stream) {
  if (!x || !y || rows <= 0 || width <= 0 || ld < width) return FTB_ERR_ARG;
  if (static_cast<int64_t>(rows) * ld > 0x7fffffffffLL) return FTB_ERR_ARG;
  int rc = check_device_sm100();
  if (rc) return rc;
  const bool aligned16 = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (aligned16 && ((width | ld) & 3) == 0 && width <= 32 * 4 * kMaxV && rows >= 8) {
    const int64_t ctas = (static_cast<int64_t>(rows) + kSoftmaxThreads / 32 - 1) / (kSoftmaxThreads / 32);
    const int64_t full = static_cast<int64_t>(current_sm_count()) * 4;
    const cudaError_t err = launch_light(online_softmax_warp_kernel, dim3(static_cast<int>(ctas < full ? ctas : full)),
                                             dim3(kSoftmaxThreads), 0, stream, x, y, rows, width, ld);
    count_launch();
    if (err != cudaSuccess) cudaGetLastError();
    return err == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
  }
  // Row cache: the row, or its first 48 K floats, in up to 192 KB of shared memory.
  constexpr int kMaxCacheFloats = 48 * 1024;
  if (x == y && width > kMaxCacheFloats) return FTB_ERR_ARG;
  const int cache_floats = width <= kMaxCacheFloats ? ((width + 3) & ~3) : kMaxCacheFloats;
  const size_t smem = static_cast<size_t>(cache_floats) * sizeof(float);
  static std::atomic<unsigned long long> configured_a{0}, configured_b{0};
  if (!ensure_dynamic_smem(online_softmax_kernel<kSoftmaxThreads>, kMaxCacheFloats * static_cast<int>(sizeof(float)),
                           configured_a) ||
      !ensure_dynamic_smem(online_softmax_kernel<1024>, kMaxCacheFloats * static_cast<int>(sizeof(float)),
                           configured_b))
    return FTB_ERR_LAUNCH;
  // A whole number of CTAs per SM: as many as the row cache lets be resident (at most 8).  A cache
  // that leaves room for one or two CTAs per SM gets CTAs of 1024 threads to keep loads in flight.
  int per_sm = static_cast<int>((200 * 1024) / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
  const int64_t want = static_cast<int64_t>(current_sm_count()) * per_sm;
  const int grid = static_cast<int>(rows < want ? rows : want);
  cudaError_t err;
  if (per_sm <= 2)
    err = launch_light(online_softmax_kernel<1024>, dim3(grid), dim3(1024), smem, stream, x, y, rows, width, ld,
                           cache_floats);
  else
    err = launch_light(online_softmax_kernel<kSoftmaxThreads>, dim3(grid), dim3(kSoftmaxThreads), smem, stream, x, y,
                           rows, width, ld, cache_floats);
  count_launch();
  if (err != cudaSuccess) cudaGetLastError();
  return err == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
}
}  // namespace ftb

extern "C" int ftb_online_softmax(const float* x, float* y, int rows, int width, void* stream_) {
  return ftb::online_softmax_rows(x, y, rows, width, width, static_cast<cudaStream_t>(stream_));
}
