// Token-level sparse attention of one head: dilated window + random + global keys.
//
// Stands in for per_head_attn / sparse_attn of the reference's sparse attention example
// (examples/sparse_attention/sparse_attention.py:24-76):
//   * the first and last n_global tokens attend to each other only,
//       softmax(g_query @ g_key.T) @ g_value                       (lines 57-64)
//   * every other token i attends to the `window` keys ops.shifted_slide(window, dilation)
//     centres on it -- positions i - half + j * dilation, half = (window - 1) * dilation / 2,
//     wrapped the way ShiftedSlide._ids does (x < 0 -> x + S - 1, x >= S -> x - S;
//     kaleido/frontend/operations/fractaltensor/access.py:389-410) -- joined with the keys at
//     the R positions rand_pos[i - n_global]                       (lines 24-38, 51-55, 66-71)
//
// This is gather work bound by memory, not a contraction: per token window + R key rows and as
// many value rows of d elements, nearly all of them L1/L2 hits because neighbouring tokens
// share window rows.  Algorithmic HBM traffic per head is one pass over q, k, v and the output,
// 4 * S * d * element size bytes, plus 4 * R bytes of positions per token.  A group of d / 8
// lanes owns a token (a warp works on 32 / (d / 8) consecutive tokens at a time): lane l of the
// group holds elements [8 l, 8 l + 8) of the query, of each gathered row and of the output; the
// scores are dot products reduced over the group's lanes by shuffles, which every lane of the
// group ends up holding, and the softmax is carried across steps of four keys as (max, sum,
// weighted values).  Rows move as 16-byte loads; the grid is a whole number of CTAs per SM
// striding over (head, token).
//
// `as_shipped`: the example calls ops.softmax(x) without a dimension and the reference's
// softmax normalises dimension 0 by default
// (kaleido/frontend/operations/tensor/arithmetic/reduction.py:26).  On the [1, window + R]
// score row of a windowed token that is a single element, so every weight is 1 and the output
// is the plain sum of the gathered values; on the global block it normalises each key's column
// over the queries.  as_shipped != 0 reproduces that bit of behaviour (it is what the
// reference's frontend returns); 0 normalises over the keys.
#include "../../include/ftb200.h"
#include "ptx.cuh"
#include "tmap.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace ftb {
namespace {

constexpr int kSparseThreads = 256;
constexpr int kMaxKeys = 64;  // window + R, and 2 * n_global

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// EPL elements of a row, owned by one lane, moved as 16-byte (or smaller) vectors.
template <typename T, int EPL>
struct alignas((sizeof(T) * EPL > 16) ? 16 : sizeof(T) * EPL) Frag {
  T v[EPL];
};

template <typename T, int EPL>
__device__ __forceinline__ void load_row(const T* __restrict__ row, int lane, float (&out)[EPL]) {
  const Frag<T, EPL> f = reinterpret_cast<const Frag<T, EPL>*>(row)[lane];
#pragma unroll
  for (int e = 0; e < EPL; ++e) out[e] = to_f32<T>(f.v[e]);
}

// Dot product of two rows spread over the LPT lanes of a token's group; every lane of the group
// gets the sum.  `mask` names the group's lanes, so groups of one warp may diverge.
template <int EPL, int LPT>
__device__ __forceinline__ float group_dot(const float (&a)[EPL], const float (&b)[EPL], unsigned mask) {
  float s = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) s = fmaf(a[e], b[e], s);
#pragma unroll
  for (int o = LPT / 2; o > 0; o >>= 1) s += __shfl_xor_sync(mask, s, o);
  return s;
}

struct SparseArgs {
  long long heads_total;  // B * heads
  int S, window, dilation, n_global, R, as_shipped;
  float scale;
};

constexpr int kEPL = 8;  // elements of a row per lane: 16 bytes of a 16-bit type, 32 of fp32

template <typename T, int LPT>
__global__ void __launch_bounds__(kSparseThreads)
sparse_attn_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                   const int* __restrict__ rand_pos, T* __restrict__ o, SparseArgs a, int* __restrict__ status) {
  constexpr int EPL = kEPL;
  constexpr int d = EPL * LPT;
  constexpr int TPW = 32 / LPT;  // tokens a warp works on at a time, one per group of LPT lanes
  // Keys per step: their key and value rows are all requested before the first score is reduced, so
  // a token costs two dependent memory round trips (positions and query, then the rows).
  constexpr int CH = 4;
  const int lane = threadIdx.x & 31;
  const int gl = lane % LPT;
  const unsigned gmask = LPT == 32 ? 0xffffffffu : (((1u << (LPT & 31)) - 1u) << (lane - gl));
  const long long warp = (static_cast<long long>(blockIdx.x) * kSparseThreads + threadIdx.x) >> 5;
  const long long n_warps = (static_cast<long long>(gridDim.x) * kSparseThreads) >> 5;
  const int S = a.S, ng = a.n_global, G = 2 * a.n_global;
  const int half = (a.window - 1) * a.dilation / 2;
  const long long total = a.heads_total * S;
  const bool small = total <= 0xffffffffLL;

  for (long long first = warp * TPW; first < total; first += n_warps * TPW) {
    const long long item = first + lane / LPT;
    if (item >= total) continue;
    const long long head = small ? static_cast<long long>(static_cast<unsigned>(item) / static_cast<unsigned>(S))
                                 : item / S;
    const int i = static_cast<int>(item - head * S);
    const T* kh = k + head * S * d;
    const T* vh = v + head * S * d;
    const T* qh = q + head * S * d;
    const bool global_tok = i < ng || i >= S - ng;
    const int nk = global_tok ? G : a.window + a.R;
    const int* rp = rand_pos + (head * (S - G) + (i - ng)) * a.R - a.window;  // indexed by key number; read for j >= window only
    const bool use_scores = !a.as_shipped || global_tok;

    float qv[EPL];
    load_row<T, EPL>(qh + static_cast<long long>(i) * d, gl, qv);

    float acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
    float m = -INFINITY, z = 0.f;

    for (int j0 = 0; j0 < nk; j0 += CH) {
      int p[CH];
#pragma unroll
      for (int u = 0; u < CH; ++u) {
        const int j = j0 + u < nk ? j0 + u : nk - 1;  // the tail repeats the last key with weight 0
        int x;
        if (global_tok) {
          x = j < ng ? j : S - G + j;
        } else if (j < a.window) {
          x = i - half + j * a.dilation;
          x = x < 0 ? x + S - 1 : (x >= S ? x - S : x);
        } else {
          x = rp[j];  // the same address in every lane of the group: one broadcast read
          if (x < 0 || x >= S) {
            if (gl == 0) atomicCAS(status, 0, FTB_ERR_INDEX);
            x = 0;
          }
        }
        p[u] = x;
      }
      float kv[CH][EPL], vv[CH][EPL];
      if (use_scores) {
#pragma unroll
        for (int u = 0; u < CH; ++u) load_row<T, EPL>(kh + static_cast<long long>(p[u]) * d, gl, kv[u]);
      }
#pragma unroll
      for (int u = 0; u < CH; ++u) load_row<T, EPL>(vh + static_cast<long long>(p[u]) * d, gl, vv[u]);

      if (!use_scores) {
        // as shipped, windowed token: every weight is 1
#pragma unroll
        for (int u = 0; u < CH; ++u) {
          const float wu = j0 + u < nk ? 1.f : 0.f;
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[e] = fmaf(wu, vv[u][e], acc[e]);
        }
      } else if (a.as_shipped) {
        // as shipped, global token: for key j the weight of query i is exp(s_ij) over the sum of
        // exp(s_i'j) across the global queries i' (a softmax down the column of key j).
#pragma unroll
        for (int u = 0; u < CH; ++u) {
          if (j0 + u >= nk) continue;
          const float s_own = group_dot<EPL, LPT>(qv, kv[u], gmask) * a.scale;
          float cm = -INFINITY, cz = 0.f;
          for (int jj = 0; jj < G; ++jj) {
            float q2[EPL];
            load_row<T, EPL>(qh + static_cast<long long>(jj < ng ? jj : S - G + jj) * d, gl, q2);
            const float s = group_dot<EPL, LPT>(q2, kv[u], gmask) * a.scale;
            const float m2 = fmaxf(cm, s);
            cz = cz * expf(cm - m2) + expf(s - m2);
            cm = m2;
          }
          const float wu = expf(s_own - cm) / cz;
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[e] = fmaf(wu, vv[u][e], acc[e]);
        }
      } else {
        // softmax over the keys, carried across steps as (max, sum, weighted values)
        float sc[CH];
        float m2 = m;
#pragma unroll
        for (int u = 0; u < CH; ++u) {
          const float s = group_dot<EPL, LPT>(qv, kv[u], gmask) * a.scale;  // every lane of the group holds it
          sc[u] = j0 + u < nk ? s : -INFINITY;
          m2 = fmaxf(m2, sc[u]);
        }
        const float keep = expf(m - m2);  // 0 on the first step (m = -inf, m2 finite)
        z *= keep;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] *= keep;
#pragma unroll
        for (int u = 0; u < CH; ++u) {
          const float wu = expf(sc[u] - m2);
          z += wu;
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[e] = fmaf(wu, vv[u][e], acc[e]);
        }
        m = m2;
      }
    }
    const float inv = a.as_shipped ? 1.f : 1.f / z;
    Frag<T, EPL> out;
#pragma unroll
    for (int e = 0; e < EPL; ++e) out.v[e] = from_f32<T>(acc[e] * inv);
    reinterpret_cast<Frag<T, EPL>*>(o + (head * S + i) * d)[gl] = out;
  }
}

template <typename T, int LPT>
int launch_sparse(const void* q, const void* k, const void* v, const int* rand_pos, void* o, const SparseArgs& a,
                  int* status, cudaStream_t stream) {
  const long long warps_needed = (a.heads_total * a.S + 32 / LPT - 1) / (32 / LPT);
  const long long ctas_needed = (warps_needed * 32 + kSparseThreads - 1) / kSparseThreads;
  const long long full = static_cast<long long>(current_sm_count()) * 8;  // 8 CTAs of 256 threads per SM
  const int grid = static_cast<int>(ctas_needed < full ? ctas_needed : full);
  sparse_attn_kernel<T, LPT><<<grid, kSparseThreads, 0, stream>>>(
      static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), rand_pos, static_cast<T*>(o), a,
      status);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
}

template <typename T>
int launch_sparse_d(int d, const void* q, const void* k, const void* v, const int* rand_pos, void* o,
                    const SparseArgs& a, int* status, cudaStream_t stream) {
  switch (d) {
    case 32: return launch_sparse<T, 4>(q, k, v, rand_pos, o, a, status, stream);
    case 64: return launch_sparse<T, 8>(q, k, v, rand_pos, o, a, status, stream);
    case 128: return launch_sparse<T, 16>(q, k, v, rand_pos, o, a, status, stream);
    case 256: return launch_sparse<T, 32>(q, k, v, rand_pos, o, a, status, stream);
    default: return FTB_ERR_ARG;
  }
}

}  // namespace
}  // namespace ftb

using namespace ftb;

extern "C" int ftb_sparse_attn_fwd(const void* q, const void* k, const void* v, const int* rand_pos, void* o, int B,
                                   int heads, int S, int d, int window, int dilation, int n_global, int R,
                                   float scale, int as_shipped, int dtype, void* workspace, size_t workspace_bytes,
                                   void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!q || !k || !v || !o || B < 0 || heads <= 0 || S <= 0 || d <= 0) return FTB_ERR_ARG;
  if (dtype != FTB_F32 && dtype != FTB_F16 && dtype != FTB_BF16) return FTB_ERR_ARG;
  if (window < 1 || window % 2 == 0 || dilation < 1 || n_global < 0 || R < 0) return FTB_ERR_ARG;
  if (R > 0 && S > 2 * n_global && !rand_pos) return FTB_ERR_ARG;
  if (d != 32 && d != 64 && d != 128 && d != 256) return FTB_ERR_ARG;
  const long long half = static_cast<long long>(window - 1) * dilation / 2;
  // The wrap of a window position is a single step: the window must fit in the sequence.
  if (window + R > kMaxKeys || 2 * n_global > kMaxKeys || 2 * n_global > S || half >= S) return FTB_ERR_ARG;
  const uintptr_t all = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                        reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(o);
  if ((all & 15) != 0 || (reinterpret_cast<uintptr_t>(rand_pos) & 3) != 0) return FTB_ERR_ALIGN;
  if (workspace == nullptr || workspace_bytes < ftb_workspace_bytes()) return FTB_ERR_WORKSPACE;
  if (B == 0) return FTB_OK;
  int rc = check_device_sm100();
  if (rc) return rc;
  SparseArgs a;
  a.heads_total = static_cast<long long>(B) * heads;
  a.S = S;
  a.window = window;
  a.dilation = dilation;
  a.n_global = n_global;
  a.R = R;
  a.as_shipped = as_shipped ? 1 : 0;
  a.scale = scale;
  int* status = static_cast<int*>(workspace);  // sticky, as for the other single-kernel entry points
  switch (dtype) {
    case FTB_F32: return launch_sparse_d<float>(d, q, k, v, rand_pos, o, a, status, stream);
    case FTB_F16: return launch_sparse_d<__half>(d, q, k, v, rand_pos, o, a, status, stream);
    default: return launch_sparse_d<__nv_bfloat16>(d, q, k, v, rand_pos, o, a, status, stream);
  }
}
