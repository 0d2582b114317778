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
// This is gather work bound by memory, not a contraction.  Algorithmic HBM traffic per head is one
// pass over q, k, v and the output, 4 * S * d * element size bytes, plus 4 * R bytes of positions
// per token.
//
// A group of d / 8 lanes owns a token (a warp works on 32 / (d / 8) tokens at a time): each lane
// holds 8 elements of the query, of each gathered row and of the output; the scores are dot
// products reduced over the group's lanes by shuffles, which every lane of the group ends up
// holding, and the softmax is carried across steps of four keys as (max, sum, weighted values).
//
// Tiled kernel (the default): a persistent CTA walks tiles of TT consecutive tokens of one head.
// The key and value rows the tile's windows can touch, positions [t0 - half, t0 + TT + half), are
// contiguous in memory, and so are the tile's queries: three bulk asynchronous copies bring them
// into shared memory under an mbarrier, for the next tile while the current one is computed (two
// stages).  The tile's random positions are fetched into registers one tile ahead and parked in
// shared memory.  Window rows, queries and positions then cost shared-memory latency; only the R
// random rows per token (and window positions that wrap around the ends of the sequence) are
// gathered from global memory, 16 bytes per lane.
// With the example's key counts (window 5, 3 random keys) the interior tiles -- no global token,
// no window position that wraps -- go through a routine with those counts at compile time: all
// eight scores in registers, one softmax, no per-key bookkeeping (16.7 M warp instructions instead
// of 29 M at the example's size).  Every CTA first walks its share of the edge tiles of all heads
// with the general routine, then its share of the interior tiles.
// Direct kernel (fallback when a tile does not fit in shared memory or R > 16): the general token
// routine with every row gathered from global memory.
//
// `as_shipped`: the example calls ops.softmax(x) without a dimension and the reference's softmax
// normalises dimension 0 by default
// (kaleido/frontend/operations/tensor/arithmetic/reduction.py:26).  On the [1, window + R] score
// row of a windowed token that is a single element, so every weight is 1 and the output is the
// plain sum of the gathered values; on the global block it normalises each key's column over the
// queries.  as_shipped != 0 reproduces that (it is what the reference's frontend returns);
// 0 normalises over the keys.
#include "../../include/ftb200.h"
#include "ptx.cuh"
#include "tmap.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace ftb {
namespace {

constexpr int kSparseThreads = 256;
constexpr int kMaxKeys = 64;    // window + R, and 2 * n_global
constexpr int kEPL = 8;         // elements of a row per lane
constexpr int kCH = 4;          // keys per step: their rows are all requested before the first score is reduced
constexpr int kPosRegs = 4;     // tiled kernel: random positions of the next tile held per thread
constexpr int kMaxTileSmem = 110 * 1024;  // two stages; leaves room for two CTAs per SM

// 8 elements of a row owned by lane `gl` of a group of LPT lanes, moved as 16-byte pieces: piece c
// of the lane is the 16 bytes at (c * LPT + gl) * 16, so that one load instruction of the group
// covers a contiguous stretch of the row.
template <typename T> struct Pieces { static constexpr int n = sizeof(T) * kEPL / 16; };

__device__ __forceinline__ void unpack16(const uint4& w, float* out, float) {
  out[0] = __uint_as_float(w.x);
  out[1] = __uint_as_float(w.y);
  out[2] = __uint_as_float(w.z);
  out[3] = __uint_as_float(w.w);
}
__device__ __forceinline__ void unpack16(const uint4& w, float* out, __half) {
  const uint32_t r[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&r[i]));
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void unpack16(const uint4& w, float* out, __nv_bfloat16) {
  const uint32_t r[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(r[i] << 16);
    out[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack16(const float* in, float) {
  return make_uint4(__float_as_uint(in[0]), __float_as_uint(in[1]), __float_as_uint(in[2]), __float_as_uint(in[3]));
}
__device__ __forceinline__ uint4 pack16(const float* in, __half) {
  uint32_t r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
    r[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(r[0], r[1], r[2], r[3]);
}
__device__ __forceinline__ uint4 pack16(const float* in, __nv_bfloat16) {
  uint32_t r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
    r[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(r[0], r[1], r[2], r[3]);
}

template <typename T, int LPT>
__device__ __forceinline__ void load_row_global(const T* __restrict__ row, int gl, float (&out)[kEPL]) {
#pragma unroll
  for (int c = 0; c < Pieces<T>::n; ++c) {
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(row) + c * LPT + gl);
    unpack16(w, out + c * (kEPL / Pieces<T>::n), T());
  }
}
template <typename T, int LPT>
__device__ __forceinline__ void load_row_shared(const T* row, int gl, float (&out)[kEPL]) {
#pragma unroll
  for (int c = 0; c < Pieces<T>::n; ++c) {
    uint4 w;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                 : "r"(smem_u32(reinterpret_cast<const uint4*>(row) + c * LPT + gl)));
    unpack16(w, out + c * (kEPL / Pieces<T>::n), T());
  }
}
template <typename T, int LPT>
__device__ __forceinline__ void store_row_global(T* row, int gl, const float (&in)[kEPL]) {
#pragma unroll
  for (int c = 0; c < Pieces<T>::n; ++c)
    __stcs(reinterpret_cast<uint4*>(row) + c * LPT + gl, pack16(in + c * (kEPL / Pieces<T>::n), T()));
}

// Dot product of two rows spread over the LPT lanes of a token's group; every lane of the group
// gets the sum.  `mask` names the group's lanes, so groups of one warp may diverge.
template <int LPT>
__device__ __forceinline__ float group_dot(const float (&a)[kEPL], const float (&b)[kEPL], unsigned mask) {
  float s = 0.f;
#pragma unroll
  for (int e = 0; e < kEPL; ++e) s = fmaf(a[e], b[e], s);
#pragma unroll
  for (int o = LPT / 2; o > 0; o >>= 1) s += __shfl_xor_sync(mask, s, o);
  return s;
}

__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

struct SparseArgs {
  long long heads_total;  // B * heads
  int S, window, dilation, n_global, R, as_shipped;
  float scale;
  // tiled kernel
  int TT;              // tokens per tile
  int tiles_per_head;  // ceil(S / TT)
  int stage_bytes;     // K rows | V rows | queries | positions of one stage
  // Which tiles of a head a launch of the tiled kernel walks: `per_head` of them, the idx-th being
  // tile idx (idx < lead), else tile idx + skip.  All tiles: per_head = tiles_per_head, lead = 0,
  // skip = 0.  Interior tiles only (no global token, no wrapped window position): lead = 0,
  // skip = leading edge tiles.  Edge tiles only: lead = leading edge tiles, skip = interior tiles.
  int per_head, lead, skip;
  // A launch that walks interior and edge tiles with different routines: the edge enumeration
  // (the one above is then the interior one).
  int edge_per_head, edge_lead, edge_skip;
};

// Where the rows of one token's head come from: global memory, and for the tiled kernel the stage
// that holds rows [lo, hi) of K and V.
template <typename T>
struct Rows {
  const T* kh;  // the head's keys, values, queries in global memory
  const T* vh;
  const T* qh;
  const T* sk;  // shared memory (tiled kernel): key / value rows lo .. hi - 1
  const T* sv;
  int lo, hi;   // lo = hi = 0 for the direct kernel
};

// One token: query row `qv` already loaded, `pos_of(r)` gives the position of random key r.
// `interior` (tiled kernel, the same for every token of a tile): no token of the tile is a global
// one and no window position wraps, so window rows are in the stage and random rows are gathered
// from global memory -- which of the two a key is then depends on its number only, and the warp
// does not diverge over it.
template <typename T, int LPT, typename PosFn>
__device__ __forceinline__ void attend_token(const SparseArgs& a, const Rows<T>& rw, int i, int gl, unsigned gmask,
                                             bool interior,
                                             const float (&qv)[kEPL], PosFn pos_of, T* __restrict__ out_row,
                                             int* __restrict__ status) {
  constexpr int d = kEPL * LPT;
  constexpr int CH = kCH;
  const int S = a.S, ng = a.n_global, G = 2 * a.n_global;
  const int half = (a.window - 1) * a.dilation / 2;
  const bool global_tok = i < ng || i >= S - ng;
  const int nk = global_tok ? G : a.window + a.R;
  const bool use_scores = !a.as_shipped || global_tok;
  const float scale2 = a.scale * 1.4426950408889634f;  // scores in the base-2 domain: exp(x) = 2^(x log2 e)

  float acc[kEPL];
#pragma unroll
  for (int e = 0; e < kEPL; ++e) acc[e] = 0.f;
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
        x = pos_of(j - a.window);
        if (x < 0 || x >= S) {
          if (gl == 0) atomicCAS(status, 0, FTB_ERR_INDEX);
          x = 0;
        }
      }
      p[u] = x;
    }
    float kv[CH][kEPL], vv[CH][kEPL];
#pragma unroll
    for (int u = 0; u < CH; ++u) {
      const bool staged = interior ? ((j0 + u < nk ? j0 + u : nk - 1) < a.window) : (p[u] >= rw.lo && p[u] < rw.hi);
      if (staged) {
        if (use_scores) load_row_shared<T, LPT>(rw.sk + (p[u] - rw.lo) * d, gl, kv[u]);
        load_row_shared<T, LPT>(rw.sv + (p[u] - rw.lo) * d, gl, vv[u]);
      } else {
        if (use_scores) load_row_global<T, LPT>(rw.kh + static_cast<long long>(p[u]) * d, gl, kv[u]);
        load_row_global<T, LPT>(rw.vh + static_cast<long long>(p[u]) * d, gl, vv[u]);
      }
    }

    if (!use_scores) {
      // as shipped, windowed token: every weight is 1
#pragma unroll
      for (int u = 0; u < CH; ++u) {
        const float wu = j0 + u < nk ? 1.f : 0.f;
#pragma unroll
        for (int e = 0; e < kEPL; ++e) acc[e] = fmaf(wu, vv[u][e], acc[e]);
      }
    } else if (a.as_shipped) {
      // as shipped, global token: for key j the weight of query i is exp(s_ij) over the sum of
      // exp(s_i'j) across the global queries i' (a softmax down the column of key j).
#pragma unroll
      for (int u = 0; u < CH; ++u) {
        if (j0 + u >= nk) continue;
        const float s_own = group_dot<LPT>(qv, kv[u], gmask) * a.scale;
        float cm = -INFINITY, cz = 0.f;
        for (int jj = 0; jj < G; ++jj) {
          float q2[kEPL];
          load_row_global<T, LPT>(rw.qh + static_cast<long long>(jj < ng ? jj : S - G + jj) * d, gl, q2);
          const float s = group_dot<LPT>(q2, kv[u], gmask) * a.scale;
          const float m2 = fmaxf(cm, s);
          cz = cz * expf(cm - m2) + expf(s - m2);
          cm = m2;
        }
        const float wu = expf(s_own - cm) / cz;
#pragma unroll
        for (int e = 0; e < kEPL; ++e) acc[e] = fmaf(wu, vv[u][e], acc[e]);
      }
    } else {
      // softmax over the keys, carried across steps as (max, sum, weighted values)
      float sc[CH];
      float m2 = m;
#pragma unroll
      for (int u = 0; u < CH; ++u) {
        const float s = group_dot<LPT>(qv, kv[u], gmask) * scale2;  // every lane of the group holds it
        sc[u] = j0 + u < nk ? s : -INFINITY;
        m2 = fmaxf(m2, sc[u]);
      }
      const float keep = exp2_fast(m - m2);  // 0 on the first step (m = -inf, m2 finite)
      z *= keep;
#pragma unroll
      for (int e = 0; e < kEPL; ++e) acc[e] *= keep;
#pragma unroll
      for (int u = 0; u < CH; ++u) {
        const float wu = exp2_fast(sc[u] - m2);
        z += wu;
#pragma unroll
        for (int e = 0; e < kEPL; ++e) acc[e] = fmaf(wu, vv[u][e], acc[e]);
      }
      m = m2;
    }
  }
  const float inv = a.as_shipped ? 1.f : 1.f / z;
#pragma unroll
  for (int e = 0; e < kEPL; ++e) acc[e] *= inv;
  store_row_global<T, LPT>(out_row, gl, acc);
}

// One token of an interior tile with the numbers of window and random keys known at compile time
// (the example's 5 and 3): no per-key bookkeeping, one softmax over the KW + KR scores.  Window rows
// come from the stage, random rows from global memory; the random rows of K and V are requested
// first, so that they arrive while the window part is computed out of shared memory.
template <typename T, int LPT, int KW, int KR>
__device__ __forceinline__ void attend_fast(const SparseArgs& a, const T* sk, const T* sv, int lo, const T* kh,
                                            const T* vh, int i, int gl, unsigned gmask, const float (&qv)[kEPL],
                                            const int* sp, T* __restrict__ out_row, int* __restrict__ status) {
  constexpr int d = kEPL * LPT;
  const int half = (KW - 1) * a.dilation / 2;
  const float scale2 = a.scale * 1.4426950408889634f;
  float kr[KR][kEPL], vr[KR][kEPL];
#pragma unroll
  for (int r = 0; r < KR; ++r) {
    int x = sp[r];
    if (x < 0 || x >= a.S) {
      if (gl == 0) atomicCAS(status, 0, FTB_ERR_INDEX);
      x = 0;
    }
    load_row_global<T, LPT>(kh + static_cast<long long>(x) * d, gl, kr[r]);
    load_row_global<T, LPT>(vh + static_cast<long long>(x) * d, gl, vr[r]);
  }
  float sc[KW + KR];
  const int row0 = i - half - lo;  // the first window row inside the stage
#pragma unroll
  for (int j = 0; j < KW; ++j) {
    float kw[kEPL];
    load_row_shared<T, LPT>(sk + (row0 + j * a.dilation) * d, gl, kw);
    sc[j] = group_dot<LPT>(qv, kw, gmask) * scale2;
  }
#pragma unroll
  for (int r = 0; r < KR; ++r) sc[KW + r] = group_dot<LPT>(qv, kr[r], gmask) * scale2;
  float m = sc[0];
#pragma unroll
  for (int j = 1; j < KW + KR; ++j) m = fmaxf(m, sc[j]);
  float z = 0.f;
#pragma unroll
  for (int j = 0; j < KW + KR; ++j) {
    sc[j] = exp2_fast(sc[j] - m);
    z += sc[j];
  }
  float acc[kEPL];
#pragma unroll
  for (int e = 0; e < kEPL; ++e) acc[e] = 0.f;
#pragma unroll
  for (int j = 0; j < KW; ++j) {
    float vw[kEPL];
    load_row_shared<T, LPT>(sv + (row0 + j * a.dilation) * d, gl, vw);
#pragma unroll
    for (int e = 0; e < kEPL; ++e) acc[e] = fmaf(sc[j], vw[e], acc[e]);
  }
#pragma unroll
  for (int r = 0; r < KR; ++r) {
#pragma unroll
    for (int e = 0; e < kEPL; ++e) acc[e] = fmaf(sc[KW + r], vr[r][e], acc[e]);
  }
  const float inv = 1.f / z;
#pragma unroll
  for (int e = 0; e < kEPL; ++e) acc[e] *= inv;
  store_row_global<T, LPT>(out_row, gl, acc);
}

template <int LPT>
__device__ __forceinline__ unsigned group_mask(int lane) {
  return LPT == 32 ? 0xffffffffu : (((1u << (LPT & 31)) - 1u) << (lane - lane % LPT));
}

// ------------------------------------------------------------------ direct kernel
template <typename T, int LPT>
__global__ void __launch_bounds__(kSparseThreads)
sparse_attn_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                   const int* __restrict__ rand_pos, T* __restrict__ o, SparseArgs a, int* __restrict__ status) {
  constexpr int d = kEPL * LPT;
  constexpr int TPW = 32 / LPT;  // tokens a warp works on at a time, one per group of LPT lanes
  const int lane = threadIdx.x & 31;
  const int gl = lane % LPT;
  const unsigned gmask = group_mask<LPT>(lane);
  const long long warp = (static_cast<long long>(blockIdx.x) * kSparseThreads + threadIdx.x) >> 5;
  const long long n_warps = (static_cast<long long>(gridDim.x) * kSparseThreads) >> 5;
  const int S = a.S, ng = a.n_global, G = 2 * a.n_global;
  const long long total = a.heads_total * S;
  const bool small = total <= 0xffffffffLL;
  grid_launch_dependents();
  grid_dependency_wait();

  for (long long first = warp * TPW; first < total; first += n_warps * TPW) {
    const long long item = first + lane / LPT;
    if (item >= total) continue;
    const long long head = small ? static_cast<long long>(static_cast<unsigned>(item) / static_cast<unsigned>(S))
                                 : item / S;
    const int i = static_cast<int>(item - head * S);
    Rows<T> rw;
    rw.kh = k + head * S * d;
    rw.vh = v + head * S * d;
    rw.qh = q + head * S * d;
    rw.sk = rw.sv = nullptr;
    rw.lo = rw.hi = 0;
    const int* rp = rand_pos + (head * (S - G) + (i - ng)) * a.R;  // read for windowed tokens only
    float qv[kEPL];
    load_row_global<T, LPT>(rw.qh + static_cast<long long>(i) * d, gl, qv);
    attend_token<T, LPT>(a, rw, i, gl, gmask, false, qv, [&](int r) { return __ldg(rp + r); },
                         o + (head * S + i) * d, status);
  }
}

// ------------------------------------------------------------------ tiled kernel
// The walk of one CTA over its work items: item number first, first + step, ... of the enumeration
// (per_head, lead, skip).  it_base = tiles the CTA has walked before (the stages and barrier phases
// carry on from there); returns that count plus the tiles of this walk, or -1 after a wait ran out.  KW > 0: the items are interior tiles and a token has KW window and KR
// random keys (attend_fast); KW = 0: any tile, any key counts (attend_token).
template <typename T, int LPT, int KW, int KR>
__device__ __forceinline__ int walk_tiles(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                          const int* __restrict__ rand_pos, T* __restrict__ o, const SparseArgs& a,
                                          int per_head, int lead, int skip, long long first, long long step,
                                          int it_base, unsigned char* smem, uint64_t* full, int* s_abort_p,
                                          int* __restrict__ status) {
  constexpr int d = kEPL * LPT;
  constexpr int TPW = 32 / LPT;
  volatile int* s_abort = s_abort_p;

  const int tid = threadIdx.x, lane = tid & 31, gl = lane % LPT;
  const unsigned gmask = group_mask<LPT>(lane);
  const int S = a.S, ng = a.n_global, G = 2 * a.n_global, TT = a.TT;
  const int half = (a.window - 1) * a.dilation / 2;
  const int rows_max = TT + 2 * half;
  const long long n_tiles = a.heads_total * per_head;  // work items of this enumeration

  auto stage_k = [&](int s) { return reinterpret_cast<T*>(smem + static_cast<size_t>(s) * a.stage_bytes); };
  auto stage_v = [&](int s) { return stage_k(s) + static_cast<size_t>(rows_max) * d; };
  auto stage_q = [&](int s) { return stage_v(s) + static_cast<size_t>(rows_max) * d; };
  auto stage_pos = [&](int s) { return reinterpret_cast<int*>(stage_q(s) + static_cast<size_t>(TT) * d); };

  struct Tile {
    long long head;
    int t0, nt, lo, hi;
  };
  auto tile_of = [&](long long t) {
    Tile x;
    x.head = t / per_head;
    const int idx = static_cast<int>(t - x.head * per_head);
    x.t0 = (idx < lead ? idx : idx + skip) * TT;
    x.nt = min(TT, S - x.t0);
    x.lo = max(0, x.t0 - half);
    x.hi = min(S, x.t0 + x.nt + half);
    return x;
  };
  // Thread 0: the three bulk copies of a tile into stage s.
  auto issue = [&](const Tile& x, int s) {
    const uint32_t kv_bytes = static_cast<uint32_t>(x.hi - x.lo) * d * sizeof(T);
    const uint32_t q_bytes = static_cast<uint32_t>(x.nt) * d * sizeof(T);
    mbar_arrive_expect_tx(&full[s], 2 * kv_bytes + q_bytes);
    bulk_load_1d(stage_k(s), k + (x.head * S + x.lo) * d, kv_bytes, &full[s]);
    bulk_load_1d(stage_v(s), v + (x.head * S + x.lo) * d, kv_bytes, &full[s]);
    bulk_load_1d(stage_q(s), q + (x.head * S + x.t0) * d, q_bytes, &full[s]);
  };
  // Every thread: its share of the tile's random positions (entry e = token * R + r of the tile).
  auto fetch_pos = [&](const Tile& x, int (&pre)[kPosRegs]) {
#pragma unroll
    for (int u = 0; u < kPosRegs; ++u) {
      const int e = tid + u * kSparseThreads;
      int val = 0;
      if (e < x.nt * a.R) {
        const int i = x.t0 + e / a.R;
        if (i >= ng && i < S - ng) val = __ldg(rand_pos + (x.head * (S - G) + (i - ng)) * a.R + e % a.R);
      }
      pre[u] = val;
    }
  };
  auto park_pos = [&](int s, const int (&pre)[kPosRegs]) {
#pragma unroll
    for (int u = 0; u < kPosRegs; ++u) {
      const int e = tid + u * kSparseThreads;
      if (e < TT * a.R) stage_pos(s)[e] = pre[u];
    }
  };

  long long tile = first;
  if (tile >= n_tiles) return it_base;
  {
    const Tile x = tile_of(tile);
    if (tid == 0) issue(x, it_base & 1);
    int pre[kPosRegs];
    fetch_pos(x, pre);
    park_pos(it_base & 1, pre);
  }
  __syncthreads();

  int it = it_base;
  for (; tile < n_tiles; tile += step, ++it) {
    const int s = it & 1;
    const Tile x = tile_of(tile);
    const long long next = tile + step;
    int pre[kPosRegs];
    if (next < n_tiles) {
      // stage s ^ 1 was last read in the previous round; the barrier that closed it orders those
      // reads before these writes
      const Tile y = tile_of(next);
      if (tid == 0) issue(y, s ^ 1);
      fetch_pos(y, pre);
    }
    if (!mbar_wait(&full[s], (it >> 1) & 1, s_abort, status, FTB_ERR_TIMEOUT_TMA)) return -1;

    Rows<T> rw;
    rw.kh = k + x.head * S * d;
    rw.vh = v + x.head * S * d;
    rw.qh = q + x.head * S * d;
    rw.sk = stage_k(s);
    rw.sv = stage_v(s);
    rw.lo = x.lo;
    rw.hi = x.hi;
    const int* sp = stage_pos(s);
    // no global token in the tile and no window position that wraps
    const bool interior = x.t0 >= ng && x.t0 + x.nt <= S - ng && x.t0 - half >= 0 && x.t0 + x.nt - 1 + half < S;
    for (int tok = (tid >> 5) * TPW + lane / LPT; tok < x.nt; tok += (kSparseThreads / 32) * TPW) {
      const int i = x.t0 + tok;
      float qv[kEPL];
      load_row_shared<T, LPT>(stage_q(s) + tok * d, gl, qv);
      if constexpr (KW > 0) {
        attend_fast<T, LPT, KW, KR>(a, rw.sk, rw.sv, x.lo, rw.kh, rw.vh, i, gl, gmask, qv, sp + tok * KR,
                                    o + (x.head * S + i) * d, status);
      } else {
        attend_token<T, LPT>(a, rw, i, gl, gmask, interior, qv, [&](int r) { return sp[tok * a.R + r]; },
                             o + (x.head * S + i) * d, status);
      }
    }
    if (next < n_tiles) park_pos(s ^ 1, pre);
    __syncthreads();
  }
  return it;
}

// ------------------------------------------------------------------ tiled kernel
// KW = 0: every CTA walks the enumeration (per_head, lead, skip) with the general routine.  KW > 0:
// every CTA first walks its share of the edge tiles with the general routine, then its share of the
// interior tiles with the routine built for KW window and KR random keys; the two walks are separate
// pieces of code, so the register count is the larger of the two, not their sum.
template <typename T, int LPT, int KW, int KR>
__global__ void __launch_bounds__(kSparseThreads)
sparse_attn_tile_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                        const int* __restrict__ rand_pos, T* __restrict__ o, SparseArgs a, int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full[2];
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    s_abort = 0;
    fence_barrier_init();
  }
  grid_launch_dependents();
  __syncthreads();
  grid_dependency_wait();  // set-up done; the first copy of the walk reads global memory
  if constexpr (KW > 0) {
    // Edge tiles are handed out from the last CTA down, interior tiles from the first up: when the
    // edge tiles are fewer than the CTAs, the CTAs with one interior tile more do not get them.
    const int done = walk_tiles<T, LPT, 0, 0>(q, k, v, rand_pos, o, a, a.edge_per_head, a.edge_lead, a.edge_skip,
                                              gridDim.x - 1 - blockIdx.x, gridDim.x, 0, smem, full, &s_abort, status);
    if (done >= 0)
      walk_tiles<T, LPT, KW, KR>(q, k, v, rand_pos, o, a, a.per_head, a.lead, a.skip, blockIdx.x, gridDim.x, done,
                                 smem, full, &s_abort, status);
  } else {
    walk_tiles<T, LPT, 0, 0>(q, k, v, rand_pos, o, a, a.per_head, a.lead, a.skip, blockIdx.x, gridDim.x, 0, smem, full,
                             &s_abort, status);
  }
}

template <typename T, int LPT>
int launch_sparse(const void* q, const void* k, const void* v, const int* rand_pos, void* o, SparseArgs a,
                  int* status, cudaStream_t stream) {
  constexpr int d = kEPL * LPT;
  const int half = (a.window - 1) * a.dilation / 2;
  // Tiled kernel: the largest tile of 64, 32 or 16 tokens whose two stages fit.
  int TT = 0, stage = 0;
  if (a.R <= 16) {
    for (int t = 64; t >= 16; t >>= 1) {
      if (t * a.R > kPosRegs * kSparseThreads) continue;
      const long long rows = static_cast<long long>(t) + 2 * half;
      const long long bytes = (2 * rows + t) * d * static_cast<long long>(sizeof(T)) + ((t * a.R * 4 + 15) / 16) * 16;
      if (2 * bytes <= kMaxTileSmem) {
        TT = t;
        stage = static_cast<int>(bytes);
        break;
      }
    }
  }
  if (TT > 0) {
    static std::atomic<unsigned long long> configured{0}, configured_fast{0};
    auto kfn = sparse_attn_tile_kernel<T, LPT, 0, 0>;
    auto kfast = sparse_attn_tile_kernel<T, LPT, 5, 3>;
    if (ensure_dynamic_smem(kfn, kMaxTileSmem, configured) && ensure_dynamic_smem(kfast, kMaxTileSmem, configured_fast)) {
      a.TT = TT;
      a.tiles_per_head = (a.S + TT - 1) / TT;
      a.stage_bytes = stage;
      // Edge tiles: those with a global token or a window position that wraps, at both ends of a head.
      const int m = a.n_global > half ? a.n_global : half;
      int lead = (m + TT - 1) / TT, trail = a.tiles_per_head - (a.S - m) / TT;
      if (m == 0) lead = trail = 0;
      const int interior = a.tiles_per_head - lead - trail;
      const long long full = static_cast<long long>(current_sm_count()) * 2;  // two CTAs per SM, persistent
      auto run = [&](auto fn, const SparseArgs& b, long long ctas_wanted) -> int {
        const int grid = static_cast<int>(ctas_wanted < full ? ctas_wanted : full);
        const cudaError_t err = launch_dependent(fn, dim3(grid), dim3(kSparseThreads), 2 * stage, stream,
                                                 static_cast<const T*>(q), static_cast<const T*>(k),
                                                 static_cast<const T*>(v), rand_pos, static_cast<T*>(o), b, status);
        count_launch();
        if (err != cudaSuccess) cudaGetLastError();
        return err == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
      };
      a.edge_per_head = a.edge_lead = a.edge_skip = 0;
      if (a.window == 5 && a.R == 3 && !a.as_shipped && interior > 0) {
        // The example's key counts: interior tiles by the routine built for them, the edge tiles of
        // every head by the general one on a share of the CTAs in proportion to their number.
        a.per_head = interior;
        a.lead = 0;
        a.skip = lead;
        a.edge_per_head = lead + trail;
        a.edge_lead = lead;
        a.edge_skip = interior;
        const long long ctas = a.heads_total * a.tiles_per_head;
        return run(kfast, a, ctas);
      }
      a.per_head = a.tiles_per_head;
      a.lead = a.skip = 0;
      return run(kfn, a, a.heads_total * a.tiles_per_head);
    }
  }
  a.TT = a.tiles_per_head = a.stage_bytes = a.per_head = a.lead = a.skip = 0;
  a.edge_per_head = a.edge_lead = a.edge_skip = 0;
  const long long warps_needed = (a.heads_total * a.S + 32 / LPT - 1) / (32 / LPT);
  const long long ctas_needed = (warps_needed * 32 + kSparseThreads - 1) / kSparseThreads;
  const long long full = static_cast<long long>(current_sm_count()) * 8;
  const int grid = static_cast<int>(ctas_needed < full ? ctas_needed : full);
  const cudaError_t err = launch_light(sparse_attn_kernel<T, LPT>, dim3(grid), dim3(kSparseThreads), 0, stream,
                                           static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v),
                                           rand_pos, static_cast<T*>(o), a, status);
  count_launch();
  if (err != cudaSuccess) cudaGetLastError();
  return err == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
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
  if (B < 0 || heads <= 0 || S <= 0 || d <= 0) return FTB_ERR_ARG;
  if (B > 0 && (!q || !k || !v || !o)) return FTB_ERR_ARG;  // an empty batch has no storage to point at
  if (dtype != FTB_F32 && dtype != FTB_F16 && dtype != FTB_BF16) return FTB_ERR_ARG;
  if (window < 1 || window % 2 == 0 || dilation < 1 || n_global < 0 || R < 0) return FTB_ERR_ARG;
  if (B > 0 && R > 0 && S > 2 * n_global && !rand_pos) return FTB_ERR_ARG;
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
  a.TT = a.tiles_per_head = a.stage_bytes = a.per_head = a.lead = a.skip = 0;
  a.edge_per_head = a.edge_lead = a.edge_skip = 0;
  int* status = static_cast<int*>(workspace);  // sticky, as for the other single-kernel entry points
  switch (dtype) {
    case FTB_F32: return launch_sparse_d<float>(d, q, k, v, rand_pos, o, a, status, stream);
    case FTB_F16: return launch_sparse_d<__half>(d, q, k, v, rand_pos, o, a, status, stream);
    default: return launch_sparse_d<__nv_bfloat16>(d, q, k, v, rand_pos, o, a, status, stream);
  }
}
