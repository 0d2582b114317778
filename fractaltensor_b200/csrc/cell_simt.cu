// fp32 RNN cell kernel (CUDA cores).  tcgen05 has no fp32 x fp32 MMA kind and
// kind::tf32 keeps 10 mantissa bits, which cannot meet a 1e-5 relative bound, so
// the fp32 configurations run on FFMA with the same work-item description and
// the same packed (K-major, gate-interleaved) weights as the 16-bit kernel.
// Follows the arithmetic of the reference cell programs
// (examples/stacked_rnn/stacked_rnn.py:12-36, examples/grid_rnn/grid_rnn.py:42-72).
#include "cell.h"
#include "ptx.cuh"
#include "tmap.h"

namespace ftb {

namespace {

// Small tiles: the fp32 configurations are latency-bound wavefronts of small cells, so what
// counts is how many SMs a level reaches and how short one tile's K loop is.
constexpr int TM = 32;   // rows per tile
constexpr int TN = 32;   // accumulator columns per tile (8 LSTM units)
constexpr int TK = 32;   // K chunk
constexpr int kGroupThreads = 128;  // threads that share one slice of K
constexpr int kSplitK = 4;          // slices of K per tile, one per group of 128 threads
constexpr int kSimtThreads = kGroupThreads * kSplitK;

struct SimtArgs {
  const float* act[kNumActMaps];
  int32_t ld_act[kNumActMaps];
  const float* w[kNumWeightMaps];  // packed weights [rows, ldw]
  int32_t ldw;
};

__device__ __forceinline__ float sigmoid_acc(float x) { return 1.f / (1.f + expf(-x)); }

__device__ __forceinline__ void group_barrier(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(kGroupThreads) : "memory");
}

// One CTA computes one 32 x 32 tile.  A wavefront level is a few hundred tiles of a short K loop
// on a 148-SM device, so a tile's latency is what counts: the K chunks of the tile are dealt out to
// four groups of 128 threads (each with its own shared-memory buffers and its own named barrier),
// every group accumulates its quarter of K in the same 32 x 32 layout, and group 0 adds the four
// partial sums in a fixed order and runs the epilogue.
template <int EPI>
__global__ void __launch_bounds__(kSimtThreads)
cell_simt_kernel(const __grid_constant__ SimtArgs args, const __grid_constant__ CellBatch batch) {
  __shared__ __align__(16) float sA[kSplitK][TM][TK + 4];  // [group][row][k]: a thread reads four k of a row at once
  __shared__ __align__(16) float sW[kSplitK][TK][TN + 4];  // [group][k][column]
  __shared__ __align__(16) float sP[kSplitK - 1][kGroupThreads][8];  // partial sums of groups 1..3

  // A kernel launched behind this one as a dependent (the attention step of the attention RNN) may
  // be scheduled while this one drains; this kernel itself waits for the one before it.
  grid_launch_dependents();
  grid_dependency_wait();
  const int tile = blockIdx.x;
  int idx = 0;
  for (int i = 1; i < batch.n_items; ++i)
    if (tile >= batch.items[i].tile0) idx = i;
  const CellItem& it = batch.items[idx];
  const int local = tile - it.tile0;
  const int n_tile = local / it.m_tiles;
  const int m_tile = local - n_tile * it.m_tiles;

  const int grp = threadIdx.x / kGroupThreads;  // which slice of K
  const int tg = threadIdx.x % kGroupThreads;   // thread within the group
  const int tx = tg & 7;   // 4 consecutive columns: one LSTM unit
  const int ty = tg >> 3;  // 2 consecutive rows
  float acc[2][4] = {};

  // K is walked in chunks of TK over the cell's segments; this group takes chunks [c_begin, c_end) of
  // the walk.  The next chunk's global loads are issued into registers before the current chunk is
  // multiplied out of shared memory, so their latency overlaps the arithmetic.
  int total_chunks = 0;
  for (int s = 0; s < it.nseg; ++s) total_chunks += it.seg_kb[s] * (64 / TK);
  const int c_begin = total_chunks * grp / kSplitK, c_end = total_chunks * (grp + 1) / kSplitK;
  const int ld_r = tg >> 3;        // first row (A) / column (W) this thread loads; second is +16
  const int ld_kq = (tg & 7) * 4;  // its four consecutive k
  const bool a_ok0 = m_tile * TM + ld_r < it.rows, a_ok1 = m_tile * TM + ld_r + 16 < it.rows;
  float4 va0 = make_float4(0.f, 0.f, 0.f, 0.f), va1 = va0, vw0 = va0, vw1 = va0;
  auto fetch = [&](int s, int k0) {
    const float* A = args.act[it.seg_map[s]];
    const int lda = args.ld_act[it.seg_map[s]];
    const int row0 = it.seg_row[s] + m_tile * TM;
    const float* W = args.w[it.w_map] + static_cast<size_t>(it.w_row0 + n_tile * TN) * args.ldw + it.seg_wk[s];
    va0 = va1 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a_ok0) va0 = *reinterpret_cast<const float4*>(A + static_cast<size_t>(row0 + ld_r) * lda + k0 + ld_kq);
    if (a_ok1) va1 = *reinterpret_cast<const float4*>(A + static_cast<size_t>(row0 + ld_r + 16) * lda + k0 + ld_kq);
    vw0 = *reinterpret_cast<const float4*>(W + static_cast<size_t>(ld_r) * args.ldw + k0 + ld_kq);
    vw1 = *reinterpret_cast<const float4*>(W + static_cast<size_t>(ld_r + 16) * args.ldw + k0 + ld_kq);
  };
  // (segment, k offset) of chunk c_begin
  int s = 0, k0 = 0;
  {
    int skip = c_begin;
    while (s < it.nseg && skip >= it.seg_kb[s] * (64 / TK)) {
      skip -= it.seg_kb[s] * (64 / TK);
      ++s;
    }
    k0 = skip * TK;
  }
  if (c_begin < c_end) fetch(s, k0);
  for (int c = c_begin; c < c_end; ++c) {
    *reinterpret_cast<float4*>(&sA[grp][ld_r][ld_kq]) = va0;
    *reinterpret_cast<float4*>(&sA[grp][ld_r + 16][ld_kq]) = va1;
    sW[grp][ld_kq + 0][ld_r] = vw0.x; sW[grp][ld_kq + 1][ld_r] = vw0.y; sW[grp][ld_kq + 2][ld_r] = vw0.z; sW[grp][ld_kq + 3][ld_r] = vw0.w;
    sW[grp][ld_kq + 0][ld_r + 16] = vw1.x; sW[grp][ld_kq + 1][ld_r + 16] = vw1.y;
    sW[grp][ld_kq + 2][ld_r + 16] = vw1.z; sW[grp][ld_kq + 3][ld_r + 16] = vw1.w;
    group_barrier(grp);
    int ns = s, nk0 = k0 + TK;
    if (nk0 >= it.seg_kb[s] * 64) {
      ++ns;
      nk0 = 0;
    }
    if (c + 1 < c_end) fetch(ns, nk0);
#pragma unroll
    for (int k4 = 0; k4 < TK; k4 += 4) {
      const float4 r0 = *reinterpret_cast<const float4*>(&sA[grp][2 * ty][k4]);
      const float4 r1 = *reinterpret_cast<const float4*>(&sA[grp][2 * ty + 1][k4]);
      const float a0[4] = {r0.x, r0.y, r0.z, r0.w}, a1[4] = {r1.x, r1.y, r1.z, r1.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 w = *reinterpret_cast<const float4*>(&sW[grp][k4 + j][4 * tx]);
        acc[0][0] = fmaf(a0[j], w.x, acc[0][0]); acc[0][1] = fmaf(a0[j], w.y, acc[0][1]);
        acc[0][2] = fmaf(a0[j], w.z, acc[0][2]); acc[0][3] = fmaf(a0[j], w.w, acc[0][3]);
        acc[1][0] = fmaf(a1[j], w.x, acc[1][0]); acc[1][1] = fmaf(a1[j], w.y, acc[1][1]);
        acc[1][2] = fmaf(a1[j], w.z, acc[1][2]); acc[1][3] = fmaf(a1[j], w.w, acc[1][3]);
      }
    }
    group_barrier(grp);
    s = ns;
    k0 = nk0;
  }

  // Partial sums of groups 1..3 to group 0, added in group order.
  if (grp > 0) {
    *reinterpret_cast<float4*>(&sP[grp - 1][tg][0]) = make_float4(acc[0][0], acc[0][1], acc[0][2], acc[0][3]);
    *reinterpret_cast<float4*>(&sP[grp - 1][tg][4]) = make_float4(acc[1][0], acc[1][1], acc[1][2], acc[1][3]);
  }
  __syncthreads();
  if (grp > 0) return;
#pragma unroll
  for (int g = 0; g < kSplitK - 1; ++g) {
    const float4 p0 = *reinterpret_cast<const float4*>(&sP[g][tg][0]);
    const float4 p1 = *reinterpret_cast<const float4*>(&sP[g][tg][4]);
    acc[0][0] += p0.x; acc[0][1] += p0.y; acc[0][2] += p0.z; acc[0][3] += p0.w;
    acc[1][0] += p1.x; acc[1][1] += p1.y; acc[1][2] += p1.z; acc[1][3] += p1.w;
  }

  const int col0 = n_tile * TN + 4 * tx;
  float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
  if (it.bias != nullptr) b = *reinterpret_cast<const float4*>(it.bias + col0);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = m_tile * TM + 2 * ty + i;
    if (row >= it.rows) continue;
    if (EPI == EPI_LSTM) {
      const int unit = col0 >> 2;
      float* cp = it.c + static_cast<size_t>(row) * batch.ld_c + unit;
      const float cprev = it.c_zero ? 0.f : *cp;
      const float gi = sigmoid_acc(acc[i][0] + b.x);
      const float gf = sigmoid_acc(acc[i][1] + b.y);
      const float go = sigmoid_acc(acc[i][2] + b.z);
      const float gc = tanhf(acc[i][3] + b.w);
      const float cn = gf * cprev + gi * gc;
      *cp = cn;
      reinterpret_cast<float*>(it.out)[static_cast<size_t>(row) * batch.ld_out + unit] = go * tanhf(cn);
    } else {
      float4 v = make_float4(acc[i][0] + b.x, acc[i][1] + b.y, acc[i][2] + b.z, acc[i][3] + b.w);
      if (EPI == EPI_TANH) {
        v.x = tanhf(v.x); v.y = tanhf(v.y); v.z = tanhf(v.z); v.w = tanhf(v.w);
      }
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(it.out) + static_cast<size_t>(row) * batch.ld_out + col0) = v;
    }
  }
}

}  // namespace

// fp32 twin of launch_cell_gemm.  Tiles are 32 rows x 32 columns, so the
// batch must have been tiled with m_tiles = ceil(rows / 32) and n_cols % 32 == 0.
int launch_cell_simt(int epi, const float* const* act, const int* ld_act, const float* const* w, int ldw,
                     const CellBatch& batch, cudaStream_t stream) {
  SimtArgs a;
  for (int i = 0; i < kNumActMaps; ++i) {
    a.act[i] = act[i];
    a.ld_act[i] = ld_act[i];
  }
  for (int i = 0; i < kNumWeightMaps; ++i) a.w[i] = w[i];
  a.ldw = ldw;
  if (batch.total_tiles <= 0) return FTB_OK;
  // Plain launches: as a dependent launch this kernel was measured 45 % slower on the 67 levels of a
  // depth-4 stack (it has no set-up to run early, and the wait for the level before it costs more
  // than an ordinary launch behind it).
  switch (epi) {
    case EPI_STORE: cell_simt_kernel<EPI_STORE><<<batch.total_tiles, kSimtThreads, 0, stream>>>(a, batch); break;
    case EPI_LSTM: cell_simt_kernel<EPI_LSTM><<<batch.total_tiles, kSimtThreads, 0, stream>>>(a, batch); break;
    case EPI_TANH: cell_simt_kernel<EPI_TANH><<<batch.total_tiles, kSimtThreads, 0, stream>>>(a, batch); break;
    default: return FTB_ERR_ARG;
  }
  count_launch();
  return cudaGetLastError() == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
}

}  // namespace ftb
