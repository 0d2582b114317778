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

constexpr int TM = 32;   // rows per tile
constexpr int TN = 64;   // accumulator columns per tile (16 LSTM units)
constexpr int TK = 32;   // K chunk
constexpr int kSimtThreads = 256;

struct SimtArgs {
  const float* act[kNumActMaps];
  int32_t ld_act[kNumActMaps];
  const float* w[kNumWeightMaps];  // packed weights [rows, ldw]
  int32_t ldw;
};

__device__ __forceinline__ float sigmoid_acc(float x) { return 1.f / (1.f + expf(-x)); }

template <int EPI>
__global__ void __launch_bounds__(kSimtThreads)
cell_simt_kernel(const __grid_constant__ SimtArgs args, const __grid_constant__ CellBatch batch) {
  __shared__ float sA[TK][TM + 1];
  __shared__ float sW[TK][TN + 4];

  const int tile = blockIdx.x;
  int idx = 0;
  for (int i = 1; i < batch.n_items; ++i)
    if (tile >= batch.items[i].tile0) idx = i;
  const CellItem& it = batch.items[idx];
  const int local = tile - it.tile0;
  const int n_tile = local / it.m_tiles;
  const int m_tile = local - n_tile * it.m_tiles;

  const int tx = threadIdx.x & 15;  // 4 consecutive columns: one LSTM unit
  const int ty = threadIdx.x >> 4;  // 2 consecutive rows
  float acc[2][4] = {};

  // K is walked in chunks of TK over the cell's segments.  The next chunk's global loads are
  // issued into registers before the current chunk is multiplied out of shared memory, so their
  // latency overlaps the arithmetic instead of preceding it (same summation order either way).
  const int ld_r = threadIdx.x >> 3;        // row (A) / first column (W) this thread loads
  const int ld_kq = (threadIdx.x & 7) * 4;  // its four consecutive k
  const bool a_row_ok = m_tile * TM + ld_r < it.rows;
  float4 va = make_float4(0.f, 0.f, 0.f, 0.f), vw0 = va, vw1 = va;
  auto fetch = [&](int s, int k0) {
    const float* A = args.act[it.seg_map[s]];
    const int lda = args.ld_act[it.seg_map[s]];
    const int row0 = it.seg_row[s] + m_tile * TM;
    const float* W = args.w[it.w_map] + static_cast<size_t>(it.w_row0 + n_tile * TN) * args.ldw + it.seg_wk[s];
    va = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a_row_ok) va = *reinterpret_cast<const float4*>(A + static_cast<size_t>(row0 + ld_r) * lda + k0 + ld_kq);
    vw0 = *reinterpret_cast<const float4*>(W + static_cast<size_t>(ld_r) * args.ldw + k0 + ld_kq);
    vw1 = *reinterpret_cast<const float4*>(W + static_cast<size_t>(ld_r + 32) * args.ldw + k0 + ld_kq);
  };
  int s = 0, k0 = 0;
  if (it.nseg > 0) fetch(0, 0);
  while (s < it.nseg) {
    sA[ld_kq + 0][ld_r] = va.x; sA[ld_kq + 1][ld_r] = va.y; sA[ld_kq + 2][ld_r] = va.z; sA[ld_kq + 3][ld_r] = va.w;
    sW[ld_kq + 0][ld_r] = vw0.x; sW[ld_kq + 1][ld_r] = vw0.y; sW[ld_kq + 2][ld_r] = vw0.z; sW[ld_kq + 3][ld_r] = vw0.w;
    sW[ld_kq + 0][ld_r + 32] = vw1.x; sW[ld_kq + 1][ld_r + 32] = vw1.y;
    sW[ld_kq + 2][ld_r + 32] = vw1.z; sW[ld_kq + 3][ld_r + 32] = vw1.w;
    __syncthreads();
    int ns = s, nk0 = k0 + TK;
    if (nk0 >= it.seg_kb[s] * 64) {
      ++ns;
      nk0 = 0;
    }
    if (ns < it.nseg) fetch(ns, nk0);
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      const float a0 = sA[k][2 * ty], a1 = sA[k][2 * ty + 1];
      const float4 w = *reinterpret_cast<const float4*>(&sW[k][4 * tx]);
      acc[0][0] = fmaf(a0, w.x, acc[0][0]); acc[0][1] = fmaf(a0, w.y, acc[0][1]);
      acc[0][2] = fmaf(a0, w.z, acc[0][2]); acc[0][3] = fmaf(a0, w.w, acc[0][3]);
      acc[1][0] = fmaf(a1, w.x, acc[1][0]); acc[1][1] = fmaf(a1, w.y, acc[1][1]);
      acc[1][2] = fmaf(a1, w.z, acc[1][2]); acc[1][3] = fmaf(a1, w.w, acc[1][3]);
    }
    __syncthreads();
    s = ns;
    k0 = nk0;
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

// fp32 twin of launch_cell_gemm.  Tiles are 32 rows x 64 columns, so the
// batch must have been tiled with m_tiles = ceil(rows / 32) and n_cols % 64 == 0.
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
