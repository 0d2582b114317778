// One-off parameter re-layout for the cell kernels: the reference keeps one
// [in, out] matrix per gate (x @ W orientation, examples/stacked_rnn/rnn_utils.py);
// the kernels want one K-major row per accumulator column with the four gates of
// a unit in adjacent rows, so that a TMEM lane holds i,f,o,c~ of a unit in
// adjacent accumulator columns.
#include "ptx.cuh"
#include "tmap.h"

namespace ftb {

namespace {

// out[(u * gates + g) * ldo + k_off + k] = in[g][k][u], in: [gates, K, H].
template <typename E>
__global__ void pack_transpose_kernel(const E* __restrict__ in, E* __restrict__ out, int gates, int K, int H,
                                      int ldo, int k_off) {
  __shared__ E tile[32][33];
  const int g = blockIdx.z;
  const int k0 = blockIdx.y * 32, u0 = blockIdx.x * 32;
  const E* src = in + static_cast<size_t>(g) * K * H;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int k = k0 + i, u = u0 + threadIdx.x;
    if (k < K && u < H) tile[i][threadIdx.x] = src[static_cast<size_t>(k) * H + u];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int u = u0 + i, k = k0 + threadIdx.x;
    if (k < K && u < H) out[(static_cast<size_t>(u) * gates + g) * ldo + k_off + k] = tile[threadIdx.x][i];
  }
}

template <typename E>
__global__ void pack_bias_kernel(const E* __restrict__ bias, float* __restrict__ out, int gates, int H) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= gates * H) return;
  const int g = i / H, u = i - g * H;
  out[u * gates + g] = static_cast<float>(bias[i]);
}

template <typename E>
int pack_matrix(const E* in, E* out, int gates, int K, int H, int ldo, int k_off, cudaStream_t s) {
  dim3 grid((H + 31) / 32, (K + 31) / 32, gates), block(32, 8);
  pack_transpose_kernel<E><<<grid, block, 0, s>>>(in, out, gates, K, H, ldo, k_off);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
}

}  // namespace

int pack_lstm(const void* W, const void* U, const void* bias, void* Wp, float* bias_p, int D, int I, int H, int dtype,
              cudaStream_t s) {
  const size_t es = dtype_size(dtype);
  const int K = I + H;
  for (int d = 0; d < D; ++d) {
    const char* w = static_cast<const char*>(W) + static_cast<size_t>(d) * 4 * I * H * es;
    const char* u = static_cast<const char*>(U) + static_cast<size_t>(d) * 4 * H * H * es;
    char* o = static_cast<char*>(Wp) + static_cast<size_t>(d) * 4 * H * K * es;
    int rc;
    if (es == 4) {
      rc = pack_matrix<float>(reinterpret_cast<const float*>(w), reinterpret_cast<float*>(o), 4, I, H, K, 0, s);
      if (rc) return rc;
      rc = pack_matrix<float>(reinterpret_cast<const float*>(u), reinterpret_cast<float*>(o), 4, H, H, K, I, s);
    } else {
      rc = pack_matrix<uint16_t>(reinterpret_cast<const uint16_t*>(w), reinterpret_cast<uint16_t*>(o), 4, I, H, K, 0, s);
      if (rc) return rc;
      rc = pack_matrix<uint16_t>(reinterpret_cast<const uint16_t*>(u), reinterpret_cast<uint16_t*>(o), 4, H, H, K, I, s);
    }
    if (rc) return rc;
    if (bias != nullptr && bias_p != nullptr) {
      const char* b = static_cast<const char*>(bias) + static_cast<size_t>(d) * 4 * H * es;
      float* bo = bias_p + static_cast<size_t>(d) * 4 * H;
      const int n = 4 * H, thr = 256;
      if (dtype == FTB_F32)
        pack_bias_kernel<float><<<(n + thr - 1) / thr, thr, 0, s>>>(reinterpret_cast<const float*>(b), bo, 4, H);
      else if (dtype == FTB_F16)
        pack_bias_kernel<__half><<<(n + thr - 1) / thr, thr, 0, s>>>(reinterpret_cast<const __half*>(b), bo, 4, H);
      else
        pack_bias_kernel<__nv_bfloat16><<<(n + thr - 1) / thr, thr, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(b), bo, 4, H);
      if (cudaGetLastError() != cudaSuccess) return FTB_ERR_LAUNCH;
      count_launch();
    }
  }
  return FTB_OK;
}

// P: [H, V] (x @ P orientation) -> Pt: [Vp, H] K-major, row v = column v of P, rows V..Vp-1 zero.
int pack_projection(const void* P, void* Pt, int H, int V, int Vp, int dtype, cudaStream_t s) {
  const size_t es = dtype_size(dtype);
  if (cudaMemsetAsync(Pt, 0, static_cast<size_t>(Vp) * H * es, s) != cudaSuccess) return FTB_ERR_LAUNCH;
  // pack_matrix with one "gate": out[u * ldo + k] = in[k][u] for k < K = H, u < V
  if (es == 4) return pack_matrix<float>(static_cast<const float*>(P), static_cast<float*>(Pt), 1, H, V, H, 0, s);
  return pack_matrix<uint16_t>(static_cast<const uint16_t*>(P), static_cast<uint16_t*>(Pt), 1, H, V, H, 0, s);
}

int pack_grid(const void* i2h, const void* h2h, void* Wp, int H, int dtype, cudaStream_t s) {
  int rc;
  if (dtype_size(dtype) == 4) {
    rc = pack_matrix<float>(static_cast<const float*>(i2h), static_cast<float*>(Wp), 1, 2 * H, H, 3 * H, 0, s);
    if (rc) return rc;
    rc = pack_matrix<float>(static_cast<const float*>(h2h), static_cast<float*>(Wp), 1, H, H, 3 * H, 2 * H, s);
  } else {
    rc = pack_matrix<uint16_t>(static_cast<const uint16_t*>(i2h), static_cast<uint16_t*>(Wp), 1, 2 * H, H, 3 * H, 0, s);
    if (rc) return rc;
    rc = pack_matrix<uint16_t>(static_cast<const uint16_t*>(h2h), static_cast<uint16_t*>(Wp), 1, H, H, 3 * H, 2 * H, s);
  }
  return rc;
}

// Tanh RNN cell: Wp[u, k] = W[k, u] for k < I, U[k - I, u] for the H recurrent inputs behind them.
int pack_rnn(const void* W, const void* U, void* Wp, int I, int H, int dtype, cudaStream_t s) {
  int rc;
  if (dtype_size(dtype) == 4) {
    rc = pack_matrix<float>(static_cast<const float*>(W), static_cast<float*>(Wp), 1, I, H, I + H, 0, s);
    if (rc) return rc;
    rc = pack_matrix<float>(static_cast<const float*>(U), static_cast<float*>(Wp), 1, H, H, I + H, I, s);
  } else {
    rc = pack_matrix<uint16_t>(static_cast<const uint16_t*>(W), static_cast<uint16_t*>(Wp), 1, I, H, I + H, 0, s);
    if (rc) return rc;
    rc = pack_matrix<uint16_t>(static_cast<const uint16_t*>(U), static_cast<uint16_t*>(Wp), 1, H, H, I + H, I, s);
  }
  return rc;
}

}  // namespace ftb
