// Attention step of the attention RNN (examples/rnn_attention/rnn_attention.py:52-70, attn_func):
//
//   scores_j = e_j @ encoder_proj + decoder @ decoder_proj      (one number per encoder position)
//   weights  = softmax over the encoder positions j
//   v        = sum_j weights_j * e_j
//
// for every sequence of the batch at one decoder step.  The decoder state itself,
// tanh(y_t @ W + v_{t-1} @ U + b), is a cell of the wavefront (csrc/cell_gemm.cu / cell_simt.cu);
// this file holds what surrounds it: the scores e_j @ encoder_proj, which do not depend on the
// decoder step and are computed once per call, and the softmax-weighted sum of the encoder rows.
//
// Layout: time-major padded batches, row (j, n) of `enc` at (j * N + n) * H.  Sequence n attends to
// encoder positions j < src_lens[n] (all Ls when src_lens is NULL).  HBM/L2-bound row work: per
// decoder step and sequence the kernel reads len * H encoder elements (they stay in L2 across the
// steps) and writes H.
#include "../../include/ftb200.h"
#include "ptx.cuh"
#include "tmap.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace ftb {
namespace {

constexpr int kStepThreads = 128;  // one output column per thread

template <typename T> __device__ __forceinline__ float ld_f32(const T* p);
template <> __device__ __forceinline__ float ld_f32<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ld_f32<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st_f32(T* p, float x);
template <> __device__ __forceinline__ void st_f32<float>(float* p, float x) { *p = x; }
template <> __device__ __forceinline__ void st_f32<__half>(__half* p, float x) { *p = __float2half_rn(x); }
template <> __device__ __forceinline__ void st_f32<__nv_bfloat16>(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

// scores[r] = rows[r, :] . proj for r < n_rows: one warp per row.
template <typename T>
__global__ void __launch_bounds__(256)
row_dot_kernel(const T* __restrict__ rows, const T* __restrict__ proj, float* __restrict__ scores, long long n_rows,
               int H) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  grid_launch_dependents();
  grid_dependency_wait();  // the encoder's last level wrote the rows
  for (long long r = warp; r < n_rows; r += n_warps) {
    float s = 0.f;
    for (int h = lane; h < H; h += 32) s = fmaf(ld_f32<T>(rows + r * H + h), ld_f32<T>(proj + h), s);
    s = warp_sum(s);
    if (lane == 0) scores[r] = s;
  }
}

// One decoder step.  grid = (N, ceil(H / 128)); CTA (n, cb) computes columns cb * 128 .. of v for
// sequence n.  Every CTA of a sequence recomputes the len weights (a dot product over H and a
// softmax over len numbers: small next to the len x 128 weighted sum).
template <typename T>
__global__ void __launch_bounds__(kStepThreads)
attn_step_kernel(const T* __restrict__ enc, const float* __restrict__ enc_scores, const T* __restrict__ dec_t,
                 const T* __restrict__ dec_proj, const int* __restrict__ src_lens, T* __restrict__ out_t, int Ls,
                 int N, int H) {
  extern __shared__ float s_w[];  // [Ls] scores, then weights
  __shared__ float s_red[kStepThreads / 32];
  const int n = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  // Launched behind the decoder cell of this step; the next step's cell may be scheduled now and
  // waits for this kernel before it reads the attention vectors.
  grid_launch_dependents();
  grid_dependency_wait();
  int len = src_lens ? src_lens[n] : Ls;
  len = len < 0 ? 0 : (len > Ls ? Ls : len);

  // c = decoder . decoder_proj
  float part = 0.f;
  for (int h = tid; h < H; h += kStepThreads) part = fmaf(ld_f32<T>(dec_t + static_cast<long long>(n) * H + h), ld_f32<T>(dec_proj + h), part);
  part = warp_sum(part);
  if (lane == 0) s_red[wid] = part;
  __syncthreads();
  float c = 0.f;
#pragma unroll
  for (int w = 0; w < kStepThreads / 32; ++w) c += s_red[w];
  __syncthreads();

  // scores and their maximum
  float mx = -INFINITY;
  for (int j = tid; j < len; j += kStepThreads) {
    const float s = enc_scores[static_cast<long long>(j) * N + n] + c;
    s_w[j] = s;
    mx = fmaxf(mx, s);
  }
  mx = warp_max(mx);
  if (lane == 0) s_red[wid] = mx;
  __syncthreads();
  mx = s_red[0];
#pragma unroll
  for (int w = 1; w < kStepThreads / 32; ++w) mx = fmaxf(mx, s_red[w]);
  __syncthreads();
  float sum = 0.f;
  for (int j = tid; j < len; j += kStepThreads) {
    const float e = expf(s_w[j] - mx);
    s_w[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  if (lane == 0) s_red[wid] = sum;
  __syncthreads();
  sum = 0.f;
#pragma unroll
  for (int w = 0; w < kStepThreads / 32; ++w) sum += s_red[w];
  const float inv = len > 0 ? 1.f / sum : 0.f;

  // weighted sum of the encoder rows, one column per thread, four rows in flight
  const int h = blockIdx.y * kStepThreads + tid;
  if (h >= H) return;
  const T* col = enc + static_cast<long long>(n) * H + h;
  const long long stride = static_cast<long long>(N) * H;
  float acc = 0.f;
  int j = 0;
  for (; j + 4 <= len; j += 4) {
    const float e0 = ld_f32<T>(col + (j + 0) * stride), e1 = ld_f32<T>(col + (j + 1) * stride);
    const float e2 = ld_f32<T>(col + (j + 2) * stride), e3 = ld_f32<T>(col + (j + 3) * stride);
    acc = fmaf(s_w[j], e0, acc);
    acc = fmaf(s_w[j + 1], e1, acc);
    acc = fmaf(s_w[j + 2], e2, acc);
    acc = fmaf(s_w[j + 3], e3, acc);
  }
  for (; j < len; ++j) acc = fmaf(s_w[j], ld_f32<T>(col + j * stride), acc);
  st_f32<T>(out_t + static_cast<long long>(n) * H + h, acc * inv);
}

template <typename T>
int enc_scores_t(const void* enc, const void* proj, float* scores, long long n_rows, int H, cudaStream_t stream) {
  const long long ctas = (n_rows + 7) / 8;
  const long long full = static_cast<long long>(current_sm_count()) * 8;
  const int grid = static_cast<int>(ctas < full ? ctas : full);
  const cudaError_t err = launch_light(row_dot_kernel<T>, dim3(grid), dim3(256), 0, stream, static_cast<const T*>(enc),
                                           static_cast<const T*>(proj), scores, n_rows, H);
  count_launch();
  if (err != cudaSuccess) cudaGetLastError();
  return err == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
}

template <typename T>
int attn_step_t(const void* enc, const float* enc_scores, const void* dec_t, const void* dec_proj, const int* src_lens,
                void* out_t, int Ls, int N, int H, cudaStream_t stream) {
  const dim3 grid(N, (H + kStepThreads - 1) / kStepThreads);
  const cudaError_t err = launch_light(attn_step_kernel<T>, grid, dim3(kStepThreads), static_cast<size_t>(Ls) * sizeof(float),
                                           stream, static_cast<const T*>(enc), enc_scores, static_cast<const T*>(dec_t),
                                           static_cast<const T*>(dec_proj), src_lens, static_cast<T*>(out_t), Ls, N, H);
  count_launch();
  if (err != cudaSuccess) cudaGetLastError();
  return err == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
}

}  // namespace

// Longest source sequence the step kernel takes: its scores sit in 48 KB of shared memory.
int rnn_attention_max_src_len() { return 48 * 1024 / static_cast<int>(sizeof(float)); }

int launch_enc_scores(int dtype, const void* enc, const void* proj, float* scores, long long n_rows, int H,
                      cudaStream_t stream) {
  switch (dtype) {
    case FTB_F32: return enc_scores_t<float>(enc, proj, scores, n_rows, H, stream);
    case FTB_F16: return enc_scores_t<__half>(enc, proj, scores, n_rows, H, stream);
    default: return enc_scores_t<__nv_bfloat16>(enc, proj, scores, n_rows, H, stream);
  }
}

int launch_attn_step(int dtype, const void* enc, const float* enc_scores, const void* dec_t, const void* dec_proj,
                     const int* src_lens, void* out_t, int Ls, int N, int H, cudaStream_t stream) {
  switch (dtype) {
    case FTB_F32: return attn_step_t<float>(enc, enc_scores, dec_t, dec_proj, src_lens, out_t, Ls, N, H, stream);
    case FTB_F16: return attn_step_t<__half>(enc, enc_scores, dec_t, dec_proj, src_lens, out_t, Ls, N, H, stream);
    default: return attn_step_t<__nv_bfloat16>(enc, enc_scores, dec_t, dec_proj, src_lens, out_t, Ls, N, H, stream);
  }
}

}  // namespace ftb
