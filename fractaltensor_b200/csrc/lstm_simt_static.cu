// fp32 stacked LSTM as one persistent launch with static tile ownership
// (examples/stacked_rnn/stacked_lstm1.py:12-76; the step structure of the reference's fused
// kernel, kaleido/core/device/kernels/lstm/stacked_lstm/region*.h: every cell reads the layer
// below at its own step and its own layer one step back).
//
// The fp32 configurations are small cells on a long dependency chain (depth 4, 64 steps: 67
// wavefront levels), so a launch per level costs more than the level's arithmetic.  Here a CTA owns
// one 32-row x 32-column accumulator tile (8 hidden units x 4 gates) of one layer for the whole
// sweep over time:
//   * its slice of the packed weights, [I + H] x 32 floats, is read once and stays in shared memory;
//   * the cell state of its units stays in registers (only the final state is stored);
//   * cells hand their output to each other through one completion counter per cell
//     (red.release / ld.acquire, every wait bounded) instead of kernel boundaries.
// The arithmetic is the level kernel's (csrc/cell_simt.cu), operation for operation: K is dealt out
// to four groups in the same chunks, every group adds its products in the same order and the four
// partial sums are added in group order, so both schedules give the same bits.
//
// The launch is cooperative: every CTA must be resident, because CTAs wait for each other.
#include "../../include/ftb200.h"
#include "ptx.cuh"
#include "tmap.h"

#include <atomic>
#include <cstdlib>

namespace ftb {

namespace {

constexpr int TM = 32;              // rows per tile
constexpr int TN = 32;              // accumulator columns per tile
constexpr int TK = 32;              // K chunk of the level kernel (fixes the summation order)
constexpr int kGroupThreads = 128;  // threads that share one slice of K
constexpr int kSplitK = 4;
constexpr int kThreads = kGroupThreads * kSplitK;
constexpr int kMaxSmem = 224 * 1024;  // dynamic part; the kernel has a few bytes of static shared memory too

struct SimtStaticArgs {
  const float* x;     // [L, N, I]
  const float* w;     // packed [D, 4H, I + H]
  const float* bias;  // packed [D, 4H] or null
  float* hs;          // [D, L, N, H]
  float* c;           // [D, N, H]
  int* done;          // one counter per cell (l * L + t), zero at launch
  int* status;
  int D, L, N, I, H;
  int m_tiles, n_tiles;  // tiles of a cell
  int G;                 // layers resident at a time: CTA (j, tile) sweeps layers j, j + G, ...
};

__device__ __forceinline__ float sigmoid_acc(float x) { return 1.f / (1.f + expf(-x)); }

__device__ __forceinline__ void group_barrier(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(kGroupThreads) : "memory");
}

__device__ __forceinline__ float4 ld_cg4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

// Thread 0 of the CTA: wait until `*counter >= target`.  False on time-out or when another CTA has
// already reported an error (its dependants would only time out one after another).
__device__ __forceinline__ bool wait_cell(const int* counter, int target, int* status) {
  if (ld_acquire_gpu(counter) >= target) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  for (;;) {
    if (ld_acquire_gpu(counter) >= target) return true;
    if (((++it) & 0xFF) == 0) {
      if (ld_relaxed_gpu(status) != 0) return false;
      if (globaltimer_ns() - t0 > FTB_WAIT_TIMEOUT_NS) {
        atomicCAS(status, 0, FTB_ERR_TIMEOUT_DEP);
        return false;
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
lstm_simt_static_kernel(const __grid_constant__ SimtStaticArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int K = a.I + a.H;
  const int ldw = TN + 4;  // sW[k][column]
  const int lda = K + 4;   // sA[row][k]
  float* sW = reinterpret_cast<float*>(smem_raw);
  float* sA = sW + static_cast<size_t>(K) * ldw;
  float* sP = sA + static_cast<size_t>(TM) * lda;  // [kSplitK][TM][TN] partial sums
  __shared__ int s_ok;

  const int tiles = a.m_tiles * a.n_tiles;
  const int j = blockIdx.x / tiles;
  const int tile = blockIdx.x - j * tiles;
  const int n_tile = tile / a.m_tiles;
  const int m_tile = tile - n_tile * a.m_tiles;
  const int row0 = m_tile * TM;

  const int tid = threadIdx.x;
  const int grp = tid / kGroupThreads;
  const int tg = tid % kGroupThreads;
  const int tx = tg & 7;   // 4 consecutive columns: one LSTM unit
  const int ty = tg >> 3;  // 2 consecutive rows
  const int target = tiles;  // every tile of a cell adds one

  for (int l = j; l < a.D; l += a.G) {
    const int Il = l == 0 ? a.I : a.H;  // width of the input half
    const int Kl = Il + a.H;
    // ---- this tile's weights: rows n_tile * 32 .. + 31 of the layer's packed matrix, [column][k]
    // in global memory, [k][column] in shared memory.
    {
      const float* W = a.w + (static_cast<size_t>(l) * 4 * a.H + n_tile * TN) * K;
      const int k4s = Kl / 4;
      for (int e = tid; e < TN * k4s; e += kThreads) {
        const int col = e / k4s, k = (e - col * k4s) * 4;
        const float4 v = *reinterpret_cast<const float4*>(W + static_cast<size_t>(col) * K + k);
        sW[(k + 0) * ldw + col] = v.x;
        sW[(k + 1) * ldw + col] = v.y;
        sW[(k + 2) * ldw + col] = v.z;
        sW[(k + 3) * ldw + col] = v.w;
      }
    }
    const int col0 = n_tile * TN + 4 * tx;
    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a.bias != nullptr) b = *reinterpret_cast<const float4*>(a.bias + static_cast<size_t>(l) * 4 * a.H + col0);
    float creg[2] = {0.f, 0.f};

    for (int t = 0; t < a.L; ++t) {
      // ---- dependencies: the layer below at this step, this layer one step back
      if (tid == 0) {
        bool ok = true;
        if (l > 0) ok = wait_cell(a.done + (l - 1) * a.L + t, target, a.status);
        if (ok && t > 0) ok = wait_cell(a.done + l * a.L + t - 1, target, a.status);
        s_ok = ok ? 1 : 0;
      }
      __syncthreads();  // also: everyone has finished with sA and sP of the previous step
      if (!s_ok) return;

      // ---- the tile's 32 rows of both operands into shared memory (L2 loads: other SMs wrote them)
      const int Kt = t == 0 ? Il : Kl;  // the first step has no recurrent half
      {
        const float* in = l == 0 ? a.x + static_cast<size_t>(t) * a.N * a.I
                                 : a.hs + (static_cast<size_t>(l - 1) * a.L + t) * a.N * a.H;
        const float* rec = t > 0 ? a.hs + (static_cast<size_t>(l) * a.L + t - 1) * a.N * a.H : nullptr;
        const int k4s = Kt / 4, n4 = TM * k4s;
        // eight loads in flight per thread before the first store (one round trip to L2 for K = 512)
        constexpr int kBatch = 8;
        for (int e0 = tid; e0 < n4; e0 += kBatch * kThreads) {
          float4 v[kBatch];
#pragma unroll
          for (int u = 0; u < kBatch; ++u) {
            const int e = e0 + u * kThreads;
            const int r = e / k4s, k = (e - r * k4s) * 4;
            v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (e < n4 && row0 + r < a.N) {
              v[u] = k < Il ? ld_cg4(in + static_cast<size_t>(row0 + r) * Il + k)
                            : ld_cg4(rec + static_cast<size_t>(row0 + r) * a.H + (k - Il));
            }
          }
#pragma unroll
          for (int u = 0; u < kBatch; ++u) {
            const int e = e0 + u * kThreads;
            const int r = e / k4s, k = (e - r * k4s) * 4;
            if (e < n4) *reinterpret_cast<float4*>(sA + r * lda + k) = v[u];
          }
        }
      }
      __syncthreads();

      // ---- this group's chunks of K, in the level kernel's order.  One warp per group multiplies:
      // a lane holds 4 rows x 8 columns of the tile, so 12 shared-memory loads feed 128 FMAs (the
      // level kernel's 2 x 4 per thread needs 6 per 32 and is bound by shared-memory bandwidth).
      // Every partial sum is still one chain over the group's K range in ascending order.
      if ((tid >> 5) == grp * 5) {  // warps 0, 5, 10, 15: one per scheduler
        const int lane = tid & 31;
        const int cx = lane & 3;   // columns 8 cx .. 8 cx + 7
        const int ry = lane >> 2;  // rows 4 ry .. 4 ry + 3
        const int total_chunks = Kt / TK;
        const int c_begin = total_chunks * grp / kSplitK, c_end = total_chunks * (grp + 1) / kSplitK;
        float acc[4][8] = {};
        const float* Ar = sA + (4 * ry) * lda;
        const float* Wc = sW + 8 * cx;
        for (int k0 = c_begin * TK; k0 < c_end * TK; k0 += 4) {
          float av[4][4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 r = *reinterpret_cast<const float4*>(Ar + i * lda + k0);
            av[i][0] = r.x; av[i][1] = r.y; av[i][2] = r.z; av[i][3] = r.w;
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 w0 = *reinterpret_cast<const float4*>(Wc + (k0 + q) * ldw);
            const float4 w1 = *reinterpret_cast<const float4*>(Wc + (k0 + q) * ldw + 4);
            const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int c = 0; c < 8; ++c) acc[i][c] = fmaf(av[i][q], wv[c], acc[i][c]);
          }
        }
        float* p = sP + static_cast<size_t>(grp) * TM * TN + (4 * ry) * TN + 8 * cx;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          *reinterpret_cast<float4*>(p + i * TN) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
          *reinterpret_cast<float4*>(p + i * TN + 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
        }
      }
      __syncthreads();

      // ---- group 0: the four partial sums added in group order, then the cell
      if (grp == 0) {
        float acc[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float* p = sP + (2 * ty + i) * TN + 4 * tx;
          float4 v = *reinterpret_cast<const float4*>(p);
#pragma unroll
          for (int g = 1; g < kSplitK; ++g) {
            const float4 pg = *reinterpret_cast<const float4*>(p + g * TM * TN);
            v.x += pg.x; v.y += pg.y; v.z += pg.z; v.w += pg.w;
          }
          acc[i][0] = v.x; acc[i][1] = v.y; acc[i][2] = v.z; acc[i][3] = v.w;
        }
        const int unit = col0 >> 2;
        float* out = a.hs + (static_cast<size_t>(l) * a.L + t) * a.N * a.H;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int row = row0 + 2 * ty + i;
          if (row >= a.N) continue;
          const float gi = sigmoid_acc(acc[i][0] + b.x);
          const float gf = sigmoid_acc(acc[i][1] + b.y);
          const float go = sigmoid_acc(acc[i][2] + b.z);
          const float gc = tanhf(acc[i][3] + b.w);
          const float cn = gf * creg[i] + gi * gc;
          creg[i] = cn;
          __stcg(out + static_cast<size_t>(row) * a.H + unit, go * tanhf(cn));
        }
        // ---- publish: all of group 0's stores, then one release by its first thread
        __threadfence();
        group_barrier(0);
        if (tg == 0) red_release_gpu_add(a.done + l * a.L + t, 1);
      }
    }
    // Final cell state of the sweep.
    if (grp == 0) {
      const int unit = col0 >> 2;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int row = row0 + 2 * ty + i;
        if (row < a.N) a.c[(static_cast<size_t>(l) * a.N + row) * a.H + unit] = creg[i];
      }
    }
    __syncthreads();  // the next layer's weights overwrite sW
  }
}

size_t smem_bytes(int I, int H) {
  const size_t K = static_cast<size_t>(I) + H;
  return (K * (TN + 4) + TM * (K + 4) + kSplitK * TM * TN) * sizeof(float);
}

}  // namespace

// True when the persistent fp32 kernel can run the problem: a tile's weights and operands fit in
// shared memory and at least one layer's tiles fit on the device at one CTA per SM.
bool lstm_simt_static_supported(int D, int N, int I, int H, int sm_count) {
  if (H % 64 != 0 || I % 64 != 0 || (D > 1 && I != H)) return false;
  if (smem_bytes(I, H) > static_cast<size_t>(kMaxSmem)) return false;
  const long long tiles = static_cast<long long>((N + TM - 1) / TM) * (4 * H / TN);
  return tiles <= sm_count;
}

// x: [L,N,I]; Wp: [D,4H,I+H] fp32 packed; hs: [D,L,N,H]; c: [D,N,H]; done: D*L ints (zeroed here).
int launch_lstm_simt_static(const float* x, const float* Wp, const float* bias_p, float* hs, float* c, int D, int L,
                            int N, int I, int H, int* done, int* status, int sm_count, cudaStream_t stream) {
  SimtStaticArgs a;
  a.x = x;
  a.w = Wp;
  a.bias = bias_p;
  a.hs = hs;
  a.c = c;
  a.done = done;
  a.status = status;
  a.D = D; a.L = L; a.N = N; a.I = I; a.H = H;
  a.m_tiles = (N + TM - 1) / TM;
  a.n_tiles = 4 * H / TN;
  const int tiles = a.m_tiles * a.n_tiles;
  a.G = sm_count / tiles;
  if (a.G < 1) return FTB_ERR_ARG;
  if (a.G > D) a.G = D;
  if (cudaMemsetAsync(done, 0, sizeof(int) * static_cast<size_t>(D) * L, stream) != cudaSuccess) return FTB_ERR_LAUNCH;
  static std::atomic<unsigned long long> configured{0};
  if (!ensure_dynamic_smem(lstm_simt_static_kernel, kMaxSmem, configured)) return FTB_ERR_LAUNCH;
  // FTB_REFUSE_COOPERATIVE=1 makes this function answer as if the driver had refused the
  // cooperative launch (host-side failure injection for the schedule fallback's tests).
  {
    const char* e = getenv("FTB_REFUSE_COOPERATIVE");
    if (e != nullptr && e[0] == '1') return FTB_ERR_LAUNCH;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.G * tiles);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem_bytes(I, H);
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int na = 0;
  // FTB_NO_COOPERATIVE=1 drops the cooperative attribute (profilers that cannot replay
  // cooperative launches); residency then rests on grid <= SM count on an otherwise idle device.
  static const bool no_coop = [] {
    const char* e = getenv("FTB_NO_COOPERATIVE");
    return e != nullptr && e[0] == '1';
  }();
  if (!no_coop) {
    attrs[na].id = cudaLaunchAttributeCooperative;
    attrs[na].val.cooperative = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  if (cudaLaunchKernelEx(&cfg, lstm_simt_static_kernel, a) != cudaSuccess) {
    cudaGetLastError();
    return FTB_ERR_LAUNCH;
  }
  count_launch();
  return FTB_OK;
}

}  // namespace ftb
