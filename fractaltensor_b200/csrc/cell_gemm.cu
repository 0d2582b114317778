// Fused RNN cell kernel for 16-bit activations on sm_100a.
//
// One persistent CTA per SM walks the tiles of a launch.  A tile is 128
// activation rows (batch entries; UMMA M) by BN accumulator columns (UMMA N) of
// one cell.  Warp roles:
//   warp 0      TMA producer: activation and weight K blocks into a shared-memory ring
//   warp 1      tcgen05.mma issuer (one lane); owns the TMEM allocation
//   warps 2..5  epilogue: tcgen05.ld of the finished accumulator, gate maths in
//               registers, stores of h (16-bit) and c (fp32)
// Two accumulator stages in TMEM let the epilogue of tile i overlap the MMAs of
// tile i+1.  Replaces the role of KeCuteLSTMGate + KeLSTMElementWise
// (kaleido/core/device/kernels/lstm_kernels.h:24-126, lstm/inner.h:594-662) and
// of VanillaRNNCellBMM (benchmarks/rnn/fractaltensor/utils.h:627-700); it is a
// new design, not a translation of them.
#include "cell.h"
#include "ptx.cuh"
#include "tmap.h"

namespace ftb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 192;

template <int BN>
struct Cfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr uint32_t kABytes = BM * BK * 2;
  static constexpr uint32_t kBBytes = BN * BK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr uint32_t kTmemCols = 2 * BN;
};

struct TileCoord {
  int item, m_tile, n_tile;
};

__device__ __forceinline__ TileCoord decode_tile(const CellBatch& b, int tile, int n_tiles_n) {
  int it = 0;
#pragma unroll 1
  for (int i = 1; i < b.n_items; ++i) {
    if (tile >= b.items[i].tile0) it = i;
  }
  const int local = tile - b.items[it].tile0;
  const int mt = b.items[it].m_tiles;
  TileCoord tc;
  tc.item = it;
  tc.n_tile = local / mt;
  tc.m_tile = local - tc.n_tile * mt;
  (void)n_tiles_n;
  return tc;
}

template <typename T>
__device__ __forceinline__ void store8(T* dst, const float (&v)[8]) {
  uint4 u;
  u.x = Fmt<T>::pack2(v[0], v[1]);
  u.y = Fmt<T>::pack2(v[2], v[3]);
  u.z = Fmt<T>::pack2(v[4], v[5]);
  u.w = Fmt<T>::pack2(v[6], v[7]);
  *reinterpret_cast<uint4*>(dst) = u;
}

template <typename T, int BN, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
cell_gemm_kernel(const __grid_constant__ CUtensorMap mapA0, const __grid_constant__ CUtensorMap mapA1,
                 const __grid_constant__ CUtensorMap mapA2, const __grid_constant__ CUtensorMap mapW,
                 const __grid_constant__ CellBatch batch, int* __restrict__ status) {
  using C = Cfg<BN>;
  constexpr int S = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[S];
  __shared__ uint64_t empty_bar[S];
  __shared__ uint64_t tfull_bar[2];
  __shared__ uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

  // A launch that follows a failed one does nothing.
  if (*reinterpret_cast<volatile int*>(status) != 0) return;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

  if (threadIdx.x == 0) {
    prefetch_tmap(&mapA0);
    prefetch_tmap(&mapA1);
    prefetch_tmap(&mapA2);
    prefetch_tmap(&mapW);
    for (int i = 0; i < S; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tfull_bar[1], 1);
    mbar_init(&tempty_bar[0], 4);
    mbar_init(&tempty_bar[1], 4);
    s_abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  const int n_tiles_n = (batch.n_cols + BN - 1) / BN;
  const int total = batch.total_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const TileCoord tc = decode_tile(batch, tile, n_tiles_n);
        const CellItem& it = batch.items[tc.item];
        const int w_row = it.w_row0 + tc.n_tile * BN;
        for (int s = 0; s < it.nseg && ok; ++s) {
          const int mi = it.seg_map[s];
          const CUtensorMap* am = (mi == 0) ? &mapA0 : ((mi == 1) ? &mapA1 : &mapA2);
          const int a_row = it.seg_row[s] + tc.m_tile * BM;
          const int wk = it.seg_wk[s];
          const int nkb = it.seg_kb[s];
          for (int kb = 0; kb < nkb; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_SLOT)) {
              ok = false;
              break;
            }
            uint8_t* sa = smem + stage * C::kStageBytes;
            uint8_t* sb = sa + C::kABytes;
            mbar_arrive_expect_tx(&full_bar[stage], C::kStageBytes);
            tma_load_2d(sa, am, &full_bar[stage], kb * BK, a_row);
            tma_load_2d(sb, &mapW, &full_bar[stage], wk + kb * BK, w_row);
            if (++stage == S) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(BM, BN, Fmt<T>::kind, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const TileCoord tc = decode_tile(batch, tile, n_tiles_n);
        const CellItem& it = batch.items[tc.item];
        int nkb = 0;
        for (int s = 0; s < it.nseg; ++s) nkb += it.seg_kb[s];
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_EPI)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, &s_abort, status, FTB_ERR_TIMEOUT_TMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = make_sdesc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bd = make_sdesc_sw128(sb + k * 32, 16, 1024);
            umma_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
      const TileCoord tc = decode_tile(batch, tile, n_tiles_n);
      const CellItem& it = batch.items[tc.item];
      // Warp-uniform outcome: tcgen05.ld below needs all 32 lanes.
      if (!__all_sync(0xffffffffu, mbar_wait(&tfull_bar[acc], acc_phase, &s_abort, status, FTB_ERR_TIMEOUT_MMA)))
        break;
      tc_fence_after();
      const int row = tc.m_tile * BM + q * 32 + lane;
      const bool row_ok = row < it.rows;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const int col_base = tc.n_tile * BN;
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        uint32_t r[32];
        tmem_ld32(taddr + ch * 32, r);
        tmem_ld_wait();
        const int col0 = col_base + ch * 32;
        if (col0 + 32 > batch.n_cols) continue;
        if (EPI == EPI_LSTM) {
          const int unit0 = col0 >> 2;
          float cprev[8];
          if (row_ok && !it.c_zero) {
            const float4* cp = reinterpret_cast<const float4*>(it.c + static_cast<size_t>(row) * batch.ld_c + unit0);
            float4 c0 = cp[0], c1 = cp[1];
            cprev[0] = c0.x; cprev[1] = c0.y; cprev[2] = c0.z; cprev[3] = c0.w;
            cprev[4] = c1.x; cprev[5] = c1.y; cprev[6] = c1.z; cprev[7] = c1.w;
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) cprev[j] = 0.f;
          }
          float cn[8], hn[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float gi = __uint_as_float(r[4 * j + 0]);
            float gf = __uint_as_float(r[4 * j + 1]);
            float go = __uint_as_float(r[4 * j + 2]);
            float gc = __uint_as_float(r[4 * j + 3]);
            if (it.bias != nullptr) {
              const float4 b = __ldg(reinterpret_cast<const float4*>(it.bias + col0) + j);
              gi += b.x; gf += b.y; go += b.z; gc += b.w;
            }
            const float c_new = sigmoid_fast(gf) * cprev[j] + sigmoid_fast(gi) * tanh_fast(gc);
            cn[j] = c_new;
            hn[j] = sigmoid_fast(go) * tanh_fast(c_new);
          }
          if (row_ok) {
            float4* cp = reinterpret_cast<float4*>(it.c + static_cast<size_t>(row) * batch.ld_c + unit0);
            cp[0] = make_float4(cn[0], cn[1], cn[2], cn[3]);
            cp[1] = make_float4(cn[4], cn[5], cn[6], cn[7]);
            store8<T>(reinterpret_cast<T*>(it.out) + static_cast<size_t>(row) * batch.ld_out + unit0, hn);
          }
        } else {
          if (row_ok) {
            T* o = reinterpret_cast<T*>(it.out) + static_cast<size_t>(row) * batch.ld_out + col0;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float x = __uint_as_float(r[8 * g + j]);
                if (EPI == EPI_TANH) {
                  if (it.bias != nullptr) x += __ldg(it.bias + col0 + 8 * g + j);
                  x = tanh_fast(x);
                }
                v[j] = x;
              }
              store8<T>(o + 8 * g, v);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (s_abort) {
      // Give copies and MMAs still in flight time to land before TMEM and
      // shared memory are handed back.
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <typename T, int BN, int EPI>
int launch_one(const CUtensorMap* maps, const CUtensorMap& mapW, const CellBatch& batch, int* status, int sm_count,
               cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool configured = false;
  auto kfn = cell_gemm_kernel<T, BN, EPI>;
  if (!configured) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess)
      return FTB_ERR_LAUNCH;
    configured = true;
  }
  int grid = batch.total_tiles < sm_count ? batch.total_tiles : sm_count;
  if (grid <= 0) return FTB_OK;
  kfn<<<grid, kThreads, C::kSmemBytes, stream>>>(maps[0], maps[1], maps[2], mapW, batch, status);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
}

template <typename T, int BN>
int launch_epi(int epi, const CUtensorMap* maps, const CUtensorMap& mapW, const CellBatch& batch, int* status,
               int sm_count, cudaStream_t stream) {
  switch (epi) {
    case EPI_STORE: return launch_one<T, BN, EPI_STORE>(maps, mapW, batch, status, sm_count, stream);
    case EPI_LSTM: return launch_one<T, BN, EPI_LSTM>(maps, mapW, batch, status, sm_count, stream);
    case EPI_TANH: return launch_one<T, BN, EPI_TANH>(maps, mapW, batch, status, sm_count, stream);
    default: return FTB_ERR_ARG;
  }
}

}  // namespace

// Launches one wavefront level.  `maps` are the three activation tensor maps
// (box 128 rows x 64 elements), `mapW` the packed-weight map (box `bn` rows x
// 64 elements).
int launch_cell_gemm(int dtype, int epi, int bn, const CUtensorMap* maps, const CUtensorMap& mapW,
                     const CellBatch& batch, int* status, int sm_count, cudaStream_t stream) {
  if (dtype == FTB_F16) {
    if (bn == 256) return launch_epi<__half, 256>(epi, maps, mapW, batch, status, sm_count, stream);
    if (bn == 128) return launch_epi<__half, 128>(epi, maps, mapW, batch, status, sm_count, stream);
  } else if (dtype == FTB_BF16) {
    if (bn == 256) return launch_epi<__nv_bfloat16, 256>(epi, maps, mapW, batch, status, sm_count, stream);
    if (bn == 128) return launch_epi<__nv_bfloat16, 128>(epi, maps, mapW, batch, status, sm_count, stream);
  }
  return FTB_ERR_ARG;
}

}  // namespace ftb
