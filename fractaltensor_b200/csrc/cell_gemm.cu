// Fused RNN cell kernel for 16-bit activations on sm_100a.
//
// One persistent CTA per SM walks tiles.  A tile is 128 activation rows (batch
// entries; UMMA M) by BN accumulator columns (UMMA N) of one cell.  Warp roles:
//   warp 0      TMA producer: activation and weight K blocks into a shared-memory ring
//   warp 1      tcgen05.mma issuer (one lane); owns the TMEM allocation
//   warps 2..5  epilogue: tcgen05.ld of the finished accumulator, gate maths in
//               registers, stores of h (16-bit) and c (fp32)
// Two accumulator stages in TMEM let the epilogue of tile i overlap the MMAs of
// tile i+1.
//
// Two scheduling modes share the kernel body:
//   level mode       one launch per wavefront level; the level's cells arrive as a
//                    kernel parameter; no CTA ever waits on another CTA.
//   persistent mode  one cooperative launch for the whole wavefront; the cells sit
//                    in global memory in an order in which every cell only depends
//                    on earlier ones; a tile's producer waits (bounded) on the
//                    completion counters of the cells whose output it reads, the
//                    epilogue bumps the counter of its own cell.
//
// PAIR variants run CTAs as pairs (cluster of 2, tcgen05 cta_group::2): the two
// CTAs of a pair work on the two 128-row halves of a 256-row block with the same
// weight tile, each loading only half of that weight tile, which cuts the
// L2 -> shared-memory traffic per FLOP by a third and deepens the ring.
//
// Replaces the role of KeCuteLSTMGate + KeLSTMElementWise
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

template <int BN, bool PAIR>
struct Cfg {
  static constexpr int kBRows = PAIR ? BN / 2 : BN;  // weight rows this CTA loads per K block
  static constexpr uint32_t kABytes = BM * BK * 2;
  static constexpr uint32_t kBBytes = kBRows * BK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (196608 / kStageBytes) > 8 ? 8 : (196608 / kStageBytes);
  static constexpr uint32_t kTxBytes = PAIR ? 2 * kStageBytes : kStageBytes;  // counted on the leader's barrier
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr uint32_t kTmemCols = 2 * BN;
};

// Walks the item list as the tile index grows (tiles are visited in increasing
// order by every role).
template <bool PERSIST>
struct ItemCursor {
  const CellItem* items;
  int n_items;
  int idx;
  __device__ ItemCursor(const CellBatch& b, const PlanView& p) : n_items(b.n_items), idx(0) {
    items = PERSIST ? p.items : b.items;
  }
  __device__ __forceinline__ const CellItem* seek(int tile) {
    while (idx + 1 < n_items && tile >= items[idx + 1].tile0) ++idx;
    return items + idx;
  }
};

template <typename T>
__device__ __forceinline__ void store8(T* dst, const float (&v)[8]) {
  uint4 u;
  u.x = Fmt<T>::pack2(v[0], v[1]);
  u.y = Fmt<T>::pack2(v[2], v[3]);
  u.z = Fmt<T>::pack2(v[4], v[5]);
  u.w = Fmt<T>::pack2(v[6], v[7]);
  *reinterpret_cast<uint4*>(dst) = u;
}

template <typename T, int BN, int EPI, bool PERSIST, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
cell_gemm_kernel(const __grid_constant__ CUtensorMap mapA0, const __grid_constant__ CUtensorMap mapA1,
                 const __grid_constant__ CUtensorMap mapA2, const __grid_constant__ CUtensorMap mapW,
                 const __grid_constant__ CellBatch batch, const PlanView plan, int* __restrict__ status) {
  using C = Cfg<BN, PAIR>;
  constexpr int S = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[S];
  __shared__ uint64_t empty_bar[S];
  __shared__ uint64_t tfull_bar[2];
  __shared__ uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t peer_tmem_base_s;
  __shared__ int s_abort;

  // A launch that follows a failed one does nothing.  (Not for pairs: both CTAs of
  // a pair must take the same path, and the persistent schedule is a single launch.)
  if (!PAIR && *reinterpret_cast<volatile int*>(status) != 0) return;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // 0 = the pair's leader: it issues the MMAs
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
    // The leader's accumulator is released by the epilogue warps of both CTAs.
    mbar_init(&tempty_bar[0], PAIR ? 8 : 4);
    mbar_init(&tempty_bar[1], PAIR ? 8 : 4);
    s_abort = 0;
    peer_tmem_base_s = 0xffffffffu;
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
  const int total = batch.total_tiles;
  if (PAIR) {
    // Both CTAs of a pair must hold their accumulators at the same TMEM columns.
    if (threadIdx.x == 0 && rank == 1) st_shared_cluster_u32(map_to_cta(smem_u32(&peer_tmem_base_s), 0), tmem_base);
    cluster_sync_all();
    if (rank == 0 && threadIdx.x == 0 && peer_tmem_base_s != tmem_base) {
      s_abort = 1;
      atomicCAS(status, 0, FTB_ERR_TMEM_LAYOUT);
    }
    __syncthreads();
  }

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      ItemCursor<PERSIST> cur(batch, plan);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const CellItem* it = cur.seek(tile);
        const int local = tile - it->tile0;
        const int mt = it->m_tiles;
        const int n_tile = local / mt;
        const int m_tile = local - n_tile * mt;
        const int w_row = it->w_row0 + n_tile * BN + static_cast<int>(rank) * C::kBRows;
        const int nseg = it->nseg;
        for (int s = 0; s < nseg && ok; ++s) {
          if (PERSIST) {
            // The rows this segment reads are written by earlier cells: wait for them.
            const int lo = plan.dep[(cur.idx * kMaxSeg + s) * 2 + 0];
            const int hi = plan.dep[(cur.idx * kMaxSeg + s) * 2 + 1];
            for (int d = lo; d >= 0 && d <= hi && ok; ++d)
              ok = flag_wait_ge(plan.done + d, plan.target[d], &s_abort, status, FTB_ERR_TIMEOUT_DEP);
            if (!ok) break;
            fence_proxy_async_all();
          }
          const int mi = it->seg_map[s];
          const CUtensorMap* am = (mi == 0) ? &mapA0 : ((mi == 1) ? &mapA1 : &mapA2);
          const int a_row = it->seg_row[s] + m_tile * BM;
          const int wk = it->seg_wk[s];
          const int nkb = it->seg_kb[s];
          for (int kb = 0; kb < nkb; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_SLOT)) {
              ok = false;
              break;
            }
            uint8_t* sa = smem + stage * C::kStageBytes;
            uint8_t* sb = sa + C::kABytes;
            if (PAIR) {
              // Both CTAs' copies are counted on the leader's barrier; only the leader arms it.
              const uint32_t lead_bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
              if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], C::kTxBytes);
              tma_load_2d_pair(sa, am, lead_bar, kb * BK, a_row);
              tma_load_2d_pair(sb, &mapW, lead_bar, wk + kb * BK, w_row);
            } else {
              mbar_arrive_expect_tx(&full_bar[stage], C::kTxBytes);
              tma_load_2d(sa, am, &full_bar[stage], kb * BK, a_row);
              tma_load_2d(sb, &mapW, &full_bar[stage], wk + kb * BK, w_row);
            }
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
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_f16(PAIR ? 2 * BM : BM, BN, Fmt<T>::kind, 0, 0);
      ItemCursor<PERSIST> cur(batch, plan);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const CellItem* it = cur.seek(tile);
        int nkb = 0;
        for (int s = 0; s < it->nseg; ++s) nkb += it->seg_kb[s];
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
            if (PAIR)
              umma_ss_pair(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
            else
              umma_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if (PAIR)
            umma_commit_pair(&empty_bar[stage]);
          else
            umma_commit(&empty_bar[stage]);
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (PAIR)
          umma_commit_pair(&tfull_bar[acc]);
        else
          umma_commit(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    ItemCursor<PERSIST> cur(batch, plan);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
      const CellItem* it = cur.seek(tile);
      const int local = tile - it->tile0;
      const int mt = it->m_tiles;
      const int n_tile = local / mt;
      const int m_tile = local - n_tile * mt;
      const int row = m_tile * BM + q * 32 + lane;
      const bool row_ok = row < it->rows;
      const bool c_zero = it->c_zero != 0;
      const float* bias = it->bias;
      float* c_row = it->c + static_cast<size_t>(row) * batch.ld_c;
      T* out_row = reinterpret_cast<T*>(it->out) + static_cast<size_t>(row) * batch.ld_out;
      const int col_base = n_tile * BN;

      // LSTM: fetch this thread's slice of the previous cell state now, while the
      // main loop of the tile is still running, so that the L2 latency is off the
      // path between the last MMA and the stores.
      float cpre[(EPI == EPI_LSTM) ? BN / 4 : 1];
      if (EPI == EPI_LSTM) {
        bool dep_ok = true;
        if (PERSIST && !c_zero) {
          // c was written by the cell this tile's last segment depends on.
          const int s_last = it->nseg - 1;
          const int lo = plan.dep[(cur.idx * kMaxSeg + s_last) * 2 + 0];
          const int hi = plan.dep[(cur.idx * kMaxSeg + s_last) * 2 + 1];
          if (lane == 0) {
            for (int d = lo; d >= 0 && d <= hi && dep_ok; ++d)
              dep_ok = flag_wait_ge(plan.done + d, plan.target[d], &s_abort, status, FTB_ERR_TIMEOUT_DEP);
          }
          dep_ok = __all_sync(0xffffffffu, dep_ok);
        }
        if (!dep_ok) break;
        const int unit_base = col_base >> 2;
#pragma unroll
        for (int v = 0; v < BN / 16; ++v) {
          float4 cv = make_float4(0.f, 0.f, 0.f, 0.f);
          // L2 loads: the previous step of this cell may have run on another SM.
          if (row_ok && !c_zero && col_base + 16 * v + 16 <= batch.n_cols)
            cv = __ldcg(reinterpret_cast<const float4*>(c_row + unit_base) + v);
          cpre[4 * v + 0] = cv.x; cpre[4 * v + 1] = cv.y; cpre[4 * v + 2] = cv.z; cpre[4 * v + 3] = cv.w;
        }
      }

      // Warp-uniform outcome: tcgen05.ld below needs all 32 lanes.
      if (!__all_sync(0xffffffffu, mbar_wait(&tfull_bar[acc], acc_phase, &s_abort, status, FTB_ERR_TIMEOUT_MMA)))
        break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll
      for (int ch = 0; ch < BN / 32; ++ch) {
        uint32_t r[32];
        tmem_ld32(taddr + ch * 32, r);
        tmem_ld_wait();
        const int col0 = col_base + ch * 32;
        if (col0 + 32 > batch.n_cols) continue;
        if (EPI == EPI_LSTM) {
          const int unit0 = col0 >> 2;
          float cprev[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) cprev[j] = cpre[(EPI == EPI_LSTM) ? 8 * ch + j : 0];
          float cn[8], hn[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float gi = __uint_as_float(r[4 * j + 0]);
            float gf = __uint_as_float(r[4 * j + 1]);
            float go = __uint_as_float(r[4 * j + 2]);
            float gc = __uint_as_float(r[4 * j + 3]);
            if (bias != nullptr) {
              const float4 b = __ldg(reinterpret_cast<const float4*>(bias + col0) + j);
              gi += b.x; gf += b.y; go += b.z; gc += b.w;
            }
            const float c_new = sigmoid_fast(gf) * cprev[j] + sigmoid_fast(gi) * tanh_fast(gc);
            cn[j] = c_new;
            hn[j] = sigmoid_fast(go) * tanh_fast(c_new);
          }
          if (row_ok) {
            __stcg(reinterpret_cast<float4*>(c_row + unit0), make_float4(cn[0], cn[1], cn[2], cn[3]));
            __stcg(reinterpret_cast<float4*>(c_row + unit0) + 1, make_float4(cn[4], cn[5], cn[6], cn[7]));
            store8<T>(out_row + unit0, hn);
          }
        } else {
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float x = __uint_as_float(r[8 * g + j]);
                if (EPI == EPI_TANH) {
                  if (bias != nullptr) x += __ldg(bias + col0 + 8 * g + j);
                  x = tanh_fast(x);
                }
                v[j] = x;
              }
              store8<T>(out_row + col0 + 8 * g, v);
            }
          }
        }
      }
      tc_fence_before();
      if (PERSIST) {
        // Publish this warp's rows: plain stores -> visible to other CTAs' TMA loads.
        fence_proxy_async_all();
        __threadfence();
      }
      __syncwarp();
      if (lane == 0) {
        if (PAIR)
          mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
        else
          mbar_arrive(&tempty_bar[acc]);
        if (PERSIST) red_release_gpu_add(plan.done + cur.idx, 1);
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  // Neither CTA of a pair may leave while the other can still signal its barriers.
  if (PAIR) cluster_sync_all();
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

template <typename T, int BN, int EPI, bool PERSIST, bool PAIR>
int launch_one(const CUtensorMap* maps, const CUtensorMap& mapW, const CellBatch& batch, const PlanView& plan,
               int* status, int sm_count, cudaStream_t stream) {
  using C = Cfg<BN, PAIR>;
  static bool configured = false;
  auto kfn = cell_gemm_kernel<T, BN, EPI, PERSIST, PAIR>;
  if (!configured) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess)
      return FTB_ERR_LAUNCH;
    configured = true;
  }
  int grid = batch.total_tiles < sm_count ? batch.total_tiles : sm_count;
  if (PAIR) grid &= ~1;  // whole pairs only; tiles 2p and 2p+1 are the two halves of one row block
  if (grid <= 0) return FTB_OK;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (PAIR) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = 2;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = 1;
    ++na;
  }
  if (PERSIST) {
    // Cooperative launch: every CTA is resident, so a CTA that waits on another
    // CTA's counter always makes progress.
    attrs[na].id = cudaLaunchAttributeCooperative;
    attrs[na].val.cooperative = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  if (cudaLaunchKernelEx(&cfg, kfn, maps[0], maps[1], maps[2], mapW, batch, plan, status) != cudaSuccess) {
    cudaGetLastError();
    return FTB_ERR_LAUNCH;
  }
  count_launch();
  return FTB_OK;
}

template <typename T, int BN, bool PERSIST, bool PAIR>
int launch_epi(int epi, const CUtensorMap* maps, const CUtensorMap& mapW, const CellBatch& batch,
               const PlanView& plan, int* status, int sm_count, cudaStream_t stream) {
  switch (epi) {
    case EPI_STORE:
      return launch_one<T, BN, EPI_STORE, PERSIST, PAIR>(maps, mapW, batch, plan, status, sm_count, stream);
    case EPI_LSTM:
      return launch_one<T, BN, EPI_LSTM, PERSIST, PAIR>(maps, mapW, batch, plan, status, sm_count, stream);
    case EPI_TANH:
      return launch_one<T, BN, EPI_TANH, PERSIST, PAIR>(maps, mapW, batch, plan, status, sm_count, stream);
    default: return FTB_ERR_ARG;
  }
}

template <bool PERSIST, bool PAIR>
int launch_any(int dtype, int epi, int bn, const CUtensorMap* maps, const CUtensorMap& mapW, const CellBatch& batch,
               const PlanView& plan, int* status, int sm_count, cudaStream_t stream) {
  if (dtype == FTB_F16) {
    if (bn == 256) return launch_epi<__half, 256, PERSIST, PAIR>(epi, maps, mapW, batch, plan, status, sm_count, stream);
    if (bn == 128) return launch_epi<__half, 128, PERSIST, PAIR>(epi, maps, mapW, batch, plan, status, sm_count, stream);
  } else if (dtype == FTB_BF16) {
    if (bn == 256)
      return launch_epi<__nv_bfloat16, 256, PERSIST, PAIR>(epi, maps, mapW, batch, plan, status, sm_count, stream);
    if (bn == 128)
      return launch_epi<__nv_bfloat16, 128, PERSIST, PAIR>(epi, maps, mapW, batch, plan, status, sm_count, stream);
  }
  return FTB_ERR_ARG;
}

}  // namespace

// Launches one wavefront level.  `maps` are the three activation tensor maps
// (box 128 rows x 64 elements), `mapW` the packed-weight map (box `bn` rows x 64
// elements, or bn/2 rows when `pair` is set).  With `pair`, every item's m_tiles
// must be even.
int launch_cell_gemm(int dtype, int epi, int bn, int pair, const CUtensorMap* maps, const CUtensorMap& mapW,
                     const CellBatch& batch, int* status, int sm_count, cudaStream_t stream) {
  PlanView none = {nullptr, nullptr, nullptr, nullptr};
  if (pair) return launch_any<false, true>(dtype, epi, bn, maps, mapW, batch, none, status, sm_count, stream);
  return launch_any<false, false>(dtype, epi, bn, maps, mapW, batch, none, status, sm_count, stream);
}

// Launches a whole wavefront as one persistent kernel.  `header` carries n_items,
// n_cols, ld_out, ld_c and total_tiles; its items[] are ignored (they live in
// plan.items in global memory).
int launch_cell_gemm_persistent(int dtype, int epi, int bn, int pair, const CUtensorMap* maps,
                                const CUtensorMap& mapW, const CellBatch& header, const PlanView& plan, int* status,
                                int sm_count, cudaStream_t stream) {
  if (pair) return launch_any<true, true>(dtype, epi, bn, maps, mapW, header, plan, status, sm_count, stream);
  return launch_any<true, false>(dtype, epi, bn, maps, mapW, header, plan, status, sm_count, stream);
}

}  // namespace ftb
