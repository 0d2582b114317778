// Fused RNN cell kernel for 16-bit activations on sm_100a.
//
// One persistent CTA per SM walks tiles.  A tile is 128 activation rows (batch
// entries; UMMA M) by BN accumulator columns (UMMA N) of one cell.  Warp roles:
//   warp 0      TMA producer: activation and weight K blocks into a shared-memory ring
//   warp 1      tcgen05.mma issuer (one lane); owns the TMEM allocation
//   warps 2..9  epilogue: tcgen05.ld of the finished accumulator, gate maths in
//               registers, hidden state straight to global memory (the next cells
//               wait for it), new cell state into a shared-memory staging tile
//   warp 10     (LSTM) cell-state traffic: TMA load of the tile's previous cell state
//               into the staging tile while the main loop runs, TMA store of the
//               new one, cell-state completion counter
// Two accumulator stages in TMEM let the epilogue of tile i overlap the MMAs of
// tile i+1.
//
// Two scheduling modes share the kernel body:
//   level mode       one launch per wavefront level; the level's cells arrive as a
//                    kernel parameter; no CTA ever waits on another CTA.
//   persistent mode  one cooperative launch for the whole wavefront; the cells sit
//                    in global memory in an order in which every cell only depends
//                    on earlier ones; a tile's producer waits (bounded) on the
//                    completion counters of the cells whose output it reads, and
//                    the cell's own counter is bumped once its outputs are written.
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
#include <cstdlib>

#include "cell.h"
#include "ptx.cuh"
#include "tmap.h"

namespace ftb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kEpiWarps = 8;

template <int BN, int EPI, bool PAIR>
struct Cfg {
  static constexpr bool kStaged = (EPI == EPI_LSTM);  // epilogue goes through shared memory + TMA
  static constexpr int kThreads = 32 * (2 + kEpiWarps + (kStaged ? 1 : 0));
  static constexpr int kUnits = BN / 4;  // LSTM units per tile
  static constexpr int kBRows = PAIR ? BN / 2 : BN;  // weight rows this CTA loads per K block
  static constexpr uint32_t kABytes = BM * BK * 2;
  static constexpr uint32_t kBBytes = kBRows * BK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  // Staging: previous/new cell state (fp32, 32-unit boxes of 128 rows x 128 B).
  static constexpr uint32_t kCBoxBytes = BM * 128;
  static constexpr int kCBoxes = kUnits / 32;
  static constexpr uint32_t kCBytes = kStaged ? kCBoxes * kCBoxBytes : 0;
  static constexpr uint32_t kHBytes = 0;
  static constexpr uint32_t kStagingBytes = kCBytes + kHBytes;
  static constexpr uint32_t kRingBudget = 229376 - 2048 - kStagingBytes;
  static constexpr int kStages = (kRingBudget / kStageBytes) > 8 ? 8 : (kRingBudget / kStageBytes);
  static constexpr uint32_t kTxBytes = PAIR ? 2 * kStageBytes : kStageBytes;  // counted on the leader's barrier
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024;
  static constexpr uint32_t kTmemCols = 2 * BN;
  static_assert(kStages >= 2, "ring too shallow");
  static_assert(!kStaged || kUnits % 32 == 0, "LSTM tiles hold whole 32-unit boxes");
};

// Walks the item list as the tile index grows (tiles are visited in increasing
// order by every role).
template <bool PERSIST>
struct ItemCursor {
  const CellItem* items;
  int n_items;
  int idx;
  int tiles_per_item;
  bool first;
  const int32_t* cta_first;
  __device__ ItemCursor(const CellBatch& b, const PlanView& p)
      : n_items(b.n_items), idx(0), tiles_per_item(PERSIST ? p.tiles_per_item : 0), first(true),
        cta_first(PERSIST ? p.cta_first : nullptr) {
    items = PERSIST ? p.items : b.items;
  }
  __device__ __forceinline__ const CellItem* seek(int tile) {
    if (PERSIST && tiles_per_item > 0) {
      idx = tile / tiles_per_item;
      return items + idx;
    }
    if (PERSIST && cta_first != nullptr) {
      // Jump close to the item, then walk the last few steps (every step of a walk through the
      // table is a dependent load from L2).
      const int hint = first ? cta_first[blockIdx.x] : items[idx].skip;
      idx = hint > idx ? hint : idx;
      first = false;
    }
    while (idx + 1 < n_items && tile >= items[idx + 1].tile0) ++idx;
    return items + idx;
  }
};

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 u;
  u.x = Fmt<T>::pack2(v[0], v[1]);
  u.y = Fmt<T>::pack2(v[2], v[3]);
  u.z = Fmt<T>::pack2(v[4], v[5]);
  u.w = Fmt<T>::pack2(v[6], v[7]);
  return u;
}

template <typename T, int BN, int EPI, bool PERSIST, bool PAIR>
__global__ void __launch_bounds__((Cfg<BN, EPI, PAIR>::kThreads), 1)
cell_gemm_kernel(const __grid_constant__ CUtensorMap mapA0, const __grid_constant__ CUtensorMap mapA1,
                 const __grid_constant__ CUtensorMap mapA2, const __grid_constant__ CUtensorMap mapA3,
                 const __grid_constant__ CUtensorMap mapW, const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CellBatch batch,
                 const PlanView plan, int* __restrict__ status) {
  using C = Cfg<BN, EPI, PAIR>;
  constexpr int S = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[S];
  __shared__ uint64_t empty_bar[S];
  __shared__ uint64_t tfull_bar[2];
  __shared__ uint64_t tempty_bar[2];
  __shared__ uint64_t c_full_bar;     // staging holds the tile's previous cell state (and is free to write)
  __shared__ uint64_t stg_ready_bar;  // the four epilogue warps have written the tile's results to staging
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t peer_tmem_base_s;
  __shared__ int s_abort;

  // One launch per level: the next level's launch may be scheduled as SMs free up; it touches no
  // global memory before its own grid_dependency_wait().
  grid_launch_dependents();

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // 0 = the pair's leader: it issues the MMAs
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* s_c = smem + S * C::kStageBytes;  // [kCBoxes][128 rows][128 B], 128-byte swizzled rows

  if (threadIdx.x == 0) {
    prefetch_tmap(&mapA0);
    prefetch_tmap(&mapA1);
    prefetch_tmap(&mapA2);
    prefetch_tmap(&mapA3);
    prefetch_tmap(&mapW);
    if (C::kStaged) prefetch_tmap(&mapC);
    for (int i = 0; i < S; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tfull_bar[1], 1);
    // The leader's accumulator is released by the epilogue warps of both CTAs.
    mbar_init(&tempty_bar[0], PAIR ? 2 * kEpiWarps : kEpiWarps);
    mbar_init(&tempty_bar[1], PAIR ? 2 * kEpiWarps : kEpiWarps);
    mbar_init(&c_full_bar, 1);
    mbar_init(&stg_ready_bar, kEpiWarps);
    s_abort = 0;
    peer_tmem_base_s = 0xffffffffu;
    fence_barrier_init();
  }
  if (warp == 1) {
    // A kernel's tcgen05 instructions all use one .cta_group: pairs allocate as pairs.
    if (PAIR) {
      tmem_alloc_pair(&tmem_base_s, C::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&tmem_base_s, C::kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  // Set-up is done; what follows reads and writes global memory, so the launch before this one
  // must have finished.  A launch that follows a failed one does nothing.  (Not for pairs: both
  // CTAs of a pair must take the same path, and the persistent schedule is a single launch.)
  grid_dependency_wait();
  const bool live = PAIR || *reinterpret_cast<volatile int*>(status) == 0;
  const int total = live ? batch.total_tiles : 0;
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
      // Weights are re-read at every step of a sweep: ask L2 to keep them over the
      // activations that stream through.
      const uint64_t w_policy = l2_policy_evict_last();
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const CellItem* it = cur.seek(tile);
        const int local = tile - it->tile0;
        const int mt = it->m_tiles;
        const int n_tile = local / mt;
        const int m_tile = local - n_tile * mt;
        const int w_row = it->w_row0 + n_tile * BN + static_cast<int>(rank) * C::kBRows;
        const int nseg = it->nseg;
#ifdef FTB_TRACE
        if (PERSIST && plan.trace) plan.trace[tile * 4 + 0] = globaltimer_ns();
#endif
        for (int s = 0; s < nseg && ok; ++s) {
          // Fine-grained schedule: the tile of the producer cell that holds the activation
          // columns of the next K block (same row tile as this one).
          int dep_tile0 = -1, dep_mt = 0, waited_n = -1;
          if (PERSIST) {
            const int lo = plan.dep[(cur.idx * kMaxSeg + s) * 2 + 0];
            const int hi = plan.dep[(cur.idx * kMaxSeg + s) * 2 + 1];
            if (plan.fine) {
              if (lo >= 0) {
                dep_tile0 = plan.items[lo].tile0;
                dep_mt = plan.items[lo].m_tiles;
              }
            } else {
              // The rows this segment reads are written by earlier cells: wait for all of them.
              for (int d = lo; d >= 0 && d <= hi && ok; ++d)
                ok = flag_wait_ge(plan.done + d, plan.target[d], &s_abort, status, FTB_ERR_TIMEOUT_DEP);
              if (!ok) break;
              fence_proxy_async_all();
            }
#ifdef FTB_TRACE
            if (plan.trace && s == nseg - 1 && !plan.fine) plan.trace[tile * 4 + 1] = globaltimer_ns();
#endif
          }
          const int mi = it->seg_map[s];
          const CUtensorMap* am = (mi == 0) ? &mapA0 : ((mi == 1) ? &mapA1 : ((mi == 2) ? &mapA2 : &mapA3));
          // Cells without a cell state (no staging traffic) may read a second weight buffer: its
          // map travels in the otherwise unused cell-state slot.
          const CUtensorMap* wm = (!C::kStaged && it->w_map != 0) ? &mapC : &mapW;
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
            const uint32_t lead_bar = PAIR ? map_to_cta(smem_u32(&full_bar[stage]), 0) : 0u;
            // Weights first: they depend on nothing.
            if (PAIR) {
              // Both CTAs' copies are counted on the leader's barrier; only the leader arms it.
              if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], C::kTxBytes);
              tma_load_2d_pair_hint(sb, wm, lead_bar, wk + kb * BK, w_row, w_policy);
            } else {
              mbar_arrive_expect_tx(&full_bar[stage], C::kTxBytes);
              tma_load_2d_hint(sb, wm, &full_bar[stage], wk + kb * BK, w_row, w_policy);
            }
            if (PERSIST && dep_tile0 >= 0) {
              // Activation columns [64 kb, 64 kb + 64) come from producer tiles up to n_last.
              const int n_last = (kb * BK + BK - 1) / plan.units_per_tile;
              if (n_last > waited_n) {
                // Poll a batch of producer tiles at once; the K loop then runs on without
                // touching the counters until it catches up with them again.
                const int n_total = (nkb * BK + plan.units_per_tile - 1) / plan.units_per_tile;
                const int* flags = plan.tile_done + dep_tile0 + m_tile;
                const uint64_t t0 = globaltimer_ns();
                uint32_t spins = 0;
                while (ok) {
                  const int from = waited_n + 1;
                  const int count = (n_total - from) < 16 ? (n_total - from) : 16;
                  const int got = flags_ready_prefix(flags, dep_mt, from, count, kEpiWarps);
                  if (got > 0) {
                    waited_n = from + got - 1;
                    if (waited_n >= n_last) break;
                    continue;
                  }
                  if (((++spins) & 0x3F) == 0) {
                    if (s_abort) ok = false;
                    if (globaltimer_ns() - t0 > FTB_WAIT_TIMEOUT_NS) {
                      s_abort = 1;
                      atomicCAS(status, 0, FTB_ERR_TIMEOUT_DEP);
                      ok = false;
                    }
                  }
                }
                if (!ok) break;
                fence_acq_rel_gpu();
                fence_proxy_async_all();
#ifdef FTB_TRACE
                if (plan.trace && s == nseg - 1 && waited_n >= n_total - 1) plan.trace[tile * 4 + 1] = globaltimer_ns();
#endif
              }
            }
            if (PAIR)
              tma_load_2d_pair(sa, am, lead_bar, kb * BK, a_row);
            else
              tma_load_2d(sa, am, &full_bar[stage], kb * BK, a_row);
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
      uint32_t stage_off = 0;  // stage * kStageBytes / 16
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // Operand descriptors of stage 0; a stage's are these plus its byte offset / 16 (nothing is rebuilt
      // per MMA: this thread's own instructions are part of a K block's time).
      const uint64_t a_desc0 = make_sdesc_sw128(smem_u32(smem), 16, 1024);
      const uint64_t b_desc0 = make_sdesc_sw128(smem_u32(smem) + C::kABytes, 16, 1024);
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const CellItem* it = cur.seek(tile);
        int nkb = 0;
        for (int s = 0; s < it->nseg; ++s) nkb += it->seg_kb[s];
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_EPI)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          // (No tcgen05 fence after a barrier that TMA completes: it would drain the tensor pipe.)
          if (!mbar_wait(&full_bar[stage], phase, &s_abort, status, FTB_ERR_TIMEOUT_TMA)) {
            ok = false;
            break;
          }
          const uint64_t ad = a_desc0 + stage_off;
          const uint64_t bd = b_desc0 + stage_off;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            if (PAIR)
              umma_ss_pair(d_tmem, ad + 2 * k, bd + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            else
              umma_ss(d_tmem, ad + 2 * k, bd + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if (PAIR)
            umma_commit_pair(&empty_bar[stage]);
          else
            umma_commit(&empty_bar[stage]);
          stage_off += C::kStageBytes >> 4;
          if (++stage == S) {
            stage = 0;
            stage_off = 0;
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
  } else if (warp < 2 + kEpiWarps) {
    // ---------------------------------------------------------------- epilogue
    // Eight warps: warp w reads TMEM lane quadrant w % 4; the two warps of a quadrant
    // split the tile's 32-column chunks between them.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int kChunks = BN / 32;
    constexpr int kChunksPerWarp = kChunks / 2;
    const int r_loc = q * 32 + lane;  // row inside the tile
    ItemCursor<PERSIST> cur(batch, plan);
    int acc = 0;
    uint32_t acc_phase = 0, stg_phase = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
      const CellItem* it = cur.seek(tile);
      const int local = tile - it->tile0;
      const int mt = it->m_tiles;
      const int n_tile = local / mt;
      const int m_tile = local - n_tile * mt;
      const int row = m_tile * BM + r_loc;
      const int rows = it->rows;
      const bool row_ok = row < rows;
      const float* bias = it->bias;
      const int col_base = n_tile * BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      T* out_row = reinterpret_cast<T*>(it->out) + static_cast<size_t>(row) * batch.ld_out;

      if (C::kStaged) {
        // ---- LSTM.  The cell state travels through the staging tile (TMA in, TMA out); the
        // hidden state, which the next cells are waiting for, goes straight to global memory.
        const bool c_zero = it->c_zero != 0;
        const bool full_tile = (m_tile + 1) * BM <= rows && col_base + BN <= batch.n_cols;
        // Staging is free and holds c(t-1) of this tile (or nothing, when that is zero).
        if (!__all_sync(0xffffffffu, mbar_wait(&c_full_bar, stg_phase, &s_abort, status, FTB_ERR_TIMEOUT_TMA))) break;
        if (!__all_sync(0xffffffffu, mbar_wait(&tfull_bar[acc], acc_phase, &s_abort, status, FTB_ERR_TIMEOUT_MMA)))
          break;
        tc_fence_after();
#ifdef FTB_TRACE
        if (PERSIST && plan.trace && warp == 2 && lane == 0) plan.trace[tile * 4 + 2] = globaltimer_ns();
#endif
        float* c_row = it->c + static_cast<size_t>(row) * batch.ld_c;
        const int sw = r_loc & 7;
#pragma unroll
        for (int cc = 0; cc < kChunksPerWarp; ++cc) {
          const int ch = half * kChunksPerWarp + cc;
          uint32_t r[32];
          tmem_ld32(taddr + ch * 32, r);
          tmem_ld_wait();
          const int col0 = col_base + ch * 32;
          const int unit0 = col0 >> 2;
          // This thread's 8 units of the chunk: two 16-byte pieces of its 128-byte row in box ch/4.
          uint8_t* c_box_row = s_c + (ch >> 2) * C::kCBoxBytes + r_loc * 128;
          float4* c_lo = reinterpret_cast<float4*>(c_box_row + (((2 * (ch & 3)) ^ sw) << 4));
          float4* c_hi = reinterpret_cast<float4*>(c_box_row + (((2 * (ch & 3) + 1) ^ sw) << 4));
          float cprev[8];
          if (c_zero) {
#pragma unroll
            for (int j = 0; j < 8; ++j) cprev[j] = 0.f;
          } else {
            const float4 a = *c_lo, b = *c_hi;
            cprev[0] = a.x; cprev[1] = a.y; cprev[2] = a.z; cprev[3] = a.w;
            cprev[4] = b.x; cprev[5] = b.y; cprev[6] = b.z; cprev[7] = b.w;
          }
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
          const bool cols_ok = col0 + 32 <= batch.n_cols;
          if (row_ok && cols_ok) *reinterpret_cast<uint4*>(out_row + unit0) = pack8<T>(hn);
          if (full_tile) {
            *c_lo = make_float4(cn[0], cn[1], cn[2], cn[3]);
            *c_hi = make_float4(cn[4], cn[5], cn[6], cn[7]);
          } else if (row_ok && cols_ok) {
            // Ragged tile: plain stores of the valid rows only.
            __stcg(reinterpret_cast<float4*>(c_row + unit0), make_float4(cn[0], cn[1], cn[2], cn[3]));
            __stcg(reinterpret_cast<float4*>(c_row + unit0) + 1, make_float4(cn[4], cn[5], cn[6], cn[7]));
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();  // staging writes -> visible to the TMA stores
        if (PERSIST) {
          fence_proxy_async_all();  // plain stores of h -> other CTAs' TMA loads
          __threadfence();
        }
        __syncwarp();
        if (lane == 0) {
          // h of this warp's rows and columns is out: the cells that read it may go.
          if (PERSIST) red_release_gpu_add(plan.fine ? plan.tile_done + tile : plan.done + cur.idx, 1);
#ifdef FTB_TRACE
          if (PERSIST && plan.trace && warp == 2) plan.trace[tile * 4 + 3] = globaltimer_ns();
#endif
          if (PAIR)
            mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
          else
            mbar_arrive(&tempty_bar[acc]);
          mbar_arrive(&stg_ready_bar);
        }
        stg_phase ^= 1u;
      } else {
        // ---- plain / tanh epilogue: straight from registers to global memory
        if (!__all_sync(0xffffffffu, mbar_wait(&tfull_bar[acc], acc_phase, &s_abort, status, FTB_ERR_TIMEOUT_MMA)))
          break;
        tc_fence_after();
#ifdef FTB_TRACE
        if (PERSIST && plan.trace && warp == 2 && lane == 0) plan.trace[tile * 4 + 2] = globaltimer_ns();
#endif
#pragma unroll 1
        for (int cc = 0; cc < kChunksPerWarp; ++cc) {
          const int ch = half * kChunksPerWarp + cc;
          uint32_t r[32];
          tmem_ld32(taddr + ch * 32, r);
          tmem_ld_wait();
          const int col0 = col_base + ch * 32;
          if (col0 + 32 > batch.n_cols || !row_ok) continue;
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
            if (EPI == EPI_STORE_F32) {
              float4* of = reinterpret_cast<float4*>(reinterpret_cast<float*>(it->out) +
                                                     static_cast<size_t>(row) * batch.ld_out + col0 + 8 * g);
              of[0] = make_float4(v[0], v[1], v[2], v[3]);
              of[1] = make_float4(v[4], v[5], v[6], v[7]);
            } else {
              *reinterpret_cast<uint4*>(out_row + col0 + 8 * g) = pack8<T>(v);
            }
          }
        }
        tc_fence_before();
        if (PERSIST) {
          fence_proxy_async_all();
          __threadfence();
        }
        __syncwarp();
        if (lane == 0) {
          if (PERSIST) red_release_gpu_add(plan.fine ? plan.tile_done + tile : plan.done + cur.idx, 1);
#ifdef FTB_TRACE
          if (PERSIST && plan.trace && warp == 2) plan.trace[tile * 4 + 3] = globaltimer_ns();
#endif
          if (PAIR)
            mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
          else
            mbar_arrive(&tempty_bar[acc]);
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  } else if (C::kStaged) {
    // ------------------------------------------- cell-state staging traffic (LSTM)
    if (lane == 0) {
      ItemCursor<PERSIST> cur(batch, plan);
      uint32_t stg_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const CellItem* it = cur.seek(tile);
        const int local = tile - it->tile0;
        const int mt = it->m_tiles;
        const int n_tile = local / mt;
        const int m_tile = local - n_tile * mt;
        const int unit_base = (n_tile * BN) >> 2;
        const bool full_tile = (m_tile + 1) * BM <= it->rows && n_tile * BN + BN <= batch.n_cols;
        const int c_row = it->c_row0 + m_tile * BM;
        // 1. previous cell state of this tile -> staging (the staging tile is free here: the
        //    stores of the previous tile have finished reading it).
        if (!it->c_zero) {
          if (PERSIST) {
            // c(t-1) was written by the cell the last segment depends on; its cell-state
            // counter follows the hidden-state counters in plan.done.
            const int s_last = it->nseg - 1;
            const int lo = plan.dep[(cur.idx * kMaxSeg + s_last) * 2 + 0];
            const int hi = plan.dep[(cur.idx * kMaxSeg + s_last) * 2 + 1];
            if (plan.fine) {
              // Same tile position in the producer cell.
              if (lo >= 0)
                ok = flag_wait_ge(plan.c_done + plan.items[lo].tile0 + n_tile * plan.items[lo].m_tiles + m_tile, 1,
                                  &s_abort, status, FTB_ERR_TIMEOUT_DEP);
            } else {
              for (int d = lo; d >= 0 && d <= hi && ok; ++d)
                ok = flag_wait_ge(plan.done + batch.n_items + d, plan.target[d] / kEpiWarps, &s_abort, status,
                                  FTB_ERR_TIMEOUT_DEP);
            }
            if (!ok) break;
            fence_proxy_async_all();
          }
          mbar_arrive_expect_tx(&c_full_bar, C::kCBytes);
#pragma unroll
          for (int b = 0; b < C::kCBoxes; ++b)
            tma_load_2d(s_c + b * C::kCBoxBytes, &mapC, &c_full_bar, unit_base + 32 * b, c_row);
        } else {
          mbar_arrive(&c_full_bar);
        }
        // 2. new cell state of this tile: staging -> global
        if (!mbar_wait(&stg_ready_bar, stg_phase, &s_abort, status, FTB_ERR_TIMEOUT_EPI)) break;
        stg_phase ^= 1u;
        if (full_tile) {
#pragma unroll
          for (int b = 0; b < C::kCBoxes; ++b) tma_store_2d(&mapC, s_c + b * C::kCBoxBytes, unit_base + 32 * b, c_row);
          tma_store_commit();
          if (PERSIST)
            tma_store_wait<0>();  // written, not just read: the cell-state counter is bumped next
          else
            tma_store_wait_read<0>();
        }
        if (PERSIST) {
          fence_proxy_async_all();
          __threadfence();
          red_release_gpu_add(plan.fine ? plan.c_done + tile : plan.done + batch.n_items + cur.idx, 1);
        }
      }
      if (!PERSIST) tma_store_wait<0>();
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
    if (PAIR)
      tmem_dealloc_pair(tmem_base, C::kTmemCols);
    else
      tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <typename T, int BN, int EPI, bool PERSIST, bool PAIR>
int launch_one(const CUtensorMap* maps, const CUtensorMap& mapW, const CUtensorMap& mapC, const CellBatch& batch,
               const PlanView& plan, int* status, int sm_count, cudaStream_t stream) {
  using C = Cfg<BN, EPI, PAIR>;
  static std::atomic<unsigned long long> configured{0};
  auto kfn = cell_gemm_kernel<T, BN, EPI, PERSIST, PAIR>;
  if (!ensure_dynamic_smem(kfn, C::kSmemBytes, configured)) return FTB_ERR_LAUNCH;
  int grid = batch.total_tiles < sm_count ? batch.total_tiles : sm_count;
  if (PAIR) grid &= ~1;  // whole pairs only; tiles 2p and 2p+1 are the two halves of one row block
  if (grid <= 0) return FTB_OK;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[3];
  int na = 0;
  if (PAIR) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = 2;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = 1;
    ++na;
  }
  // FTB_NO_COOPERATIVE=1 drops the cooperative attribute (profilers that cannot replay
  // cooperative launches); residency then rests on grid <= SM count on an otherwise idle
  // device, and the bounded waits turn a violated assumption into a status code.
  static const bool no_coop = [] {
    const char* e = getenv("FTB_NO_COOPERATIVE");
    return e != nullptr && e[0] == '1';
  }();
  // FTB_REFUSE_COOPERATIVE=1 makes this function answer as if the driver had refused the
  // cooperative launch (host-side failure injection for the schedule fallback's tests).
  {
    const char* e = getenv("FTB_REFUSE_COOPERATIVE");
    if (PERSIST && e != nullptr && e[0] == '1') return FTB_ERR_LAUNCH;
  }
  if (PERSIST && !no_coop) {
    // Cooperative launch: every CTA is resident, so a CTA that waits on another
    // CTA's counter always makes progress.
    attrs[na].id = cudaLaunchAttributeCooperative;
    attrs[na].val.cooperative = 1;
    ++na;
  }
  if (!PERSIST && grid < sm_count) {
    // Level launches follow one another on the stream: when a level leaves SMs idle, let the next one
    // set up there while this one drains (with grids that fill the device it was measured slower).
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  if (cudaLaunchKernelEx(&cfg, kfn, maps[0], maps[1], maps[2], maps[3], mapW, mapC, batch, plan, status) != cudaSuccess) {
    cudaGetLastError();
    return FTB_ERR_LAUNCH;
  }
  count_launch();
  return FTB_OK;
}

template <typename T, int BN, bool PERSIST, bool PAIR>
int launch_epi(int epi, const CUtensorMap* maps, const CUtensorMap& mapW, const CUtensorMap& mapC,
               const CellBatch& batch, const PlanView& plan, int* status, int sm_count, cudaStream_t stream) {
  switch (epi) {
    case EPI_STORE:
      return launch_one<T, BN, EPI_STORE, PERSIST, PAIR>(maps, mapW, mapC, batch, plan, status, sm_count, stream);
    case EPI_LSTM:
      return launch_one<T, BN, EPI_LSTM, PERSIST, PAIR>(maps, mapW, mapC, batch, plan, status, sm_count, stream);
    case EPI_TANH:
      return launch_one<T, BN, EPI_TANH, PERSIST, PAIR>(maps, mapW, mapC, batch, plan, status, sm_count, stream);
    case EPI_STORE_F32:
      if constexpr (!PERSIST && !PAIR)
        return launch_one<T, BN, EPI_STORE_F32, false, false>(maps, mapW, mapC, batch, plan, status, sm_count, stream);
      return FTB_ERR_ARG;
    default: return FTB_ERR_ARG;
  }
}

template <bool PERSIST, bool PAIR>
int launch_any(int dtype, int epi, int bn, const CUtensorMap* maps, const CUtensorMap& mapW, const CUtensorMap& mapC,
               const CellBatch& batch, const PlanView& plan, int* status, int sm_count, cudaStream_t stream) {
  if (dtype == FTB_F16) {
    if (bn == 256)
      return launch_epi<__half, 256, PERSIST, PAIR>(epi, maps, mapW, mapC, batch, plan, status, sm_count, stream);
    if (bn == 128)
      return launch_epi<__half, 128, PERSIST, PAIR>(epi, maps, mapW, mapC, batch, plan, status, sm_count, stream);
  } else if (dtype == FTB_BF16) {
    if (bn == 256)
      return launch_epi<__nv_bfloat16, 256, PERSIST, PAIR>(epi, maps, mapW, mapC, batch, plan, status, sm_count,
                                                            stream);
    if (bn == 128)
      return launch_epi<__nv_bfloat16, 128, PERSIST, PAIR>(epi, maps, mapW, mapC, batch, plan, status, sm_count,
                                                            stream);
  }
  return FTB_ERR_ARG;
}

}  // namespace

// Launches one wavefront level.  `maps` are the four activation tensor maps
// (box 128 rows x 64 elements; LSTM outputs are stored through the map named by
// each item's out_map), `mapW` the packed-weight map (box `bn` rows x 64
// elements, or bn/2 rows when `pair` is set), `mapC` the fp32 cell-state map (box
// 128 rows x 32 elements) for LSTM cells and, for the other epilogues, the map of the
// second packed-weight buffer (items with w_map == 1).  With `pair`, every item's m_tiles must be
// even.
int launch_cell_gemm(int dtype, int epi, int bn, int pair, const CUtensorMap* maps, const CUtensorMap& mapW,
                     const CUtensorMap& mapC, const CellBatch& batch, int* status, int sm_count,
                     cudaStream_t stream) {
  PlanView none = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, nullptr, nullptr};
  if (pair) return launch_any<false, true>(dtype, epi, bn, maps, mapW, mapC, batch, none, status, sm_count, stream);
  return launch_any<false, false>(dtype, epi, bn, maps, mapW, mapC, batch, none, status, sm_count, stream);
}

// Launches a whole wavefront as one persistent kernel.  `header` carries n_items,
// n_cols, ld_out, ld_c and total_tiles; its items[] are ignored (they live in
// plan.items in global memory).
int launch_cell_gemm_persistent(int dtype, int epi, int bn, int pair, const CUtensorMap* maps,
                                const CUtensorMap& mapW, const CUtensorMap& mapC, const CellBatch& header,
                                const PlanView& plan, int* status, int sm_count, cudaStream_t stream) {
  if (pair) return launch_any<true, true>(dtype, epi, bn, maps, mapW, mapC, header, plan, status, sm_count, stream);
  return launch_any<true, false>(dtype, epi, bn, maps, mapW, mapC, header, plan, status, sm_count, stream);
}

}  // namespace ftb
