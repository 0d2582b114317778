// Stacked LSTM forward with static tile ownership ("each CTA keeps its slice of a
// layer for a whole sweep over time").
//
// Layers are processed in groups of G whose packed weights fit in L2.  Within a
// group every CTA pair owns one 256-row x 256-column accumulator tile of one
// layer -- always the same hidden units and batch rows -- and walks the time steps
// t = 0 .. L-1 with it.  Consequences:
//   * the fp32 cell state of those units never leaves the registers of the
//     epilogue threads between steps (no cell-state traffic at all, only the
//     final state is stored);
//   * layers pipeline by themselves: a layer's step t needs the layer below at
//     step t and itself at step t-1, both published through per-cell completion
//     counters, so lower layers simply run ahead and a group's CTAs roll over into
//     the next group as soon as they finish (waiting per producer tile instead of
//     per cell was measured and is no faster: the tiles of a cell finish together);
//   * the tensor pipe is kept busy across the recurrence: the half of the K loop
//     that reads the layer below for step t+1 is issued before the half that
//     reads the own layer's step t-1, into the second TMEM accumulator, so it runs
//     while the epilogue of step t-1 is writing h and the counters propagate.
//
// Same arithmetic, in the same order, as cell_gemm_kernel's LSTM path (the
// results are bit-identical); the same roles: warp 0 TMA producer, warp 1 MMA
// issuer, warps 2..9 epilogue.  CTA pairs (tcgen05 cta_group::2) only; no
// cluster-multicast loads.  Launched cooperatively: a CTA that waits for a
// counter relies on the CTAs that bump it being resident.
//
// Takes the place of the reference's per-hyperplane region drivers
// (kaleido/core/device/kernels/lstm/stacked_lstm/region{1,2,3}.h) for the
// 16-bit stacked LSTM; the program it implements is stacked_lstm()
// (examples/stacked_rnn/stacked_lstm1.py:66-76).
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "ptx.cuh"
#include "tmap.h"

namespace ftb {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int kEpiWarps = 8;
#ifndef FTB_STATIC_FIRST
#define FTB_STATIC_FIRST 2
#endif
// An epilogue warp reads its four 32-column accumulator chunks in two rounds: kFirstRound chunks,
// their gate arithmetic, then the rest.
constexpr int kFirstRound = FTB_STATIC_FIRST;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kStages = 6;
constexpr uint32_t kABytes = BM * BK * 2;
constexpr uint32_t kBBytes = (BN / 2) * BK * 2;
constexpr uint32_t kStageBytes = kABytes + kBBytes;
// One [128 rows x 64 units] output tile per CTA, in the 128-byte-swizzled layout of the tensor map
// the next cells load it with, so that one TMA store publishes a step's hidden states.
constexpr uint32_t kOutTileBytes = BM * (BN / 4) * 2;
constexpr uint32_t kSmemBytes = kStages * kStageBytes + kOutTileBytes + 1024;
constexpr uint32_t kTmemCols = 2 * BN;

struct StaticArgs {
  int D, L, N, I, H, G;
  int n_tiles;         // 4H / 256
  int m_tiles;         // 2 * ceil(N / 256)
  int tiles_per_cell;  // n_tiles * m_tiles
  const float* bias_p; // [D, 4H] packed order, or nullptr
  void* hs;            // [D, L, N, H]
  float* c_out;        // [D, N, H]
  int* done;           // [D * L] completion counters, zero before the launch
  int* status;
  int tma_out;         // 1: every row tile is full (N % 128 == 0), outputs leave through TMA stores
  unsigned long long* trace;  // debug builds (FTB_TRACE): [D*L][tiles_per_cell][4] globaltimer stamps, else nullptr
};

// The order in which a CTA issues the two halves of its tiles over one sweep:
// X(t) = input half of step t (reads the layer below), H(t) = recurrent half
// (reads the own layer's step t-1; absent at t = 0).  X(t+1) goes before H(t).
template <typename F>
__device__ __forceinline__ bool for_each_half(int L, F f) {
  if (!f(true, 0)) return false;
  if (L > 1 && !f(true, 1)) return false;
  for (int t = 1; t < L; ++t) {
    if (t + 1 < L && !f(true, t + 1)) return false;
    if (!f(false, t)) return false;
  }
  return true;
}

template <typename T>
#ifdef FTB_STATIC_MAXNREG
__global__ void __maxnreg__(FTB_STATIC_MAXNREG)
#else
__global__ void __launch_bounds__(kThreads, 1)
#endif
lstm_static_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapH,
                   const __grid_constant__ CUtensorMap mapW, const StaticArgs a) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[kStages];
  __shared__ uint64_t empty_bar[kStages];
  __shared__ uint64_t tfull_bar[2];
  __shared__ uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t peer_tmem_base_s;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = the pair's leader: it issues the MMAs
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* s_out = smem + kStages * kStageBytes;  // the CTA's output tile (TMA-store path)
  int* status = a.status;

  if (threadIdx.x == 0) {
    prefetch_tmap(&mapX);
    prefetch_tmap(&mapH);
    prefetch_tmap(&mapW);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tfull_bar[1], 1);
    mbar_init(&tempty_bar[0], 2 * kEpiWarps);  // the epilogue warps of both CTAs of the pair
    mbar_init(&tempty_bar[1], 2 * kEpiWarps);
    s_abort = 0;
    peer_tmem_base_s = 0xffffffffu;
    fence_barrier_init();
  }
  if (warp == 1) {
    // Every tcgen05 instruction of this kernel is .cta_group::2, the allocation included.
    tmem_alloc_pair(&tmem_base_s, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  // Both CTAs of a pair must hold their accumulators at the same TMEM columns.
  if (threadIdx.x == 0 && rank == 1) st_shared_cluster_u32(map_to_cta(smem_u32(&peer_tmem_base_s), 0), tmem_base);
  cluster_sync_all();
  if (rank == 0 && threadIdx.x == 0 && peer_tmem_base_s != tmem_base) {
    s_abort = 1;
    atomicCAS(status, 0, FTB_ERR_TMEM_LAYOUT);
  }
  __syncthreads();

  // This CTA's slot: layer index inside a group, column tile, row tile.
  const int j = blockIdx.x / a.tiles_per_cell;
  const int tile = blockIdx.x - j * a.tiles_per_cell;
  const int n_tile = tile / a.m_tiles;
  const int m_tile = tile - n_tile * a.m_tiles;  // parity == rank
  // completions a cell's counter collects: one per tile with TMA stores, one per epilogue warp without
  const int target = (a.tma_out ? 1 : kEpiWarps) * a.tiles_per_cell;
  const int n_groups = (a.D + a.G - 1) / a.G;
  const int kb_x0 = a.I / BK, kb_h = a.H / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t w_policy = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int g = 0; g < n_groups && ok; ++g) {
        const int l = g * a.G + j;
        if (l >= a.D) continue;
        const int w_row = l * 4 * a.H + n_tile * BN + static_cast<int>(rank) * (BN / 2);
        ok = for_each_half(a.L, [&](bool is_x, int t) -> bool {
          // Which counter guards the activations, where they are, where the weights' K range is.
          const int* dep = nullptr;
          const CUtensorMap* am;
          int a_row, wk, nkb;
          if (is_x) {
            if (l == 0) {
              am = &mapX;
              a_row = t * a.N;
              nkb = kb_x0;
            } else {
              am = &mapH;
              a_row = ((l - 1) * a.L + t) * a.N;
              nkb = kb_h;
              dep = a.done + (l - 1) * a.L + t;
            }
            wk = 0;
          } else {
            am = &mapH;
            a_row = (l * a.L + t - 1) * a.N;
            nkb = kb_h;
            wk = a.I;
            dep = a.done + l * a.L + t - 1;
          }
          a_row += m_tile * BM;
          // A half that has to wait for a counter first puts the weights of its leading K blocks
          // in flight (they depend on nothing), as many as there are free stages right now, then
          // waits, then sends the activations after them.
          int pre = 0;
          if (dep != nullptr) {
            int st = stage;
            uint32_t ph = phase;
            while (pre < nkb && pre < kStages && mbar_try_wait(&empty_bar[st], ph ^ 1u)) {
              const uint32_t lead_bar = map_to_cta(smem_u32(&full_bar[st]), 0);
              if (rank == 0) mbar_arrive_expect_tx(&full_bar[st], 2 * kStageBytes);
              tma_load_2d_pair_hint(smem + st * kStageBytes + kABytes, &mapW, lead_bar, wk + pre * BK, w_row, w_policy);
              ++pre;
              if (++st == kStages) {
                st = 0;
                ph ^= 1u;
              }
            }
            if (!flag_wait_ge(dep, target, &s_abort, status, FTB_ERR_TIMEOUT_DEP)) return false;
            // plain stores of h by other CTAs -> this thread's TMA loads; TMA-stored h needs no fence
            if (!a.tma_out) fence_proxy_async_all();
#ifdef FTB_TRACE
            if (a.trace && !is_x) a.trace[(static_cast<size_t>(l * a.L + t) * a.tiles_per_cell + tile) * 4 + 0] = globaltimer_ns();
#endif
          }
          for (int kb = 0; kb < nkb; ++kb) {
            uint8_t* sa = smem + stage * kStageBytes;
            uint8_t* sb = sa + kABytes;
            const uint32_t lead_bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
            if (kb >= pre) {
              if (!mbar_wait(&empty_bar[stage], phase ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_SLOT)) return false;
              // Both CTAs' copies are counted on the leader's barrier; only the leader arms it.
              if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * kStageBytes);
              tma_load_2d_pair_hint(sb, &mapW, lead_bar, wk + kb * BK, w_row, w_policy);
            }
            tma_load_2d_pair(sa, am, lead_bar, kb * BK, a_row);
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          return true;
        });
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_f16(2 * BM, BN, Fmt<T>::kind, 0, 0);
      const uint64_t a_desc0 = make_sdesc_sw128(smem_u32(smem), 16, 1024);
      const uint64_t b_desc0 = make_sdesc_sw128(smem_u32(smem) + kABytes, 16, 1024);
      int stage = 0;
      uint32_t stage_off = 0;  // stage * kStageBytes / 16
      uint32_t phase = 0;
      int k_base = 0;  // tiles this CTA has started before the current sweep
      bool ok = true;
      for (int g = 0; g < n_groups && ok; ++g) {
        const int l = g * a.G + j;
        if (l >= a.D) continue;
        ok = for_each_half(a.L, [&](bool is_x, int t) -> bool {
          const int k = k_base + t;         // running tile number of this CTA
          const int acc = k & 1;
          const int nkb = is_x ? (l == 0 ? kb_x0 : kb_h) : kb_h;
          if (is_x) {
            // First MMA of tile k: its accumulator must have been drained (tile k-2).
            if (!mbar_wait(&tempty_bar[acc], ((k >> 1) & 1) ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_EPI)) return false;
            tc_fence_after();
          }
          const uint32_t d_tmem = tmem_base + acc * BN;
          uint32_t accumulate = is_x ? 0u : 1u;  // the first MMA of a tile overwrites the accumulator
          for (int kb = 0; kb < nkb; ++kb) {
            // (No tcgen05 fence after a barrier that TMA completes: the fence orders against other threads'
            // tcgen05 operations, which do not touch the stage, and it drains the tensor pipe.)
            if (!mbar_wait(&full_bar[stage], phase, &s_abort, status, FTB_ERR_TIMEOUT_TMA)) return false;
#ifdef FTB_TRACE
            if (a.trace && !is_x && kb == 0) a.trace[(static_cast<size_t>(l * a.L + t) * a.tiles_per_cell + tile) * 4 + 1] = globaltimer_ns();
#endif
            // This thread's own instructions are the floor of a K block: the operand descriptors are the
            // stage-0 descriptors plus byte offsets / 16, nothing is rebuilt per MMA.
            const uint64_t ad = a_desc0 + stage_off;
            const uint64_t bd = b_desc0 + stage_off;
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
              umma_ss_pair(d_tmem, ad + 2 * kk, bd + 2 * kk, idesc, accumulate);
              accumulate = 1u;
            }
            umma_commit_pair(&empty_bar[stage]);
            stage_off += kStageBytes >> 4;
            if (++stage == kStages) {
              stage = 0;
              stage_off = 0;
              phase ^= 1u;
            }
          }
          // The tile is complete after its recurrent half (or after the input half at t = 0).
          if (!is_x || t == 0) umma_commit_pair(&tfull_bar[acc]);
          return true;
        });
        k_base += a.L;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    // Eight warps: warp w reads TMEM lane quadrant w % 4; the two warps of a quadrant split
    // the tile's eight 32-column chunks.  Each thread owns 32 hidden units of one batch row and
    // keeps their cell state in registers across the whole sweep.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r_loc = q * 32 + lane;
    const int row = m_tile * BM + r_loc;
    const bool row_ok = row < a.N;
    const int col_base = n_tile * BN;
    int k_base = 0;
    bool ok = true;
    for (int g = 0; g < n_groups && ok; ++g) {
      const int l = g * a.G + j;
      if (l >= a.D) continue;
      const float* bias = a.bias_p ? a.bias_p + static_cast<size_t>(l) * 4 * a.H : nullptr;
      float creg[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) creg[i] = 0.f;
      for (int t = 0; t < a.L && ok; ++t) {
        const int k = k_base + t;
        const int acc = k & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&tfull_bar[acc], (k >> 1) & 1, &s_abort, status, FTB_ERR_TIMEOUT_MMA))) {
          ok = false;
          break;
        }
        tc_fence_after();
#ifdef FTB_TRACE
        if (a.trace && warp == 2 && lane == 0) a.trace[(static_cast<size_t>(l * a.L + t) * a.tiles_per_cell + tile) * 4 + 2] = globaltimer_ns();
#endif
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
        T* out_row = reinterpret_cast<T*>(a.hs) + (static_cast<size_t>(l) * a.L + t) * a.N * a.H +
                     static_cast<size_t>(row) * a.H;
        // With TMA stores the step's [128 x 64] tile is built in shared memory first (row r_loc, 16-byte
        // chunk = 8 units, chunk index XOR row % 8: the tensor map's 128-byte swizzle).  The previous
        // step's tile must have left shared memory: the storing thread arrives here after its store.
        uint8_t* tile_row = s_out + r_loc * 128;
        if (a.tma_out) asm volatile("bar.sync 2, %0;" ::"n"(32 * kEpiWarps) : "memory");
        // After the last read of the accumulator the MMA warp gets it back, before the arithmetic of
        // the chunks just read: it is the accumulator of the tile after next, whose input half is the
        // very next thing the tensor pipe has to do.
        auto round = [&](auto c0_, auto n_, auto last_) {
          constexpr int c0 = decltype(c0_)::value, n = decltype(n_)::value;
          uint32_t r[n][32];
#pragma unroll
          for (int cd = 0; cd < n; ++cd) tmem_ld32(taddr + (half * 4 + c0 + cd) * 32, r[cd]);
          tmem_ld_wait();
          if constexpr (decltype(last_)::value) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
          }
#pragma unroll
          for (int cd = 0; cd < n; ++cd) {
            const int cc = c0 + cd;
            const int col0 = col_base + (half * 4 + cc) * 32;
            const int unit0 = col0 >> 2;
            float hn[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              float gi = __uint_as_float(r[cd][4 * u + 0]);
              float gf = __uint_as_float(r[cd][4 * u + 1]);
              float go = __uint_as_float(r[cd][4 * u + 2]);
              float gc = __uint_as_float(r[cd][4 * u + 3]);
              if (bias != nullptr) {
                const float4 b = __ldg(reinterpret_cast<const float4*>(bias + col0) + u);
                gi += b.x; gf += b.y; go += b.z; gc += b.w;
              }
              const float c_new = sigmoid_fast(gf) * creg[8 * cc + u] + sigmoid_fast(gi) * tanh_fast(gc);
              creg[8 * cc + u] = c_new;
              hn[u] = sigmoid_fast(go) * tanh_fast(c_new);
            }
            uint4 v;
            v.x = Fmt<T>::pack2(hn[0], hn[1]);
            v.y = Fmt<T>::pack2(hn[2], hn[3]);
            v.z = Fmt<T>::pack2(hn[4], hn[5]);
            v.w = Fmt<T>::pack2(hn[6], hn[7]);
            if (a.tma_out) {
              const int chunk = half * 4 + cc;
              *reinterpret_cast<uint4*>(tile_row + ((chunk ^ (r_loc & 7)) << 4)) = v;
            } else if (row_ok) {
              *reinterpret_cast<uint4*>(out_row + unit0) = v;
            }
          }
        };
        round(std::integral_constant<int, 0>{}, std::integral_constant<int, kFirstRound>{}, std::false_type{});
        round(std::integral_constant<int, kFirstRound>{}, std::integral_constant<int, 4 - kFirstRound>{}, std::true_type{});
        if (a.tma_out) {
          // One thread stores the tile once the eight warps have written it, waits for the store and
          // counts the tile in; the readers are other CTAs' TMA loads (same proxy: no fence).
          fence_proxy_async_smem();
          asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory");
          if (warp == 2 && lane == 0) {
            // (a pair covers 256 rows: with 128 sequences the second CTA's tile is all padding)
            if (m_tile * BM < a.N) {
              tma_store_2d(&mapH, s_out, n_tile * (BN / 4), (l * a.L + t) * a.N + m_tile * BM);
              tma_store_commit();
              tma_store_wait<0>();
            }
            red_release_gpu_add(a.done + l * a.L + t, 1);
#ifdef FTB_TRACE
            if (a.trace) a.trace[(static_cast<size_t>(l * a.L + t) * a.tiles_per_cell + tile) * 4 + 3] = globaltimer_ns();
#endif
          }
        } else {
          fence_proxy_async_all();  // plain stores of h -> other CTAs' TMA loads
          __threadfence();
          __syncwarp();
          if (lane == 0) {
            red_release_gpu_add(a.done + l * a.L + t, 1);
#ifdef FTB_TRACE
            if (a.trace && warp == 2) a.trace[(static_cast<size_t>(l * a.L + t) * a.tiles_per_cell + tile) * 4 + 3] = globaltimer_ns();
#endif
          }
        }
      }
      // Final cell state of the sweep.
      if (ok && row_ok) {
        float* c_row = a.c_out + (static_cast<size_t>(l) * a.N + row) * a.H + (col_base >> 2) + half * 32;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          __stcg(reinterpret_cast<float4*>(c_row) + i,
                 make_float4(creg[4 * i], creg[4 * i + 1], creg[4 * i + 2], creg[4 * i + 3]));
      }
      k_base += a.L;
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  // Neither CTA of a pair may leave while the other can still signal its barriers.
  cluster_sync_all();
  if (warp == 1) {
    if (s_abort) {
      // Give copies and MMAs still in flight time to land before TMEM and shared memory go back.
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <typename T>
int launch(const CUtensorMap& mX, const CUtensorMap& mH, const CUtensorMap& mW, const StaticArgs& a, int grid,
           cudaStream_t stream) {
  static std::atomic<unsigned long long> configured{0};
  auto kfn = lstm_static_kernel<T>;
  if (!ensure_dynamic_smem(kfn, kSmemBytes, configured)) return FTB_ERR_LAUNCH;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  attrs[na].id = cudaLaunchAttributeClusterDimension;
  attrs[na].val.clusterDim.x = 2;
  attrs[na].val.clusterDim.y = 1;
  attrs[na].val.clusterDim.z = 1;
  ++na;
  // FTB_NO_COOPERATIVE=1 drops the cooperative attribute (profilers that cannot replay
  // cooperative launches); residency then rests on grid <= SM count on an otherwise idle device.
  static const bool no_coop = [] {
    const char* e = getenv("FTB_NO_COOPERATIVE");
    return e != nullptr && e[0] == '1';
  }();
  // FTB_REFUSE_COOPERATIVE=1 makes this function answer as if the driver had refused the
  // cooperative launch (host-side failure injection for the schedule fallback's tests).
  {
    const char* e = getenv("FTB_REFUSE_COOPERATIVE");
    if (e != nullptr && e[0] == '1') return FTB_ERR_LAUNCH;
  }
  if (!no_coop) {
    attrs[na].id = cudaLaunchAttributeCooperative;
    attrs[na].val.cooperative = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  if (cudaLaunchKernelEx(&cfg, kfn, mX, mH, mW, a) != cudaSuccess) {
    cudaGetLastError();
    return FTB_ERR_LAUNCH;
  }
  count_launch();
  return FTB_OK;
}

}  // namespace

// True when the static-ownership kernel can run the problem: 16-bit, a group of G
// layers' tiles fits on the device at one CTA per SM.
bool lstm_static_supported(int dtype, int D, int N, int I, int H, int G, int sm_count) {
  if (dtype != FTB_F16 && dtype != FTB_BF16) return false;
  if (H % 64 != 0 || I % 64 != 0 || (D > 1 && I != H) || G < 1) return false;
  const int tiles = (4 * H / BN) * 2 * ((N + 255) / 256);
  return (4 * H) % BN == 0 && G * tiles <= sm_count;
}

// x: [L,N,I]; Wp: [D,4H,I+H]; hs: [D,L,N,H]; c: [D,N,H]; done: D*L ints (zeroed here).
int launch_lstm_static(int dtype, const void* x, const void* Wp, const float* bias_p, void* hs, float* c, int D, int L,
                       int N, int I, int H, int G, int* done, int* status, unsigned long long* trace,
                       cudaStream_t stream) {
  StaticArgs a;
  a.D = D; a.L = L; a.N = N; a.I = I; a.H = H; a.G = G;
  a.n_tiles = 4 * H / BN;
  a.m_tiles = 2 * ((N + 255) / 256);
  a.tiles_per_cell = a.n_tiles * a.m_tiles;
  a.bias_p = bias_p;
  a.hs = hs;
  a.c_out = c;
  a.done = done;
  a.status = status;
  a.tma_out = (N % BM == 0) ? 1 : 0;
  a.trace = trace;
  const int K = I + H;
  CUtensorMap mX, mH, mW;
  int rc;
  if ((rc = make_tmap_2d(&mX, x, dtype, static_cast<uint64_t>(L) * N, I, I, 128, 64))) return rc;
  if ((rc = make_tmap_2d(&mH, hs, dtype, static_cast<uint64_t>(D) * L * N, H, H, 128, 64))) return rc;
  if ((rc = make_tmap_2d(&mW, Wp, dtype, static_cast<uint64_t>(D) * 4 * H, K, K, BN / 2, 64))) return rc;
  if (cudaMemsetAsync(done, 0, sizeof(int) * static_cast<size_t>(D) * L, stream) != cudaSuccess) return FTB_ERR_LAUNCH;
  const int grid = std::min(G, D) * a.tiles_per_cell;
  if (dtype == FTB_F16) return launch<__half>(mX, mH, mW, a, grid, stream);
  return launch<__nv_bfloat16>(mX, mH, mW, a, grid, stream);
}

}  // namespace ftb
