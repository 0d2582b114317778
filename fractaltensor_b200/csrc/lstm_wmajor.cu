// Stacked LSTM forward for small batches (at most 128 sequences per call): the
// weights are the M operand of the MMA and the batch is its N operand.
//
// The other stacked-LSTM kernels put 128 (or 256) batch rows on the M side of the
// tensor-core instruction; with 32 sequences per GPU -- a batch of 256 split over
// eight GPUs -- seven eighths of every MMA would multiply padding.  Here a tile is
// 128 packed gate rows (32 hidden units x 4 gates: UMMA M = 128) by NB batch
// columns (UMMA N = NB in {32, 64, 128}), D^T = Wp_tile . act^T, which is the
// orientation of the reference's own gate GEMM ([4H, K] x [K, batch],
// kaleido/core/device/kernels/lstm_kernels.h:24-48).  The price of this orientation
// is that the four gates of a hidden unit land in four neighbouring TMEM lanes,
// i.e. in four threads: the epilogue brings them together with a 4x4 register
// transpose over warp shuffles (one shuffle per accumulator element).
//
// Scheduling is static tile ownership, as in lstm_static.cu: layers run in groups of
// G whose packed weights stay in L2; inside a group CTA (j, n_tile) owns the same 32
// hidden units of layer j for the whole sweep over time, keeps their fp32 cell state
// in registers, and layers chain through per-cell completion counters in global
// memory.
//
// A step is latency-bound at these batch sizes.  What the kernel does about it:
//   * an MMA of 32 or 64 columns occupies the tensor pipe for about 50 cycles whatever its
//     width (measured: a fixed floor per instruction, no penalty for accumulating into the
//     same columns back to back), so a 64-wide K block costs ~200 cycles and a step ~6400;
//   * weights and activations move through two independent rings with their own
//     producer threads, so weight blocks stream ahead while the activation producer
//     waits for a flag, and most of shared memory is the weight ring (the rate at which
//     an SM streams from L2 is bytes in flight over latency);
//   * the first K blocks of the recurrent half of the CTA's weight tile stay resident
//     in tensor memory for the whole sweep, as the A operand of the MMA, in the TMEM
//     columns the accumulators leave free ("recurrent weights resident on chip where
//     they fit"); these blocks cost no L2 traffic and no shared-memory reads;
//   * the input half of step t+1 (which never waits for this layer) is issued right
//     after the recurrent half of step t, so it runs while step t's hidden state
//     travels to the other CTAs of the layer.
//
// Roles: warp 0 activation producer (TMA), warp 1 MMA issuer (owns TMEM), warp 2 weight
// producer (TMA), warp 3 idle, warps 4..11 epilogue (two per TMEM lane quadrant, each taking
// half of the batch columns).  Single CTAs (tcgen05 cta_group::1); no
// cluster-multicast loads.  Launched cooperatively.
//
// The program is stacked_lstm() (examples/stacked_rnn/stacked_lstm1.py:66-76) on a
// batch shard; it stands in for the region drivers
// kaleido/core/device/kernels/lstm/stacked_lstm/region{1,2,3}.h.
#include <algorithm>
#include <cstdlib>

#include "ptx.cuh"
#include "tmap.h"

namespace ftb {

namespace {

constexpr int BMW = 128;  // packed gate rows per tile
constexpr int BK = 64;
constexpr int kEpiWarps = 8;
constexpr int kFirstEpiWarp = 4;
constexpr int kThreads = 32 * (kFirstEpiWarp + kEpiWarps);
constexpr uint32_t kBlockBytes = 16384;  // one weight K block [128 x 64]; also one activation stage

template <int NB>
struct WCfg {
  // An activation stage is 16 KB whatever NB is: 4, 2 or 1 K blocks of [NB x 64].
  static constexpr int kActBlocks = 128 / NB;
  static constexpr uint32_t kActBlockBytes = NB * BK * 2;
  static constexpr uint32_t kAccCols = 2 * NB;  // two tiles in flight
  // Recurrent weight blocks resident in TMEM beside the accumulators (32 columns per block).
  static constexpr int kTmemBlocks = (512 - kAccCols) / 32;
  static constexpr int kActStages = NB == 128 ? 5 : 3;
  // A weight stage holds two K blocks (32 KB): half as many commits and barrier waits per byte.
  static constexpr int kWStages = (14 - kActStages) / 2;
  // The step's output tile, row-major [NB sequences][32 units], staged for one TMA store (13 ring
  // stages of 16 KB are left beside it).
  static constexpr uint32_t kOutBytes = NB * (BMW / 4) * 2;
  static constexpr uint32_t kSmemBytes = (kActStages + 2 * kWStages) * kBlockBytes + kOutBytes + 1024;
};

struct WArgs {
  int D, L, N, I, H, G;
  int n_tiles;          // 4H / 128
  int res_tmem;         // recurrent K blocks resident in TMEM (<= WCfg::kTmemBlocks)
  const float* bias_p;  // [D, 4H] packed order, or nullptr
  const void* Wp;       // [D, 4H, I+H]
  void* hs;             // [D, L, N, H]
  float* c_out;         // [D, N, H]
  int* done;            // [D * L * n_tiles] flags, zero before the launch: tile `n` of cell (l, t) has published its h
  int* status;
  unsigned long long* trace;  // debug builds (FTB_TRACE): [D*L][16 tiles][16] globaltimer stamps, else nullptr
};

#ifdef FTB_TRACE
#define FTB_WM_STAMP(l, t, s) \
  if (a.trace && n_tile < 16) a.trace[((static_cast<size_t>((l) * a.L + (t))) * 16 + n_tile) * 16 + (s)] = globaltimer_ns()
#else
#define FTB_WM_STAMP(l, t, s)
#endif

// The halves of a sweep in issue order: X(t) = input half of step t (reads the layer below),
// H(t) = recurrent half (reads the own layer's step t-1; absent at t = 0).
template <typename F>
__device__ __forceinline__ bool for_each_half(int L, F f) {
  for (int t = 0; t < L; ++t) {
    if (!f(true, t)) return false;
    if (t > 0 && !f(false, t)) return false;
  }
  return true;
}

// 4x4 transpose across the four lanes of a quad: before, lane q (= lane & 3) holds a[j] = M[q][j];
// after, it holds a[j] = M[j][q].
__device__ __forceinline__ void quad_transpose(float& a0, float& a1, float& a2, float& a3, int lane) {
  const bool b0 = (lane & 1) != 0, b1 = (lane & 2) != 0;
  float r;
  r = __shfl_xor_sync(0xffffffffu, b0 ? a0 : a1, 1);
  if (b0) a0 = r; else a1 = r;
  r = __shfl_xor_sync(0xffffffffu, b0 ? a2 : a3, 1);
  if (b0) a2 = r; else a3 = r;
  r = __shfl_xor_sync(0xffffffffu, b1 ? a0 : a2, 2);
  if (b1) a0 = r; else a2 = r;
  r = __shfl_xor_sync(0xffffffffu, b1 ? a1 : a3, 2);
  if (b1) a1 = r; else a3 = r;
}

template <typename T>
__device__ __forceinline__ void store_h(T* p, float v);
template <>
__device__ __forceinline__ void store_h<__half>(__half* p, float v) { *p = __float2half_rn(v); }
template <>
__device__ __forceinline__ void store_h<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Whole-warp bounded wait until the n flags at `flags` are all non-zero: lane i polls flags i, i+32, ...
// (one coalesced request per poll for up to 32 flags).  Every lane acquires the flags it read; the
// warp-wide vote orders those acquires before what any lane does next.
__device__ __forceinline__ bool warp_wait_flags(const int* flags, int n, int lane, volatile int* s_abort, int* g_status) {
  uint64_t t0 = 0;
  uint32_t it = 0;
  for (;;) {
    bool ready = true;
    for (int i = lane; i < n; i += 32) ready = ready && (ld_acquire_gpu(flags + i) != 0);
    if (__all_sync(0xffffffffu, ready)) return true;
    if (((++it) & 0x3F) == 0) {
      if (t0 == 0) t0 = globaltimer_ns();
      const bool give_up = *s_abort != 0 || globaltimer_ns() - t0 > FTB_WAIT_TIMEOUT_NS;
      if (__any_sync(0xffffffffu, give_up)) {
        if (lane == 0 && *s_abort == 0) {
          *s_abort = 1;
          atomicCAS(g_status, 0, FTB_ERR_TIMEOUT_DEP);
        }
        return false;
      }
    }
  }
}

template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[N]) {
  if constexpr (N == 32) tmem_ld32(taddr, r);
  else tmem_ld16(taddr, r);
}

template <typename T, int NB>
__global__ void __launch_bounds__(kThreads, 1)
lstm_wmajor_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapH,
                   const __grid_constant__ CUtensorMap mapW, const __grid_constant__ CUtensorMap mapO,
                   const WArgs a) {
  using C = WCfg<NB>;
  constexpr int AS = C::kActStages, WS = C::kWStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t act_full[AS], act_empty[AS];
  __shared__ uint64_t w_full[WS], w_empty[WS];
  __shared__ uint64_t tfull_bar[2], tempty_bar[2];
  __shared__ uint64_t res_full;  // the sweep's resident weight blocks are in TMEM
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* s_act = smem;
  uint8_t* s_w = s_act + AS * kBlockBytes;
  uint8_t* s_out = s_w + 2 * WS * kBlockBytes;
  int* status = a.status;

  if (threadIdx.x == 0) {
    prefetch_tmap(&mapX);
    prefetch_tmap(&mapH);
    prefetch_tmap(&mapW);
    prefetch_tmap(&mapO);
    for (int i = 0; i < AS; ++i) {
      mbar_init(&act_full[i], 1);
      mbar_init(&act_empty[i], 1);
    }
    for (int i = 0; i < WS; ++i) {
      mbar_init(&w_full[i], 1);
      mbar_init(&w_empty[i], 1);
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tfull_bar[1], 1);
    mbar_init(&tempty_bar[0], kEpiWarps);
    mbar_init(&tempty_bar[1], kEpiWarps);
    mbar_init(&res_full, kEpiWarps);  // the eight TMEM-filling warps
    s_abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t tmem_w = tmem_base + C::kAccCols;  // resident weights start behind the accumulators

  // This CTA's slot: layer index inside a group and tile of 128 packed gate rows (32 hidden units).
  const int j = blockIdx.x / a.n_tiles;
  const int n_tile = blockIdx.x - j * a.n_tiles;
  const int n_groups = (a.D + a.G - 1) / a.G;
  const int kb_x0 = a.I / BK, kb_h = a.H / BK;
  const int res_t = min(min(a.res_tmem, C::kTmemBlocks), kb_h);  // recurrent K blocks [0, res_t) live in TMEM

  if (warp == 0) {
    // ----------------------------------------------- activation producer (TMA)
    // The whole warp waits for flags; lane 0 issues the copies.
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int g = 0; g < n_groups && ok; ++g) {
      const int l = g * a.G + j;
      if (l >= a.D) continue;
      ok = for_each_half(a.L, [&](bool is_x, int t) -> bool {
        const int* dep = nullptr;
        const CUtensorMap* am;
        int a_row, nkb;
        if (is_x) {
          if (l == 0) {
            am = &mapX;
            a_row = t * a.N;
            nkb = kb_x0;
          } else {
            am = &mapH;
            a_row = ((l - 1) * a.L + t) * a.N;
            nkb = kb_h;
            dep = a.done + ((l - 1) * a.L + t) * a.n_tiles;
          }
        } else {
          am = &mapH;
          a_row = (l * a.L + t - 1) * a.N;
          nkb = kb_h;
          dep = a.done + (l * a.L + t - 1) * a.n_tiles;
        }
        if (dep != nullptr && !warp_wait_flags(dep, a.n_tiles, lane, &s_abort, status)) return false;
        bool fine = true;
        if (lane == 0) {
          FTB_WM_STAMP(l, t, is_x ? 1 : 0);
          // (The hidden states were written by TMA stores and are read by TMA loads: both sides are in
          // the async proxy, so the flag's release/acquire is all the ordering there is.)
          for (int kb0 = 0; kb0 < nkb && fine; kb0 += C::kActBlocks) {
            const int nb = min(C::kActBlocks, nkb - kb0);
            fine = mbar_wait(&act_empty[stage], phase ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_SLOT);
            if (!fine) break;
            mbar_arrive_expect_tx(&act_full[stage], nb * C::kActBlockBytes);
            for (int b = 0; b < nb; ++b)
              tma_load_2d(s_act + stage * kBlockBytes + b * C::kActBlockBytes, am, &act_full[stage], (kb0 + b) * BK,
                          a_row);
            if (++stage == AS) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (!is_x) { FTB_WM_STAMP(l, t, 6); }
        }
        return __all_sync(0xffffffffu, fine);
      });
    }
  } else if (warp == 2) {
    // --------------------------------------------------- weight producer (TMA)
    if (lane == 0) {
      const uint64_t w_policy = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int g = 0; g < n_groups && ok; ++g) {
        const int l = g * a.G + j;
        if (l >= a.D) continue;
        const int w_row = l * 4 * a.H + n_tile * BMW;
        ok = for_each_half(a.L, [&](bool is_x, int t) -> bool {
          const int nkb = is_x ? (l == 0 ? kb_x0 : kb_h) : kb_h;
          const int wk = is_x ? 0 : a.I;
          for (int kb = is_x ? 0 : res_t; kb < nkb; kb += 2) {
            const int nb = min(2, nkb - kb);
            if (!mbar_wait(&w_empty[stage], phase ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_SLOT)) return false;
            mbar_arrive_expect_tx(&w_full[stage], nb * kBlockBytes);
            for (int b = 0; b < nb; ++b)
              tma_load_2d_hint(s_w + (2 * stage + b) * kBlockBytes, &mapW, &w_full[stage], wk + (kb + b) * BK, w_row,
                               w_policy);
            if (++stage == WS) {
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
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(BMW, NB, Fmt<T>::kind, 0, 0);
      // Operand descriptors of the ring bases; a tile further on is the base plus its byte offset / 16.
      const uint64_t act_desc0 = make_sdesc_sw128(smem_u32(s_act), 16, 1024);
      const uint64_t w_desc0 = make_sdesc_sw128(smem_u32(s_w), 16, 1024);
      int as = 0, ws = 0;
      uint32_t aphase = 0, wphase = 0;
      int k_base = 0;  // tiles this CTA has started before the current sweep
      int sweep = 0;
      bool ok = true;
      for (int g = 0; g < n_groups && ok; ++g) {
        const int l = g * a.G + j;
        if (l >= a.D) continue;
        bool res_ready = false;
        ok = for_each_half(a.L, [&](bool is_x, int t) -> bool {
          const int k = k_base + t;  // running tile number of this CTA
          const int acc = k & 1;
          const int nkb = is_x ? (l == 0 ? kb_x0 : kb_h) : kb_h;
          const int kb_ring = is_x ? 0 : res_t;  // first K block of this half that comes through the weight ring
          bool okw = true;
          if (is_x) {
            // First MMA of tile k: its accumulators must have been drained (tile k-2).
            okw = mbar_wait(&tempty_bar[acc], ((k >> 1) & 1) ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_EPI);
            if (!okw) return false;
            tc_fence_after();
          } else if (!res_ready) {
            if (!mbar_wait(&res_full, sweep & 1, &s_abort, status, FTB_ERR_TIMEOUT_TMA)) return false;
            tc_fence_after();
            res_ready = true;
          }
          const uint32_t d_tmem = tmem_base + acc * NB;
          for (int kb = 0; kb < nkb; ++kb) {
            const int ab = kb % C::kActBlocks;  // position inside the activation stage
            if (ab == 0) {
              // (No tcgen05 fence after a barrier that TMA completes: the fence is for data handed over
              // by other threads' tcgen05 operations, and it drains the tensor pipe.)
              okw = mbar_wait(&act_full[as], aphase, &s_abort, status, FTB_ERR_TIMEOUT_TMA);
              if (!is_x && kb == 0) { FTB_WM_STAMP(l, t, 2); }
              if (!is_x && kb + C::kActBlocks >= nkb) { FTB_WM_STAMP(l, t, 3); }
              if (!okw) return false;
            }
            const uint64_t bd = act_desc0 + static_cast<uint64_t>((as * kBlockBytes + ab * C::kActBlockBytes) >> 4);
            if (kb < kb_ring) {
              // weights of this K block live in TMEM: 8 columns per 16 of K
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk)
                umma_ts(d_tmem, tmem_w + kb * 32 + kk * 8, bd + 2 * kk, idesc, 1u);
            } else {
              const int wb = (kb - kb_ring) & 1;  // position inside the weight stage
              if (wb == 0) {
                okw = mbar_wait(&w_full[ws], wphase, &s_abort, status, FTB_ERR_TIMEOUT_TMA);
                if (!okw) return false;
              }
              const uint64_t ad = w_desc0 + static_cast<uint64_t>(((2 * ws + wb) * kBlockBytes) >> 4);
              // The first MMA of a tile overwrites the accumulator.
#pragma unroll
              for (int kk = 0; kk < BK / 16; ++kk)
                umma_ss(d_tmem, ad + 2 * kk, bd + 2 * kk, idesc, (is_x && kb == 0 && kk == 0) ? 0u : 1u);
              if (wb == 1 || kb == nkb - 1) {
                umma_commit(&w_empty[ws]);
                if (++ws == WS) {
                  ws = 0;
                  wphase ^= 1u;
                }
              }
            }
            if (ab == C::kActBlocks - 1 || kb == nkb - 1) {
              umma_commit(&act_empty[as]);
              if (++as == AS) {
                as = 0;
                aphase ^= 1u;
              }
            }
          }
          // The tile is complete after its recurrent half (or after the input half at t = 0).
          if (!is_x || t == 0) umma_commit(&tfull_bar[acc]);
          FTB_WM_STAMP(l, t, is_x ? 5 : 4);
          return true;
        });
        k_base += a.L;
        ++sweep;
      }
    }
  } else if (warp >= kFirstEpiWarp) {
    // ---------------------------------------------------------------- epilogue
    // Warp w reads TMEM lane quadrant w % 4; the two warps of a quadrant split the batch columns.
    // Lane r of the tile is gate (r & 3) of hidden unit (r >> 2); after the quad transpose a thread
    // holds the four gates of its unit for the batch columns congruent to (lane & 3) modulo 4.
    constexpr int kCols = NB / 2;                    // batch columns per warp
    constexpr int kChunk = kCols < 32 ? kCols : 32;  // columns per tcgen05.ld
    constexpr int kChunks = kCols / kChunk;
    constexpr int kOwn = kCols / 4;                  // (unit, batch) elements per thread
    const int q = warp & 3;
    const int half = (warp - kFirstEpiWarp) >> 2;
    const int r_loc = q * 32 + lane;
    const int gate = lane & 3;
    const int unit = n_tile * (BMW / 4) + (r_loc >> 2);
    int k_base = 0;
    bool ok = true;
    for (int g = 0; g < n_groups && ok; ++g) {
      const int l = g * a.G + j;
      if (l >= a.D) continue;
      // Resident recurrent weights -> TMEM: thread r copies its own packed weight row, two 16-bit
      // values per 32-bit column (the layout of an A operand in tensor memory); the two warps of a
      // quadrant take alternate K blocks.  (Every MMA of the previous sweep had finished before this
      // thread read that sweep's last accumulator.)
      {
        const uint4* wrow = reinterpret_cast<const uint4*>(
            reinterpret_cast<const T*>(a.Wp) + (static_cast<size_t>(l) * 4 * a.H + n_tile * BMW + r_loc) * (a.I + a.H) + a.I);
        for (int kb = half; kb < res_t; kb += 2) {
          uint32_t v[32];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint4 x4 = __ldg(wrow + kb * 8 + i);
            v[4 * i + 0] = x4.x; v[4 * i + 1] = x4.y; v[4 * i + 2] = x4.z; v[4 * i + 3] = x4.w;
          }
          tmem_st32(tmem_w + (static_cast<uint32_t>(q * 32) << 16) + kb * 32, v);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&res_full);
      }
      float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
      if (a.bias_p != nullptr)
        bias = __ldg(reinterpret_cast<const float4*>(a.bias_p + static_cast<size_t>(l) * 4 * a.H + n_tile * BMW) + (r_loc >> 2));
      float creg[kOwn];
#pragma unroll
      for (int i = 0; i < kOwn; ++i) creg[i] = 0.f;
      for (int t = 0; t < a.L && ok; ++t) {
        const int k = k_base + t;
        const int acc = k & 1;
        {
          // every lane waits on the accumulator's barrier (a single sleeping lane per warp and a vote were
          // measured slower: this wait is on the chain of a step)
          const bool mine = mbar_wait(&tfull_bar[acc], (k >> 1) & 1, &s_abort, status, FTB_ERR_TIMEOUT_MMA);
          if (!__all_sync(0xffffffffu, mine)) {
            ok = false;
            break;
          }
        }
        tc_fence_after();
        if (warp == kFirstEpiWarp && lane == 0) { FTB_WM_STAMP(l, t, 10); }
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * NB + half * kCols;
        // The step's output goes through a row-major [NB][32] tile in shared memory and one TMA store.
        // The previous step's tile must have left shared memory: the publishing thread arrives here
        // only after its store has completed.
        T* s_tile = reinterpret_cast<T*>(s_out) + (r_loc >> 2);
        asm volatile("bar.sync 2, %0;" ::"n"(32 * kEpiWarps) : "memory");
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch) {
          float v[kChunk];
          {
            uint32_t r[kChunk];
            tmem_ld_cols<kChunk>(taddr + ch * kChunk, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < kChunk; ++i) v[i] = __uint_as_float(r[i]);
          }
#pragma unroll
          for (int kq = 0; kq < kChunk / 4; ++kq) {
            quad_transpose(v[4 * kq], v[4 * kq + 1], v[4 * kq + 2], v[4 * kq + 3], lane);
            const float gi = v[4 * kq + 0] + bias.x;
            const float gf = v[4 * kq + 1] + bias.y;
            const float go = v[4 * kq + 2] + bias.z;
            const float gc = v[4 * kq + 3] + bias.w;
            const int ci = ch * (kChunk / 4) + kq;
            const float c_new = sigmoid_fast(gf) * creg[ci] + sigmoid_fast(gi) * tanh_fast(gc);
            creg[ci] = c_new;
            const float h_new = sigmoid_fast(go) * tanh_fast(c_new);
            const int n = half * kCols + ch * kChunk + 4 * kq + gate;
            store_h<T>(s_tile + n * (BMW / 4), h_new);  // rows past the batch stay in the tile
          }
        }
        if (warp == kFirstEpiWarp && lane == 0) { FTB_WM_STAMP(l, t, 11); }
        // Publish: once the eight epilogue warps have written the tile, one thread stores it with TMA
        // (the first a.N rows), waits for the store and releases the tile's flag; the readers are other
        // CTAs' TMA loads.
        tc_fence_before();
        fence_proxy_async_smem();  // plain shared-memory stores -> the TMA store's reads
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory");
        if (warp == kFirstEpiWarp && lane == 0) {
          tma_store_2d(&mapO, s_out, n_tile * (BMW / 4), (l * a.L + t) * a.N);
          tma_store_commit();
          tma_store_wait<0>();
          st_release_gpu(a.done + (l * a.L + t) * a.n_tiles + n_tile, 1);
          FTB_WM_STAMP(l, t, 12);
        }
      }
      // Final cell state of the sweep.
      if (ok) {
#pragma unroll
        for (int ci = 0; ci < kOwn; ++ci) {
          const int n = half * kCols + (ci / (kChunk / 4)) * kChunk + 4 * (ci % (kChunk / 4)) + gate;
          if (n < a.N) a.c_out[(static_cast<size_t>(l) * a.N + n) * a.H + unit] = creg[ci];
        }
      }
      k_base += a.L;
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (s_abort) {
      // Give copies and MMAs still in flight time to land before TMEM and shared memory go back.
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T, int NB>
int launch(const CUtensorMap& mX, const CUtensorMap& mH, const CUtensorMap& mW, const CUtensorMap& mO, const WArgs& a,
           int grid, cudaStream_t stream) {
  using C = WCfg<NB>;
  static std::atomic<unsigned long long> configured{0};
  auto kfn = lstm_wmajor_kernel<T, NB>;
  if (!ensure_dynamic_smem(kfn, C::kSmemBytes, configured)) return FTB_ERR_LAUNCH;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int na = 0;
  // FTB_NO_COOPERATIVE=1 drops the cooperative attribute (profilers that cannot replay
  // cooperative launches); residency then rests on grid <= SM count on an otherwise idle device,
  // and the bounded waits turn a violated assumption into a status code.
  static const bool no_coop = [] {
    const char* e = getenv("FTB_NO_COOPERATIVE");
    return e != nullptr && e[0] == '1';
  }();
  // FTB_REFUSE_COOPERATIVE=1 answers as if the driver had refused the cooperative launch
  // (host-side failure injection for the tests of the schedule fallback).
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
  if (cudaLaunchKernelEx(&cfg, kfn, mX, mH, mW, mO, a) != cudaSuccess) {
    cudaGetLastError();
    return FTB_ERR_LAUNCH;
  }
  count_launch();
  return FTB_OK;
}

int batch_tile(int N) { return N <= 32 ? 32 : (N <= 64 ? 64 : 128); }

}  // namespace

// True when the weights-major kernel can run the problem: 16-bit, at most 128 sequences, and a
// group of G layers' tiles (4H / 128 each) fits on the device at one CTA per SM.
bool lstm_wmajor_supported(int dtype, int D, int N, int I, int H, int G, int sm_count) {
  if (dtype != FTB_F16 && dtype != FTB_BF16) return false;
  if (N < 1 || N > 128 || H % 64 != 0 || I % 64 != 0 || (D > 1 && I != H) || G < 1) return false;
  return std::min(G, D) * (4 * H / BMW) <= sm_count;
}

// x: [L,N,I]; Wp: [D,4H,I+H]; hs: [D,L,N,H]; c: [D,N,H]; done: D*L*(4H/128) ints (zeroed here).
// resident: < 0 = as many recurrent weight blocks in TMEM as fit, else at most that many (0 = stream all).
int launch_lstm_wmajor(int dtype, const void* x, const void* Wp, const float* bias_p, void* hs, float* c, int D, int L,
                       int N, int I, int H, int G, int resident, int* done, int* status, unsigned long long* trace,
                       cudaStream_t stream) {
  const int NB = batch_tile(N);
  WArgs a;
  a.D = D; a.L = L; a.N = N; a.I = I; a.H = H; a.G = G;
  a.n_tiles = 4 * H / BMW;
  a.res_tmem = resident < 0 ? 16 : resident;
  a.bias_p = bias_p;
  a.Wp = Wp;
  a.hs = hs;
  a.c_out = c;
  a.done = done;
  a.status = status;
  a.trace = trace;
  const int K = I + H;
  CUtensorMap mX, mH, mW, mO;
  int rc;
  if ((rc = make_tmap_2d(&mX, x, dtype, static_cast<uint64_t>(L) * N, I, I, NB, 64))) return rc;
  if ((rc = make_tmap_2d(&mH, hs, dtype, static_cast<uint64_t>(D) * L * N, H, H, NB, 64))) return rc;
  if ((rc = make_tmap_2d(&mW, Wp, dtype, static_cast<uint64_t>(D) * 4 * H, K, K, BMW, 64))) return rc;
  // output boxes: the batch's N rows x the 32 units of a CTA, un-swizzled
  if ((rc = make_tmap_2d(&mO, hs, dtype, static_cast<uint64_t>(D) * L * N, H, H, N, BMW / 4, false))) return rc;
  if (cudaMemsetAsync(done, 0, sizeof(int) * static_cast<size_t>(D) * L * a.n_tiles, stream) != cudaSuccess)
    return FTB_ERR_LAUNCH;
  const int grid = std::min(G, D) * a.n_tiles;
#define FTB_WM_LAUNCH(TT)                                              \
  switch (NB) {                                                        \
    case 32: return launch<TT, 32>(mX, mH, mW, mO, a, grid, stream);       \
    case 64: return launch<TT, 64>(mX, mH, mW, mO, a, grid, stream);       \
    default: return launch<TT, 128>(mX, mH, mW, mO, a, grid, stream);      \
  }
  if (dtype == FTB_F16) {
    FTB_WM_LAUNCH(__half)
  }
  FTB_WM_LAUNCH(__nv_bfloat16)
#undef FTB_WM_LAUNCH
}

}  // namespace ftb
