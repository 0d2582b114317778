// Latency-bound recurrences with small hidden size (H <= 256): the dilated stacked LSTM
// and the 2-D grid RNN, one thread-block cluster per chain of dependent steps.
//
// These programs are chains of small cells: 512 dependent steps of [256 x 512].[512 x 1024]
// in the first layer of the dilated LSTM, 63 anti-diagonals of [64 x 768].[768 x 256] cells
// in the grid.  Run as a generic wavefront, every dependent level costs a trip through
// global memory (store, fence, flag, poll, TMA load: 6-9 us) plus a re-read of the layer's
// weights from L2.  Here
//   * the weights never move: a cluster of CL CTAs owns one chain (one layer and batch slice of
//     the dilated LSTM; one grid row and batch slice of the grid RNN), CTA r of the cluster owns
//     128 packed weight rows (32 LSTM units x 4 gates, or 128 tanh units) for the whole launch,
//     and that slice of the weights sits in tensor memory as the A operand of every MMA
//     ("recurrent weights resident on chip");
//   * the batch is the N side of the MMA (NB = 128 or 64 columns per slice);
//   * the state a chain hands to its own next step -- h(t) of a layer with dilation 1, h_y of
//     the grid cell to the left -- never leaves the cluster: each CTA writes its units into a
//     staging tile and copies it with one bulk shared-memory-to-shared-memory copy per peer into
//     the next step's B operand in every CTA of the cluster (distributed shared memory),
//     completion counted on the receiver's mbarrier.  The receiving layout is the un-swizzled
//     K-major core-matrix layout, in which one CTA's units are one contiguous block;
//   * everything that crosses chains (the layer below, the grid row above, a layer's own state
//     `dilation` >= 2 steps back) goes through global memory with one release flag per
//     (cell, tile), polled by a whole warp, and TMA loads; those consumers run a few steps behind
//     their producers, so this latency adds to the pipeline's depth, not to every step.  The
//     global flag is published by a warp of its own, off the chain.
// Same arithmetic in the same order as the cell kernels of the generic wavefront (input first,
// then the recurrent state(s)): the results are bit-identical.
//
// Roles: warp 0 producer of the TMA-fed operand blocks, warp 1 MMA issuer (owns TMEM), warp 2
// output store and flag publisher, warp 3 idle, warps 4.. epilogue (16 for the LSTM cell, 8 for the
// tanh cell).  tcgen05 cta_group::1; no multicast loads;
// cooperative cluster launch (a chain waits for flags of other clusters).
//
// Programs: dilated_layer()/model() (examples/dilated_rnn/dilated_rnn.py:16-41) in place of
// DilatedLstmRegion1/2 (kaleido/core/device/kernels/lstm/dilated_lstm/region{1,2}.h), and
// stacked_grid_rnns() (examples/grid_rnn/grid_rnn.py:42-122) in place of the grid regions
// (benchmarks/rnn/fractaltensor/grid_lstm/regions/region{1..8}.h).
#include <algorithm>
#include <cstdio>
#include <cstdlib>

#include "ptx.cuh"
#include "tmap.h"

namespace ftb {

namespace {

constexpr int BK = 64;
constexpr int kFirstEpiWarp = 4;
// Epilogue warps: four per TMEM lane quadrant for the LSTM cell (five MUFU operations and a quad
// transpose per element: latency-bound with fewer), two for the tanh cell.
__host__ __device__ constexpr int epi_warps(int mode) { return mode == 0 ? 16 : 8; }
__host__ __device__ constexpr int cta_threads(int mode) { return 32 * (kFirstEpiWarp + epi_warps(mode)); }
constexpr uint32_t kStageBytes = 16384;

constexpr int kMaxLayers = 16;

enum ClusterMode : int { kDilated = 0, kGrid = 1 };

#ifdef FTB_TRACE
// Debug builds: globaltimer stamps of CTA rank 0 of every cluster, [cluster][step][16].
__device__ unsigned long long* g_cluster_trace = nullptr;
#define FTB_CL_STAMP(i, s) \
  if (g_cluster_trace != nullptr && rank == 0) g_cluster_trace[(static_cast<size_t>(cid) * n_steps + (i)) * 16 + (s)] = globaltimer_ns()
#else
#define FTB_CL_STAMP(i, s)
#endif
#ifdef FTB_ACCT
// Debug builds: cycles a role of CTA rank 0 spends in each of its waits, summed over the launch and
// written once at the end: [cluster][16].
__device__ unsigned long long* g_cluster_acct = nullptr;
#define ACCT_DECL(n) long long acct_[n] = {}; long long acct_t0_ = 0; (void)acct_t0_
#define ACCT_BEGIN() acct_t0_ = clock64()
#define ACCT_END(k) acct_[k] += clock64() - acct_t0_
#define ACCT_WRITE(k, slot) if (g_cluster_acct != nullptr && rank == 0) g_cluster_acct[static_cast<size_t>(cid) * 16 + (slot)] = acct_[k]
#else
#define ACCT_DECL(n)
#define ACCT_BEGIN()
#define ACCT_END(k)
#define ACCT_WRITE(k, slot)
#endif

struct ClusterArgs {
  int D, L, N, H;  // layers, steps of a chain (dilated: time steps; grid: B), batch, hidden size
  int A;           // grid: rows of the grid (chains per layer and slice); dilated: 1
  int S;           // grid: batch slices of NB columns; dilated: flag slots per cell (slices of 64)
  int CL;          // CTAs per cluster
  int max_dil;
  int dil[kMaxLayers];
  int nb[kMaxLayers];              // dilated: batch columns per cluster of the layer (64 or 128)
  int first_cluster[kMaxLayers + 1];  // dilated: index of the layer's first cluster
  const void* W0;       // dilated: Wp [D,4H,2H]; grid: Wpx [D,H,3H]
  const void* W1;       // grid: Wpy
  const float* bias0;   // dilated: bias_p [D,4H]; grid: bias_x [D,H]   (or nullptr)
  const float* bias1;   // grid: bias_y
  void* out0;           // dilated: hs [D,L,N,H]; grid: hx [D,A,B,N,H]
  void* out1;           // grid: hy
  float* c;             // dilated: fp32 [D, max_dil*N, H]
  int* flags;           // [cells][CL], zero before the launch
  int* status;
};

// One TMA-fed operand segment of a step: activation rows `row`.. of tensor map `map`, nkb 64-wide K
// blocks, multiplied with the weight K blocks wkb0.. of this CTA's tile; flags to wait for first.
struct Segment {
  int map, row, nkb, wkb0;
  const int* flags;  // nullptr: an input of the call
  int nflags;
};
struct StepPlan {
  int nseg;
  Segment seg[2];
  bool self;       // the cluster's own previous output is an operand (through shared memory)
  int self_wkb0, self_nkb;
};

__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Whole-warp bounded wait until the n flags at `flags` are all non-zero (lane i polls flags i, i+32, ...).
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

// Shared-memory operand descriptor for an un-swizzled K-major tile: core matrices of 8 rows x 16 B
// stored contiguously (128 B); `lbo` = bytes between the two 16-byte K chunks of an MMA's K = 16,
// `sbo` = bytes between consecutive 8-row groups.
__device__ __forceinline__ uint64_t make_sdesc_plain(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  return d;
}

// Bulk copy from this CTA's shared memory into a peer's; completion (bytes) counted on the peer's mbarrier.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster_addr, uint32_t src_addr, uint32_t bytes,
                                                  uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   dst_cluster_addr),
               "r"(src_addr), "r"(bytes), "r"(bar_cluster_addr)
               : "memory");
}

// Arrives, once the MMAs issued so far by this thread are done, on the mbarrier at the same
// shared-memory offset in every CTA of the cluster whose bit is set in `mask`.
__device__ __forceinline__ void umma_commit_to(uint64_t* bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}

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
__device__ __forceinline__ T to_elem(float v);
template <>
__device__ __forceinline__ __half to_elem<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 to_elem<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// What this CTA multiplies at step `i` of its chain.  Every role calls it with the same arguments.
//   dilated: chain = (layer l, slice s), step = time step t.
//   grid:    chain = (layer d, row a, slice s), step = column b.
template <int MODE, int NB>
__device__ __forceinline__ StepPlan plan_step(const ClusterArgs& a, int layer, int row_a, int slice, int rank, int i) {
  StepPlan p;
  p.nseg = 0;
  p.self = false;
  p.self_wkb0 = p.self_nkb = 0;
  const int kbh = a.H / BK;
  if (MODE == kDilated) {
    const int d = a.dil[layer];
    Segment& x = p.seg[p.nseg++];
    x.nkb = kbh;
    x.wkb0 = 0;
    if (layer == 0) {
      x.map = 0;
      x.row = i * a.N + slice * NB;
      x.flags = nullptr;
      x.nflags = 0;
    } else {
      x.map = 1;
      x.row = ((layer - 1) * a.L + i) * a.N + slice * NB;
      // One flag slot per 64 sequences of a cell; a cluster publishes in the slot of its first 64.  The
      // layer below may be cut differently: its clusters that hold this slice's rows own consecutive slots.
      const int nbp = a.nb[layer - 1];
      const int first = (slice * NB / nbp) * (nbp / 64);
      x.flags = a.flags + (((layer - 1) * a.L + i) * a.S + first) * a.CL;
      // (only the clusters that exist: the last slice of the batch may be short)
      x.nflags = (nbp < NB ? min(NB / nbp, (a.N - slice * NB + nbp - 1) / nbp) : 1) * a.CL;
    }
    if (i >= d) {
      if (d == 1) {
        p.self = true;
        p.self_wkb0 = kbh;
        p.self_nkb = kbh;
      } else {
        Segment& h = p.seg[p.nseg++];
        h.map = 1;
        h.row = (layer * a.L + i - d) * a.N + slice * NB;
        h.nkb = kbh;
        h.wkb0 = kbh;
        h.flags = a.flags + ((layer * a.L + i - d) * a.S + slice * (NB / 64)) * a.CL;
        h.nflags = a.CL;
      }
    }
  } else {
    // packed K order of a grid cell: [state_x | state_y | input]; issue order: input, state_x, state_y
    const bool ydir = rank >= a.CL / 2;
    const int cell = (layer * a.A + row_a) * a.L + i;  // a.L = B
    Segment& in = p.seg[p.nseg++];
    in.nkb = kbh;
    in.wkb0 = 2 * kbh;
    if (layer == 0) {
      in.map = ydir ? 1 : 0;
      in.row = ((row_a * a.L + i) * a.N) + slice * NB;
      in.flags = nullptr;
      in.nflags = 0;
    } else {
      const int below = ((layer - 1) * a.A + row_a) * a.L + i;
      in.map = ydir ? 3 : 2;
      in.row = below * a.N + slice * NB;
      in.flags = a.flags + (below * a.S + slice) * a.CL + (ydir ? a.CL / 2 : 0);
      in.nflags = a.CL / 2;
    }
    if (row_a > 0) {
      const int up = (layer * a.A + row_a - 1) * a.L + i;
      Segment& sx = p.seg[p.nseg++];
      sx.map = 2;
      sx.row = up * a.N + slice * NB;
      sx.nkb = kbh;
      sx.wkb0 = 0;
      sx.flags = a.flags + (up * a.S + slice) * a.CL;  // the x-direction tiles come first
      sx.nflags = a.CL / 2;
    }
    if (i > 0) {
      p.self = true;
      p.self_wkb0 = kbh;
      p.self_nkb = kbh;
    }
    (void)cell;
  }
  return p;
}

// map0..map3: activation inputs (boxes of NB rows x 64 columns, 128-byte swizzle).  mapO0/mapO1:
// outputs (dilated: hs; grid: hx, hy) as un-swizzled boxes of NB rows x this CTA's units; mapT0/mapT1:
// the same with the row count of the last, partial batch slice.
template <typename T, int MODE, int NB>
__device__ __forceinline__ void cluster_body(const CUtensorMap& map0, const CUtensorMap& map1, const CUtensorMap& map2,
                                             const CUtensorMap& map3, const CUtensorMap& mapO0,
                                             const CUtensorMap& mapO1, const CUtensorMap& mapT0,
                                             const CUtensorMap& mapT1, const ClusterArgs& a, const int cid,
                                             const int layer, const int row_a, const int slice) {
  constexpr int kEpiWarps = epi_warps(MODE);
  constexpr int kSub = kEpiWarps / 4;              // epilogue warps per TMEM lane quadrant
  constexpr int kBlocksPerStage = 128 / NB;        // [NB x 64] 16-bit blocks per 16 KB stage
  constexpr uint32_t kBlockBytes = NB * BK * 2;
  constexpr int kRing = MODE == kDilated ? 4 : 6;  // stages of the TMA-fed ring when the chain also uses the self slots
  constexpr int kOutUnits = MODE == kDilated ? 32 : 128;                   // units this CTA produces
  constexpr uint32_t kOutTileBytes = static_cast<uint32_t>(NB) * kOutUnits * 2;  // row-major [NB][units] staging
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t ring_full[12], ring_empty[12];  // up to 12 ring stages
  __shared__ uint64_t self_full[2];   // the slot holds the whole previous output (bytes counted)
  __shared__ uint64_t self_free[2];   // producers only: every CTA of the cluster has multiplied the slot's contents
  __shared__ uint64_t stg_ready;      // the eight epilogue warps have written the step's staging tile
  __shared__ int seg_seq;             // operand segments issued into the ring so far (two producer warps)
  __shared__ int out_issued;          // epilogue warps that have staged a step's outputs, summed over steps
  __shared__ int out_stored;          // steps whose output staging tile the publisher has finished reading
  __shared__ uint64_t tfull_bar[2], tempty_bar[2];
  __shared__ uint64_t res_full;
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  int* status = a.status;

  const int kbh = a.H / BK;
  const int n_wkb = MODE == kDilated ? 2 * kbh : 3 * kbh;  // K blocks of this CTA's weight tile, all in TMEM
  const int K = n_wkb * BK;
  // Does the chain hand its own output to its next step through the cluster's shared memory?
  const bool self_chain = MODE == kGrid ? true : (a.dil[layer] == 1);
  // Units of the self operand this CTA produces: dilated: 32 of H; grid: 128 of H, y-direction tiles only.
  const bool self_producer = self_chain && (MODE == kDilated || rank >= a.CL / 2);
  const int self_units = MODE == kDilated ? 32 : 128;
  const int self_first_chunk = (MODE == kDilated ? rank : rank - a.CL / 2) * (self_units / 8);
  const uint16_t producer_mask = static_cast<uint16_t>(MODE == kDilated ? ((1u << a.CL) - 1u)
                                                                        : (((1u << a.CL) - 1u) & ~((1u << (a.CL / 2)) - 1u)));
  const uint32_t self_slot_bytes = static_cast<uint32_t>(a.H / 8) * NB * 16;  // H units x NB rows, 16-bit
  const uint32_t stage_tile_bytes = static_cast<uint32_t>(self_units / 8) * NB * 16;
  // Shared memory: [self slot 0][self slot 1][staging 0][staging 1][output tile 0][output tile 1][ring ...];
  // chains without a self operand have the output tiles and a longer ring only.
  uint8_t* s_self = smem;
  uint8_t* s_stg = s_self + (self_chain ? 2 * self_slot_bytes : 0);
  uint8_t* s_out = s_stg + (self_chain ? 2 * stage_tile_bytes : 0);  // two row-major output tiles for the TMA stores
  uint8_t* s_ring = s_out + 2 * kOutTileBytes;
  const int n_ring = self_chain ? kRing : 12;
  // ring stages a segment (the H / 64 K blocks of NB rows) takes
  const int seg_stages = (a.H / BK + kBlocksPerStage - 1) / kBlocksPerStage;

  if (threadIdx.x == 0) {
    prefetch_tmap(&map0);
    prefetch_tmap(&map1);
    prefetch_tmap(&map2);
    prefetch_tmap(&map3);
    prefetch_tmap(&mapO0);
    prefetch_tmap(&mapO1);
    prefetch_tmap(&mapT0);
    prefetch_tmap(&mapT1);
    for (int i = 0; i < 12; ++i) {
      mbar_init(&ring_full[i], 1);
      mbar_init(&ring_empty[i], 1);
    }
    mbar_init(&self_full[0], 1);
    mbar_init(&self_full[1], 1);
    mbar_init(&self_free[0], a.CL);
    mbar_init(&self_free[1], a.CL);
    mbar_init(&stg_ready, kEpiWarps);
    seg_seq = 0;
    out_issued = 0;
    out_stored = 0;
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tfull_bar[1], 1);
    mbar_init(&tempty_bar[0], kEpiWarps);
    mbar_init(&tempty_bar[1], kEpiWarps);
    mbar_init(&res_full, kEpiWarps);
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
  // Peers copy into this CTA's shared memory and arrive on its barriers: nobody starts before all are set up.
  cluster_sync_all();
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t tmem_w = tmem_base + 2 * NB;  // the weight tile sits behind the two accumulators

  const CUtensorMap* maps[4] = {&map0, &map1, &map2, &map3};
  const int n_steps = a.L;
  const int my_flag_cell0 = MODE == kDilated ? (layer * a.L) : ((layer * a.A + row_a) * a.L);

  if (warp == 0 || warp == 3) {
    // ------------------------------------------ producers of the TMA-fed operand blocks
    // One three-dimensional copy per segment: the NB rows of all its K blocks land in consecutive
    // [NB x 64] tiles of the ring (a segment never wraps: the ring is a whole number of segments long)
    // and complete on the barrier of the segment's first stage; the MMA warp frees a segment through
    // the empty barrier of that same stage.
    // Two warps share the work by segment: warp 0 takes a step's first segment (the input), warp 3
    // its second (the state that arrives through global memory), so one segment's flag wait overlaps
    // the other's ring wait and copy.  Both walk every segment to keep the ring position, and the ring
    // is filled in segment order whichever warp fills it: a warp waits for `seg_seq` to reach its
    // segment's number before it touches the ring (otherwise the warp with the lighter segments could
    // lap the other one and meet a stage's barrier a whole round early, where the parity test cannot
    // tell "not yet filled" from "already drained").
    const int mine = warp == 0 ? 0 : 1;
    int stage = 0, q = 0;
    uint32_t phase = 0;
    bool ok = true;
    volatile int* seq = &seg_seq;
    ACCT_DECL(4);
    for (int i = 0; i < n_steps && ok; ++i) {
      const StepPlan p = plan_step<MODE, NB>(a, layer, row_a, slice, rank, i);
      for (int s = 0; s < p.nseg && ok; ++s) {
        const Segment& sg = p.seg[s];
        if ((s & 1) == mine) {
          ACCT_BEGIN();
          if (sg.flags != nullptr && !warp_wait_flags(sg.flags, sg.nflags, lane, &s_abort, status)) {
            ok = false;
            break;
          }
          ACCT_END(0);
          bool fine = true;
          if (lane == 0) {
            // (Producers write their outputs with TMA stores and consumers read them with TMA loads: both
            // sides are in the async proxy, so the flag's release/acquire is all the ordering there is.)
            FTB_CL_STAMP(i, 7 + 2 * s);
            ACCT_BEGIN();
            if (*seq != q) {
              const uint64_t t0 = globaltimer_ns();
              uint32_t it = 0;
              while (*seq != q) {
                if (((++it) & 0xFF) == 0 && (s_abort || globaltimer_ns() - t0 > FTB_WAIT_TIMEOUT_NS)) break;
              }
              if (*seq != q) {
                fine = false;
                if (!s_abort) {
                  s_abort = 1;
                  atomicCAS(status, 0, FTB_ERR_TIMEOUT_SLOT);
                }
              }
            }
            ACCT_END(1);
            ACCT_BEGIN();
            if (fine) fine = mbar_wait(&ring_empty[stage], phase ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_SLOT);
            ACCT_END(2);
            ACCT_BEGIN();
            if (fine) {
              mbar_arrive_expect_tx(&ring_full[stage], sg.nkb * kBlockBytes);
              tma_load_3d(s_ring + stage * kStageBytes, maps[sg.map], &ring_full[stage], 0, sg.row, 0);
              *seq = q + 1;
            }
            ACCT_END(3);
            FTB_CL_STAMP(i, 8 + 2 * s);
          }
          ok = __all_sync(0xffffffffu, fine);
        }
        ++q;
        stage += seg_stages;
        if (stage == n_ring) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    if (lane == 0) {
      ACCT_WRITE(0, mine * 4 + 0);  // flags
      ACCT_WRITE(1, mine * 4 + 1);  // segment order
      ACCT_WRITE(2, mine * 4 + 2);  // ring slots
      ACCT_WRITE(3, mine * 4 + 3);  // issue
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(128, NB, Fmt<T>::kind, 0, 0);
      const uint64_t ring_desc0 = make_sdesc_sw128(smem_u32(s_ring), 16, 1024);
      const uint64_t self_desc0 = make_sdesc_plain(smem_u32(s_self), NB * 16, 128);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = mbar_wait(&res_full, 0, &s_abort, status, FTB_ERR_TIMEOUT_TMA);
      tc_fence_after();
      ACCT_DECL(6);
#ifdef FTB_ACCT
      const long long acct_loop0 = clock64();
#endif
      // What this thread needs of a step's plan, without the addresses the other roles compute (it is
      // the one thread every MMA of the CTA goes through: its own instructions are the step's floor).
      const int kbh = a.H / BK;
      const int d_layer = MODE == kDilated ? a.dil[layer] : 1;
      for (int i = 0; i < n_steps && ok; ++i) {
        int nseg, wkb0[2];
        bool self;
        if (MODE == kDilated) {
          nseg = (d_layer > 1 && i >= d_layer) ? 2 : 1;
          wkb0[0] = 0;
          wkb0[1] = kbh;
          self = d_layer == 1 && i >= 1;
        } else {
          nseg = row_a > 0 ? 2 : 1;
          wkb0[0] = 2 * kbh;  // packed K order of a grid cell: [state_x | state_y | input]
          wkb0[1] = 0;
          self = i > 0;
        }
        const int acc = i & 1;
        ACCT_BEGIN();
        ok = mbar_wait(&tempty_bar[acc], ((i >> 1) & 1) ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_EPI);
        ACCT_END(0);
        if (!ok) break;
        tc_fence_after();
        FTB_CL_STAMP(i, 0);
        const uint32_t d_tmem = tmem_base + acc * NB;
        uint32_t accumulate = 0;  // the first MMA of a step overwrites the accumulator
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (s >= nseg) break;
          ACCT_BEGIN();
          ok = mbar_wait(&ring_full[stage], phase, &s_abort, status, FTB_ERR_TIMEOUT_TMA);
          ACCT_END(1);
          if (!ok) break;
          FTB_CL_STAMP(i, 12 + s);
          const uint64_t bd0 = ring_desc0 + static_cast<uint64_t>((stage * kStageBytes) >> 4);
          const uint32_t aw = tmem_w + wkb0[s] * 32;
          ACCT_BEGIN();
          for (int kb = 0; kb < kbh; ++kb) {
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
              umma_ts(d_tmem, aw + kb * 32 + kk * 8, bd0 + static_cast<uint64_t>((kb * kBlockBytes) >> 4) + 2 * kk, idesc,
                      accumulate);
              accumulate = 1;
            }
          }
          ACCT_END(4);
          ACCT_BEGIN();
          umma_commit(&ring_empty[stage]);  // the whole segment, on its first stage's barrier
          ACCT_END(5);
          stage += seg_stages;
          if (stage == n_ring) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        FTB_CL_STAMP(i, 1);
        if (self) {
          // The cluster's own output of step i-1, copied by its producers into slot (i-1) & 1 of every CTA.
          const int slot = (i - 1) & 1;
          mbar_arrive_expect_tx(&self_full[slot], self_slot_bytes);
          ACCT_BEGIN();
          ok = mbar_wait(&self_full[slot], ((i - 1) >> 1) & 1, &s_abort, status, FTB_ERR_TIMEOUT_TMA);
          ACCT_END(2);
          if (!ok) break;
          FTB_CL_STAMP(i, 2);
          // K = 16 is two 16-byte chunks, NB * 16 bytes apart; 8-row groups are 128 bytes apart; the
          // descriptor of MMA j is the slot's plus j * 2 * NB (bytes / 16): nothing is rebuilt per MMA.
          uint64_t bd = self_desc0 + static_cast<uint64_t>((slot * self_slot_bytes) >> 4);
          uint32_t aw = tmem_w + kbh * 32;
          const int n_self = kbh * (BK / 16);
#pragma unroll 4
          for (int j = 0; j < n_self; ++j) {
            umma_ts(d_tmem, aw, bd, idesc, accumulate);
            accumulate = 1;
            aw += 8;
            bd += 2 * NB;
          }
          umma_commit_to(&self_free[slot], producer_mask);
        }
        umma_commit(&tfull_bar[acc]);
        FTB_CL_STAMP(i, 3);
      }
#ifdef FTB_ACCT
      acct_[3] = clock64() - acct_loop0;
#endif
      ACCT_WRITE(0, 8);   // accumulator free
      ACCT_WRITE(1, 9);   // ring data
      ACCT_WRITE(2, 10);  // self operand
      ACCT_WRITE(3, 11);  // whole loop
      ACCT_WRITE(4, 15);  // MMA issue (ring operands)
      if (MODE == kDilated && a.dil[layer] > 1) { ACCT_WRITE(5, 10); }  // commits (the slot of the self operand, unused here)
    }
  } else if (warp == 2) {
    // ------------------------------------------------ output store and flag publisher
    // The epilogue warps count themselves in `out_issued` once their part of a step's output tile is
    // staged in shared memory; this thread writes the tile to global memory with one TMA store, waits
    // for it to complete and releases the step's flag -- all of it off the chain's critical path.
    // (A running count, not an mbarrier: this thread may fall more than one step behind.)
    if (lane == 0) {
      volatile int* issued = &out_issued;
      volatile int* stored = &out_stored;
      const int n_valid = min(NB, a.N - slice * NB);
      const bool ydir = MODE == kGrid && rank >= a.CL / 2;
      const CUtensorMap* om = n_valid == NB ? (ydir ? &mapO1 : &mapO0) : (ydir ? &mapT1 : &mapT0);
      const int unit0 = MODE == kDilated ? rank * 32 : (ydir ? rank - a.CL / 2 : rank) * 128;
      ACCT_DECL(2);
      for (int i = 0; i < n_steps; ++i) {
        const int want = kEpiWarps * (i + 1);
        ACCT_BEGIN();
        if (*issued < want) {
          const uint64_t t0 = globaltimer_ns();
          uint32_t it = 0;
          while (*issued < want) {
            if (((++it) & 0xFF) == 0 && (s_abort || globaltimer_ns() - t0 > FTB_WAIT_TIMEOUT_NS)) break;
          }
          if (*issued < want) {
            if (!s_abort) {
              s_abort = 1;
              atomicCAS(status, 0, FTB_ERR_TIMEOUT_EPI);
            }
            break;
          }
        }
        ACCT_END(0);
        ACCT_BEGIN();
        __threadfence_block();
        const int cell_row = (MODE == kDilated ? (layer * a.L + i) : ((layer * a.A + row_a) * a.L + i)) * a.N + slice * NB;
        tma_store_2d(om, s_out + (i & 1) * kOutTileBytes, unit0, cell_row);
        tma_store_commit();
        tma_store_wait_read<0>();
        *stored = i + 1;  // the tile may be overwritten (two steps from now)
        tma_store_wait<0>();
        st_release_gpu(a.flags + ((my_flag_cell0 + i) * a.S + slice * (MODE == kDilated ? NB / 64 : 1)) * a.CL + rank, 1);
        ACCT_END(1);
        FTB_CL_STAMP(i, 11);
      }
      ACCT_WRITE(0, 13);  // staged outputs
      ACCT_WRITE(1, 14);  // store, wait, flag
    }
  } else if (warp >= kFirstEpiWarp) {
    // ---------------------------------------------------------------- epilogue
    constexpr int kCols = NB / kSub;  // batch columns per warp (32 in both modes)
    static_assert(kCols == 32 || kCols == 16, "an epilogue warp takes 16 or 32 accumulator columns");
    const int q = warp & 3;
    const int sub = (warp - kFirstEpiWarp) >> 2;
    const int r_loc = q * 32 + lane;  // row of the 128-row tile = TMEM lane
    // Resident weights -> TMEM: thread r copies its packed weight row, two 16-bit values per 32-bit
    // column (the layout of an A operand in tensor memory); the warps of a quadrant alternate K blocks.
    {
      const T* wbase;
      if (MODE == kDilated) {
        wbase = reinterpret_cast<const T*>(a.W0) + (static_cast<size_t>(layer) * 4 * a.H + rank * 128 + r_loc) * K;
      } else {
        const bool ydir = rank >= a.CL / 2;
        const int tile = ydir ? rank - a.CL / 2 : rank;
        wbase = reinterpret_cast<const T*>(ydir ? a.W1 : a.W0) + (static_cast<size_t>(layer) * a.H + tile * 128 + r_loc) * K;
      }
      const uint4* wrow = reinterpret_cast<const uint4*>(wbase);
      for (int kb = sub; kb < n_wkb; kb += kSub) {
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

    // Per-thread constants of the two epilogues.
    const int gate = lane & 3;
    int unit;        // hidden unit this thread produces (dilated: after the quad transpose)
    int u_local;     // the same, counted inside this CTA's tile
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float bias1 = 0.f;
    if (MODE == kDilated) {
      u_local = r_loc >> 2;
      unit = rank * 32 + u_local;
      if (a.bias0 != nullptr)
        bias4 = __ldg(reinterpret_cast<const float4*>(a.bias0 + static_cast<size_t>(layer) * 4 * a.H + rank * 128) + u_local);
    } else {
      const bool ydir = rank >= a.CL / 2;
      u_local = r_loc;
      unit = (ydir ? rank - a.CL / 2 : rank) * 128 + r_loc;
      const float* bp = ydir ? a.bias1 : a.bias0;
      if (bp != nullptr) bias1 = __ldg(bp + static_cast<size_t>(layer) * a.H + unit);
    }
    const int dil = MODE == kDilated ? a.dil[layer] : 1;
    constexpr int kOwn = kCols / 4;  // LSTM: (unit, batch column) elements per thread
    float creg[kOwn];
#pragma unroll
    for (int i = 0; i < kOwn; ++i) creg[i] = 0.f;
    const int n_valid = min(NB, a.N - slice * NB);  // batch columns of this slice that exist
    // Where this thread's unit sits (a) in the self operand / its staging tile: 16-byte chunk
    // (u_local / 8) of NB rows, then row n, then the unit's 2 bytes; (b) in the row-major output tile.
    const uint32_t stg_unit_off = static_cast<uint32_t>(u_local >> 3) * NB * 16 + (u_local & 7) * 2;
    const uint32_t out_unit_off = static_cast<uint32_t>(u_local) * 2;
    volatile int* stored = &out_stored;
    ACCT_DECL(2);

    bool ok = true;
    for (int i = 0; i < n_steps && ok; ++i) {
      const int acc = i & 1;
      // cell state of a layer with dilation > 1 lives in global memory between the steps that share it
      float* c_rows = nullptr;
      if (MODE == kDilated && dil > 1)
        c_rows = a.c + (static_cast<size_t>(layer) * a.max_dil + (i % dil)) * a.N * a.H + static_cast<size_t>(slice) * NB * a.H;
      if (MODE == kDilated && dil > 1 && i >= dil) {
#pragma unroll
        for (int ci = 0; ci < kOwn; ++ci) {
          const int n = sub * kCols + 4 * ci + gate;
          creg[ci] = n < n_valid ? __ldcg(c_rows + static_cast<size_t>(n) * a.H + unit) : 0.f;
        }
      } else if (MODE == kDilated && dil > 1) {
#pragma unroll
        for (int ci = 0; ci < kOwn; ++ci) creg[ci] = 0.f;
      }
      {
        // every lane waits on the accumulator's barrier (a single sleeping lane per warp and a vote
        // were measured slower: this wait is on the chain of a step)
        bool mine = mbar_wait(&tfull_bar[acc], (i >> 1) & 1, &s_abort, status, FTB_ERR_TIMEOUT_MMA);
        if (lane == 0) {
          ACCT_BEGIN();
          ACCT_END(0);
          // the output tile of two steps ago must have left shared memory
          if (mine && *stored < i - 1) {
            const uint64_t t0 = globaltimer_ns();
            while (*stored < i - 1 && !s_abort && globaltimer_ns() - t0 < FTB_WAIT_TIMEOUT_NS) __nanosleep(64);
            mine = *stored >= i - 1;
          }
        }
        if (!__all_sync(0xffffffffu, mine)) {
          ok = false;
          break;
        }
      }
      tc_fence_after();
      if (warp == kFirstEpiWarp && lane == 0) { FTB_CL_STAMP(i, 4); }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * NB + sub * kCols;
      uint8_t* stg = s_stg + (i & 1) * stage_tile_bytes + stg_unit_off;
      uint8_t* outp = s_out + (i & 1) * kOutTileBytes + out_unit_off;
      float v[kCols];
      {
        uint32_t r[kCols];
        tmem_ld_cols<kCols>(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < kCols; ++k) v[k] = __uint_as_float(r[k]);
      }
      // the accumulator is in registers: the MMA issuer may reuse it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (MODE == kDilated) {
#pragma unroll
        for (int kq = 0; kq < kCols / 4; ++kq) {
          quad_transpose(v[4 * kq], v[4 * kq + 1], v[4 * kq + 2], v[4 * kq + 3], lane);
          const float gi = v[4 * kq + 0] + bias4.x;
          const float gf = v[4 * kq + 1] + bias4.y;
          const float go = v[4 * kq + 2] + bias4.z;
          const float gc = v[4 * kq + 3] + bias4.w;
          const float c_new = sigmoid_fast(gf) * creg[kq] + sigmoid_fast(gi) * tanh_fast(gc);
          creg[kq] = c_new;
          const T h_new = to_elem<T>(sigmoid_fast(go) * tanh_fast(c_new));
          const int n = sub * kCols + 4 * kq + gate;
          *reinterpret_cast<T*>(outp + n * (kOutUnits * 2)) = h_new;
          if (self_producer) *reinterpret_cast<T*>(stg + n * 16) = h_new;
        }
      } else {
#pragma unroll
        for (int k = 0; k < kCols; ++k) {
          const T h_new = to_elem<T>(tanh_fast(v[k] + bias1));
          const int n = sub * kCols + k;
          *reinterpret_cast<T*>(outp + n * (kOutUnits * 2)) = h_new;
          if (self_producer) *reinterpret_cast<T*>(stg + n * 16) = h_new;
        }
      }
      if (MODE == kDilated && (dil > 1 || i == n_steps - 1)) {
        float* c_out = dil > 1 ? c_rows : a.c + static_cast<size_t>(layer) * a.max_dil * a.N * a.H + static_cast<size_t>(slice) * NB * a.H;
#pragma unroll
        for (int ci = 0; ci < kOwn; ++ci) {
          const int n = sub * kCols + 4 * ci + gate;
          if (n < n_valid) c_out[static_cast<size_t>(n) * a.H + unit] = creg[ci];
        }
      }
      if (warp == kFirstEpiWarp && lane == 0) { FTB_CL_STAMP(i, 5); }
      fence_proxy_async_smem();  // plain shared-memory stores -> the bulk copies' and the TMA store's reads
      __syncwarp();
      if (warp == kFirstEpiWarp && lane == 0) { FTB_CL_STAMP(i, 14); }
      if (self_producer && i + 1 < n_steps) {
        // Hand the step's output to every CTA of the cluster, once all of them have multiplied what the
        // destination slot held before (two steps ago).
        // Once all epilogue warps have staged their parts, the tile goes to every CTA of the cluster by
        // bulk copies issued side by side by different warps.  (Measured: the SM's copy engine moves
        // about 64 KB in 1.3-2 us however the tile is cut -- 128 copies of 512 B, 32 of 2 KB or 8 of
        // 8 KB -- so the hand-off is bound by the bytes every CTA must receive, not by the slicing.)
        if (lane == 0) mbar_arrive(&stg_ready);
        const uint32_t kPiece = MODE == kGrid ? stage_tile_bytes : 2048u;
        const int n_pieces = static_cast<int>(stage_tile_bytes / kPiece);
        const int n_copies = n_pieces * a.CL;
        const int per_warp = (n_copies + kEpiWarps - 1) / kEpiWarps;
        const int ci = (warp - kFirstEpiWarp) * per_warp + lane;
        if (lane < per_warp && ci < n_copies) {
          bool go = mbar_wait(&stg_ready, i & 1, &s_abort, status, FTB_ERR_TIMEOUT_EPI);
          if (warp == kFirstEpiWarp && lane == 0) { FTB_CL_STAMP(i, 15); }
          if (go && i >= 2) go = mbar_wait(&self_free[i & 1], ((i - 2) >> 1) & 1, &s_abort, status, FTB_ERR_TIMEOUT_EPI);
          if (go) {
            const int peer = ci / n_pieces;
            const uint32_t off = static_cast<uint32_t>(ci - peer * n_pieces) * kPiece;
            const uint32_t src = smem_u32(s_stg + (i & 1) * stage_tile_bytes) + off;
            const uint32_t dst = smem_u32(s_self + (i & 1) * self_slot_bytes) +
                                 static_cast<uint32_t>(self_first_chunk) * NB * 16 + off;
            bulk_copy_to_peer(map_to_cta(dst, peer), src, kPiece, map_to_cta(smem_u32(&self_full[i & 1]), peer));
            if (warp == kFirstEpiWarp && lane == 0) { FTB_CL_STAMP(i, 6); }
          }
        }
      }
      // this warp's part of the output tile is staged: count it in for the publisher
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        atomicAdd(&out_issued, 1);
      }
    }
    if (warp == kFirstEpiWarp && lane == 0) { ACCT_WRITE(0, 12); }  // accumulator complete
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  // No CTA of the cluster may leave while a peer can still copy into it or signal its barriers.
  cluster_sync_all();
  if (warp == 1) {
    if (s_abort) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Grid RNN: every cluster has the same shape; cluster -> (layer, grid row, batch slice).
template <typename T, int MODE, int NB>
__global__ void __launch_bounds__(cta_threads(MODE), 1)
rnn_cluster_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                   const __grid_constant__ CUtensorMap map2, const __grid_constant__ CUtensorMap map3,
                   const __grid_constant__ CUtensorMap mapO0, const __grid_constant__ CUtensorMap mapO1,
                   const __grid_constant__ CUtensorMap mapT0, const __grid_constant__ CUtensorMap mapT1,
                   const ClusterArgs a) {
  const int cid = blockIdx.x / a.CL;
  const int slice = cid % a.S;
  const int ra = cid / a.S;
  const int layer = ra / a.A;
  const int row_a = ra - layer * a.A;
  cluster_body<T, MODE, NB>(map0, map1, map2, map3, mapO0, mapO1, mapT0, mapT1, a, cid, layer, row_a, slice);
}

// Dilated LSTM: a layer's clusters take 64 or 128 sequences each (a.nb[layer]).  A layer whose step
// depends on its own previous step (dilation 1) is a chain of hand-offs inside the cluster, whose
// latency grows with the slice (state bytes every CTA receives, accumulator columns per epilogue
// warp): it runs on slices of 64; the other layers, whose steps are bound by throughput, on 128.
// x128/h128/o128/t128: the input, the hidden states, the output tile and the output tile of the
// batch's last (short) slice as boxes of 128 rows; x64... the same with 64 rows.
template <typename T>
__global__ void __launch_bounds__(cta_threads(kDilated), 1)
rnn_cluster_dilated_kernel(const __grid_constant__ CUtensorMap x128, const __grid_constant__ CUtensorMap h128,
                           const __grid_constant__ CUtensorMap x64, const __grid_constant__ CUtensorMap h64,
                           const __grid_constant__ CUtensorMap o128, const __grid_constant__ CUtensorMap o64,
                           const __grid_constant__ CUtensorMap t128, const __grid_constant__ CUtensorMap t64,
                           const ClusterArgs a) {
  const int cid = blockIdx.x / a.CL;
  int layer = 0;
  while (layer + 1 < a.D && cid >= a.first_cluster[layer + 1]) ++layer;
  const int slice = cid - a.first_cluster[layer];
  if (a.nb[layer] == 64)
    cluster_body<T, kDilated, 64>(x64, h64, h64, h64, o64, o64, t64, t64, a, cid, layer, 0, slice);
  else
    cluster_body<T, kDilated, 128>(x128, h128, h128, h128, o128, o128, t128, t128, a, cid, layer, 0, slice);
}

// Tensor map of a row-major [rows, H] activation matrix as the kernel's operand loads see it: three
// dimensions (64 columns of a K block, rows, K blocks), so that one copy brings the NB rows of all
// H / 64 K blocks of a segment into consecutive 128-byte-swizzled [NB x 64] tiles of the ring.
int make_operand_map(CUtensorMap* out, const void* base, int dtype, uint64_t rows, int H, int nb) {
  return make_tmap_3d(out, base, dtype, 64, rows, static_cast<uint64_t>(H / 64), static_cast<uint64_t>(H) * 2, 128, 64,
                      static_cast<uint32_t>(nb), static_cast<uint32_t>(H / 64));
}

template <typename Kernel>
int launch_kernel(Kernel kfn, int threads, std::atomic<unsigned long long>& configured, const CUtensorMap* m,
                  const ClusterArgs& a, int grid, uint32_t smem_bytes, cudaStream_t stream) {
  // the largest request of this instantiation (static shared memory comes on top of it)
  constexpr int kMaxDynamic = 226 * 1024;
  if (smem_bytes > static_cast<uint32_t>(kMaxDynamic) || !ensure_dynamic_smem(kfn, kMaxDynamic, configured))
    return FTB_ERR_LAUNCH;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  attrs[na].id = cudaLaunchAttributeClusterDimension;
  attrs[na].val.clusterDim.x = a.CL;
  attrs[na].val.clusterDim.y = 1;
  attrs[na].val.clusterDim.z = 1;
  ++na;
  // FTB_NO_COOPERATIVE=1 drops the cooperative attribute (profilers that cannot replay cooperative
  // launches); residency then rests on the grid fitting an otherwise idle device, and the bounded
  // waits turn a violated assumption into a status code.
  static const bool no_coop = [] {
    const char* e = getenv("FTB_NO_COOPERATIVE");
    return e != nullptr && e[0] == '1';
  }();
  // FTB_REFUSE_COOPERATIVE=1 answers as if the driver had refused the launch (host-side failure
  // injection for the tests of the fallback to the generic wavefront).
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
  const cudaError_t err = cudaLaunchKernelEx(&cfg, kfn, m[0], m[1], m[2], m[3], m[4], m[5], m[6], m[7], a);
  if (err != cudaSuccess) {
    if (getenv("FTB_VERBOSE") != nullptr) fprintf(stderr, "rnn_cluster launch: %s\n", cudaGetErrorString(err));
    cudaGetLastError();
    return FTB_ERR_LAUNCH;
  }
  count_launch();
  return FTB_OK;
}

template <typename T, int MODE, int NB>
int launch(const CUtensorMap* m, const ClusterArgs& a, int grid, uint32_t smem_bytes, cudaStream_t stream) {
  static std::atomic<unsigned long long> configured{0};
  return launch_kernel(rnn_cluster_kernel<T, MODE, NB>, cta_threads(MODE), configured, m, a, grid, smem_bytes, stream);
}
template <typename T>
int launch_dilated(const CUtensorMap* m, const ClusterArgs& a, int grid, uint32_t smem_bytes, cudaStream_t stream) {
  static std::atomic<unsigned long long> configured{0};
  return launch_kernel(rnn_cluster_dilated_kernel<T>, cta_threads(kDilated), configured, m, a, grid, smem_bytes, stream);
}

uint32_t smem_for(bool any_self, int H, int NB, int self_units, int out_units, int ring_self) {
  // worst case over the chains of the launch; must agree with the kernel's carve-up
  const uint32_t out_tiles = 2u * NB * out_units * 2;
  const uint32_t with_self = 2u * (H / 8) * NB * 16 + 2u * (self_units / 8) * NB * 16 + out_tiles + ring_self * kStageBytes;
  const uint32_t without = out_tiles + 12u * kStageBytes;
  return (any_self ? std::max(with_self, without) : without) + 1024;
}

}  // namespace

// ------------------------------------------------------------------ dilated LSTM
namespace {
// Slice width per layer: 64 for the layers with dilation 1 when the clusters still fit, else 128
// everywhere.  Returns the number of clusters, 0 when even slices of 128 do not fit.
int dilated_slices(const int* dilations, int D, int N, int max_clusters, int* nb) {
  const int s128 = (N + 127) / 128, s64 = (N + 63) / 64;
  auto narrow = [&](int l) { return N <= 64 || (dilations != nullptr && dilations[l] == 1); };
  int mixed = 0;
  for (int l = 0; l < D; ++l) mixed += narrow(l) ? s64 : s128;
  const bool use_mixed = s64 <= 8 && mixed <= max_clusters;
  int total = 0;
  for (int l = 0; l < D; ++l) {
    const bool n64 = use_mixed && narrow(l);
    if (nb != nullptr) nb[l] = n64 ? 64 : 128;
    total += n64 ? s64 : s128;
  }
  return s128 <= 8 && total <= max_clusters ? total : 0;
}

// Clusters of `cl` CTAs of the dilated kernel that can be resident at once on the current device (a
// cluster needs its CTAs' SMs inside one GPC, so this is less than SMs / cl: 15 clusters of 8 on a
// 148-SM B200).  0 when the query fails.
int dilated_max_clusters(int dtype, int cl, uint32_t smem) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cl * 32);
  cfg.blockDim = dim3(cta_threads(kDilated));
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = cl;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  int n = 0;
  cudaError_t e;
  if (dtype == FTB_F16) {
    static std::atomic<unsigned long long> configured{0};
    if (!ensure_dynamic_smem(rnn_cluster_dilated_kernel<__half>, 226 * 1024, configured)) return 0;
    e = cudaOccupancyMaxActiveClusters(&n, rnn_cluster_dilated_kernel<__half>, &cfg);
  } else {
    static std::atomic<unsigned long long> configured{0};
    if (!ensure_dynamic_smem(rnn_cluster_dilated_kernel<__nv_bfloat16>, 226 * 1024, configured)) return 0;
    e = cudaOccupancyMaxActiveClusters(&n, rnn_cluster_dilated_kernel<__nv_bfloat16>, &cfg);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}
}  // namespace

bool lstm_dilated_cluster_supported(int dtype, int D, int N, int H, int sm_count) {
  if (dtype != FTB_F16 && dtype != FTB_BF16) return false;
  if (H != 64 && H != 128 && H != 256) return false;  // 4H / 128 = 2, 4 or 8 CTAs per cluster
  if (D < 1 || D > kMaxLayers || N < 1) return false;
  // (coarse: the launcher asks the driver how many clusters fit and falls back if these do not)
  return dilated_slices(nullptr, D, N, sm_count / (4 * H / 128), nullptr) > 0;
}

// one flag per (cell, slot of 64 sequences, CTA of the cluster); at most 16 slots (8 slices of 128) x 8 CTAs
size_t lstm_dilated_cluster_flag_ints(int D, int L) { return static_cast<size_t>(D) * L * 16 * 8; }

// x: [L,N,H]; Wp: [D,4H,2H]; hs: [D,L,N,H]; c: [D, max_dil*N, H]; flags: D*L*S*CL ints (zeroed here).
int launch_lstm_dilated_cluster(int dtype, const void* x, const void* Wp, const float* bias_p, void* hs, float* c,
                                const int* dilations, int D, int L, int N, int H, int* flags, int* status,
                                cudaStream_t stream) {
  ClusterArgs a = {};
  a.D = D; a.L = L; a.N = N; a.H = H; a.A = 1;
  a.S = 2 * ((N + 127) / 128);  // flag slots per cell
  a.CL = 4 * H / 128;
  a.max_dil = 1;
  bool any_self = false;
  for (int l = 0; l < D; ++l) {
    a.dil[l] = dilations[l];
    a.max_dil = std::max(a.max_dil, dilations[l]);
    any_self = any_self || dilations[l] == 1;
  }
  const uint32_t smem = smem_for(any_self, H, 128, 32, 32, 4);
  const int clusters = dilated_slices(dilations, D, N, dilated_max_clusters(dtype, a.CL, smem), a.nb);
  if (clusters <= 0) return FTB_ERR_LAUNCH;  // does not fit on this device: the caller's generic wavefront takes it
  a.first_cluster[0] = 0;
  for (int l = 0; l < D; ++l) a.first_cluster[l + 1] = a.first_cluster[l] + (N + a.nb[l] - 1) / a.nb[l];
  a.W0 = Wp; a.bias0 = bias_p; a.out0 = hs; a.c = c; a.flags = flags; a.status = status;
  CUtensorMap m[8];
  int rc;
  const uint64_t x_rows = static_cast<uint64_t>(L) * N, h_rows = static_cast<uint64_t>(D) * L * N;
  if ((rc = make_operand_map(&m[0], x, dtype, x_rows, H, 128))) return rc;
  if ((rc = make_operand_map(&m[1], hs, dtype, h_rows, H, 128))) return rc;
  if ((rc = make_operand_map(&m[2], x, dtype, x_rows, H, 64))) return rc;
  if ((rc = make_operand_map(&m[3], hs, dtype, h_rows, H, 64))) return rc;
  // output boxes: the slice's (or the last, short slice's) rows x the 32 units of a CTA, un-swizzled
  const int tail128 = N - ((N + 127) / 128 - 1) * 128, tail64 = N - ((N + 63) / 64 - 1) * 64;
  if ((rc = make_tmap_2d(&m[4], hs, dtype, h_rows, H, H, 128, 32, false))) return rc;
  if ((rc = make_tmap_2d(&m[5], hs, dtype, h_rows, H, H, 64, 32, false))) return rc;
  if ((rc = make_tmap_2d(&m[6], hs, dtype, h_rows, H, H, tail128, 32, false))) return rc;
  if ((rc = make_tmap_2d(&m[7], hs, dtype, h_rows, H, H, tail64, 32, false))) return rc;
  const size_t n_flags = static_cast<size_t>(D) * L * a.S * a.CL;
  if (cudaMemsetAsync(flags, 0, sizeof(int) * n_flags, stream) != cudaSuccess) return FTB_ERR_LAUNCH;
  const int grid = clusters * a.CL;
  if (dtype == FTB_F16) return launch_dilated<__half>(m, a, grid, smem, stream);
  return launch_dilated<__nv_bfloat16>(m, a, grid, smem, stream);
}

// --------------------------------------------------------------------- grid RNN
constexpr int kGridNB = 64;

bool grid_rnn_cluster_supported(int dtype, int D, int A, int B, int N, int H, int sm_count) {
  if (dtype != FTB_F16 && dtype != FTB_BF16) return false;
  if (H != 128 && H != 256) return false;  // 2 * H / 128 = 2 or 4 CTAs per cluster; 3H/64 K blocks fit TMEM
  if (D < 1 || A < 1 || B < 1 || N < 1) return false;
  const int S = (N + kGridNB - 1) / kGridNB;
  return D * A * S * (2 * H / 128) <= sm_count;
}

// X,Y: [A,B,N,H]; Wpx,Wpy: [D,H,3H]; hx,hy: [D,A,B,N,H]; flags: D*A*B*S*CL ints (zeroed here).
int launch_grid_rnn_cluster(int dtype, const void* X, const void* Y, const void* Wpx, const void* Wpy,
                            const float* bias_x, const float* bias_y, void* hx, void* hy, int D, int A, int B, int N,
                            int H, int* flags, int* status, cudaStream_t stream) {
  ClusterArgs a = {};
  a.D = D; a.L = B; a.N = N; a.H = H; a.A = A;
  a.S = (N + kGridNB - 1) / kGridNB;
  a.CL = 2 * H / 128;
  a.max_dil = 1;
  a.W0 = Wpx; a.W1 = Wpy; a.bias0 = bias_x; a.bias1 = bias_y; a.out0 = hx; a.out1 = hy; a.flags = flags; a.status = status;
  CUtensorMap m[8];
  int rc;
  const uint64_t grid_rows = static_cast<uint64_t>(A) * B * N;
  if ((rc = make_operand_map(&m[0], X, dtype, grid_rows, H, kGridNB))) return rc;
  if ((rc = make_operand_map(&m[1], Y, dtype, grid_rows, H, kGridNB))) return rc;
  if ((rc = make_operand_map(&m[2], hx, dtype, grid_rows * D, H, kGridNB))) return rc;
  if ((rc = make_operand_map(&m[3], hy, dtype, grid_rows * D, H, kGridNB))) return rc;
  // output boxes: NB (or the last slice's) rows x the 128 units of a CTA, un-swizzled
  const int tail = N - (a.S - 1) * kGridNB;
  if ((rc = make_tmap_2d(&m[4], hx, dtype, grid_rows * D, H, H, kGridNB, 128, false))) return rc;
  if ((rc = make_tmap_2d(&m[5], hy, dtype, grid_rows * D, H, H, kGridNB, 128, false))) return rc;
  if ((rc = make_tmap_2d(&m[6], hx, dtype, grid_rows * D, H, H, tail, 128, false))) return rc;
  if ((rc = make_tmap_2d(&m[7], hy, dtype, grid_rows * D, H, H, tail, 128, false))) return rc;
  const size_t n_flags = static_cast<size_t>(D) * A * B * a.S * a.CL;
  if (cudaMemsetAsync(flags, 0, sizeof(int) * n_flags, stream) != cudaSuccess) return FTB_ERR_LAUNCH;
  const int grid = D * A * a.S * a.CL;
  const uint32_t smem = smem_for(true, H, kGridNB, 128, 128, 6);
  if (dtype == FTB_F16) return launch<__half, kGrid, kGridNB>(m, a, grid, smem, stream);
  return launch<__nv_bfloat16, kGrid, kGridNB>(m, a, grid, smem, stream);
}

}  // namespace ftb

#ifdef FTB_ACCT
extern "C" int ftb_debug_set_cluster_acct(unsigned long long* buf) {
  return cudaMemcpyToSymbol(ftb::g_cluster_acct, &buf, sizeof(buf)) == cudaSuccess ? 0 : 1;
}
#endif
#ifdef FTB_TRACE
extern "C" int ftb_debug_set_cluster_trace(unsigned long long* buf) {
  return cudaMemcpyToSymbol(ftb::g_cluster_trace, &buf, sizeof(buf)) == cudaSuccess ? 0 : 1;
}
#endif

