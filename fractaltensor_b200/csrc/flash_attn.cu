// Flash attention forward with online softmax for 16-bit inputs on sm_100a, head
// dimension 128: unmasked, and (second instantiation) masked to keys i-left..i+right
// of query i, which covers causal attention (no lower limit, right = 0) and one- and
// two-sided sliding windows.  A masked query tile only walks the key/value blocks its
// rows can see; the blocks the window's edges cross are masked element by element.
//
// Follows the recurrence of attn_func (examples/flash_attention/flash_attention.py:14-44):
// per key/value block, scores S = scale * q k^T, running row maximum m and row sum
// l, output rescaled when the maximum moves.  Two algebraic rearrangements that
// leave the result unchanged up to rounding: the division by l is done once at the
// end instead of per block, and the running maximum is only advanced when it
// moves by more than 2^8 (the stale maximum cancels in the final division), so
// the accumulator in TMEM is rarely touched.  The (m, l) merge itself is the one of
// the reference's online softmax (kaleido/core/device/kernels/online_softmax.h:15-112).
//
// One CTA handles 256 query rows of one (batch, head): two 128-row query tiles
// that ping-pong through the tensor pipe.
//   warp 0        TMA producer: Q tiles, ring of K and V tiles
//   warp 1        MMA issuer: S_t = Q_t K^T and O_t += P_t V, accumulators in TMEM
//   warps 2..9    softmax of query tile 0: two threads per query row, one per half
//                 of the 128 keys of a block (warps 2..5 keys 0..63, warps 6..9 keys 64..127)
//   warps 10..17  softmax of query tile 1, same split
// A row's chain per key/value block (S ready -> maximum -> exponentials -> P written) is
// serial and sits between two dependent MMAs, so its length, not the arithmetic, bounds
// the tensor pipe; splitting the row over two threads halves it.  The two threads of a
// row exchange their partial maximum through shared memory (one float each per block) and
// their partial row sums once at the end.
// P never touches shared memory: the softmax threads write it (16-bit pairs) with
// tcgen05.st over the TMEM columns of the S values they have just read, and the PV
// MMA takes its A operand from TMEM.  V is consumed MN-major straight from its
// row-major tile.  Per query tile the tensor pipe sees S(j), [softmax], PV(j),
// S(j+1), ...; the two query tiles are offset so that one is in its softmax while
// the other one's MMAs run.
#include "../../include/ftb200.h"
#include "ptx.cuh"
#include "tmap.h"

namespace ftb {
namespace {

constexpr int kHalfBytes = 128 * 128;  // 128 rows x 64 16-bit columns
constexpr int kTileBytes = 2 * kHalfBytes;
constexpr int kKVSlots = 5;
constexpr int kThreads = 64 + 512;
constexpr float kRescaleThreshold = 8.0f;
constexpr int kCausalGroup = 16;   // (batch, head) entries whose CTAs are ordered longest first together

// Shared memory, all dynamic so that the 1024-byte alignment of the swizzled tiles costs
// no more than the bytes actually skipped: tiles, then the small control block.
struct Control {
  float xchg[2][2][128];  // [query tile][key half][row]: partial row maximum / row sum
  uint64_t q_full;
  uint64_t kv_full[kKVSlots], kv_empty[kKVSlots];
  uint64_t s_full[2], p_full[2], pv_done[2], o_staged[2];
  uint64_t pair_bar[2][4];  // [query tile][TMEM lane quadrant]: the two warps that share 32 rows
  uint32_t tmem_base;
  int abort;
};
constexpr uint32_t kTilesBytes = (2 + kKVSlots) * kTileBytes;  // Q0, Q1 (reused as output staging), KV ring
constexpr uint32_t kSmemBytes = 232448;                        // everything an SM offers one CTA
static_assert(kTilesBytes + sizeof(Control) + 512 <= kSmemBytes, "shared memory budget");

__device__ __forceinline__ void tmem_ld32p(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// 16-byte chunk `chunk16` (0..15) of row `row` in a 128x128 16-bit tile stored as
// two 64-column halves of 128-byte swizzled rows.
__device__ __forceinline__ uint8_t* sw128_chunk_ptr(uint8_t* tile, int row, int chunk16) {
  return tile + (chunk16 >> 3) * kHalfBytes + row * 128 + (((chunk16 & 7) ^ (row & 7)) << 4);
}

#ifdef FTB_TRACE
__device__ unsigned long long g_fa_trace[2][32][8];
#define FA_STAMP(tt, jj, k) if (blockIdx.x == 300 && lane == 0 && q == 0 && h == 0) g_fa_trace[tt][jj][k] = clock64()
#define FA_STAMP_MMA(tt, jj, k) if (blockIdx.x == 300) g_fa_trace[tt][jj][k] = clock64()
#else
#define FA_STAMP(tt, jj, k)
#define FA_STAMP_MMA(tt, jj, k)
#endif

template <typename T, bool kMasked>
__global__ void __launch_bounds__(kThreads, 1)
flash_attn_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                  const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO, int S,
                  int n_bh, int group, int left, int right, float scale_log2, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];

  if (*reinterpret_cast<volatile int*>(status) != 0) return;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  if (pad + kTilesBytes + sizeof(Control) > kSmemBytes) {
    // The dynamic segment starts later than this layout allows for: report, do not run.
    if (threadIdx.x == 0) atomicCAS(status, 0, FTB_ERR_ALIGN);
    return;
  }
  uint8_t* smem = smem_raw + pad;
  uint8_t* sQ = smem;                      // 2 tiles
  uint8_t* sKV = sQ + 2 * kTileBytes;      // ring
  Control& ctl = *reinterpret_cast<Control*>(smem + kTilesBytes);
  volatile int* s_abort = &ctl.abort;

  const int pairs = S / 256;
  int bh = blockIdx.x / pairs;
  int qpair = blockIdx.x - bh * pairs;
  if (kMasked) {
    // A pair's run length grows with its position, so CTAs are handed out longest first: within
    // a group of `group` (batch, head) entries all last pairs, then all pairs before them, ...
    // The grid's last CTAs are then the shortest, and the group bounds the K/V set in flight.
    const int per_group = group * pairs;
    const int g = blockIdx.x / per_group;
    const int r = blockIdx.x - g * per_group;
    const int gsize = min(group, n_bh - g * group);
    qpair = pairs - 1 - r / gsize;
    bh = g * group + r % gsize;
  }
  const int row_base = bh * S;            // first row of this (batch, head) in the flattened [B*heads*S, d] view
  const int q_row0 = row_base + qpair * 256;
  // Key/value blocks this CTA walks.  Masked: query i sees keys i-left .. i+right (left < 0: no
  // lower limit; causal attention is left < 0, right = 0).  A query tile walks from the block of the
  // first key its first row sees to the block of the last key its last row sees.  The CTA walks the
  // union, blocks [blk0, blk0 + n_kv); tile 0 takes part in iterations 0..last0 of that walk, tile 1
  // in first1..n_kv-1 (tile 1 starts and ends at most one block after tile 0).
  int blk0 = 0, n_kv = S / 128, first1 = 0, last0 = n_kv - 1;
  if (kMasked) {
    const int r0 = qpair * 256;
    const int lo0 = left >= 0 ? max(0, r0 - left) >> 7 : 0;
    const int lo1 = left >= 0 ? max(0, r0 + 128 - left) >> 7 : 0;
    const int hi0 = min(S / 128 - 1, (r0 + 127 + right) >> 7);
    const int hi1 = min(S / 128 - 1, (r0 + 255 + right) >> 7);
    blk0 = lo0;
    n_kv = hi1 - lo0 + 1;
    first1 = lo1 - lo0;
    last0 = hi0 - lo0;
  }

  if (threadIdx.x == 0) {
    prefetch_tmap(&mapQ);
    prefetch_tmap(&mapK);
    prefetch_tmap(&mapV);
    prefetch_tmap(&mapO);
    mbar_init(&ctl.q_full, 1);
    for (int i = 0; i < kKVSlots; ++i) {
      mbar_init(&ctl.kv_full[i], 1);
      mbar_init(&ctl.kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl.s_full[i], 1);
      mbar_init(&ctl.p_full[i], 8);
      mbar_init(&ctl.pv_done[i], 1);
      mbar_init(&ctl.o_staged[i], 8);
      for (int k = 0; k < 4; ++k) mbar_init(&ctl.pair_bar[i][k], 2);
    }
    ctl.abort = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  // K0, V0, K1, V1, ... stream: tile n into ring slot n % kKVSlots.
  auto load_kv = [&](int n) {
    const int slot = n % kKVSlots;
    uint8_t* dst = sKV + slot * kTileBytes;
    const CUtensorMap* m = (n & 1) ? &mapV : &mapK;
    const int r = row_base + (blk0 + (n >> 1)) * 128;
    mbar_arrive_expect_tx(&ctl.kv_full[slot], kTileBytes);
    tma_load_2d(dst, m, &ctl.kv_full[slot], 0, r);
    tma_load_2d(dst + kHalfBytes, m, &ctl.kv_full[slot], 64, r);
  };
  const int n_pre = min(kKVSlots, 2 * n_kv);
  if (threadIdx.x == 0) {
    // Q and the first pass over the (empty) ring are on their way while TMEM is allocated.
    mbar_arrive_expect_tx(&ctl.q_full, 2 * kTileBytes);
    for (int t = 0; t < 2; ++t) {
      tma_load_2d(sQ + t * kTileBytes, &mapQ, &ctl.q_full, 0, q_row0 + t * 128);
      tma_load_2d(sQ + t * kTileBytes + kHalfBytes, &mapQ, &ctl.q_full, 64, q_row0 + t * 128);
    }
    for (int n = 0; n < n_pre; ++n) load_kv(n);
  }
  if (warp == 1) {
    tmem_alloc(&ctl.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl.tmem_base;
  // TMEM columns: S0 [0,128), S1 [128,256), O0 [256,384), O1 [384,512).  P_t (16-bit pairs)
  // overlays S_t: keys 0..63 in columns [0,32), keys 64..127 in columns [64,96), i.e. each
  // half of the row over the S columns its own thread has read.

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int slot = 0;
      uint32_t phase = 1;  // the first pass was issued above
      for (int n = n_pre; n < 2 * n_kv; ++n) {
        if (!mbar_wait(&ctl.kv_empty[slot], phase ^ 1u, s_abort, status, FTB_ERR_TIMEOUT_SLOT)) break;
        load_kv(n);
        if (++slot == kKVSlots) {
          slot = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(128, 128, Fmt<T>::kind, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_f16(128, 128, Fmt<T>::kind, 0, 1);  // V is MN-major
      // This thread's own instructions sit between every softmax hand-off and the MMAs that follow it:
      // operand descriptors are base descriptors plus byte offsets / 16 (nothing is rebuilt per MMA),
      // and the K/V slots' phases are bits of one register.
      const uint64_t dQ = make_sdesc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t dK = make_sdesc_sw128(smem_u32(sKV), 16, 1024);
      const uint64_t dV = make_sdesc_sw128(smem_u32(sKV), kHalfBytes, 1024);
      uint32_t full_bits = 0;  // bit s: parity of the next fill of slot s
      bool ok = mbar_wait(&ctl.q_full, 0, s_abort, status, FTB_ERR_TIMEOUT_TMA);

      // (No tcgen05 fence after these waits: TMA completes the barriers, and the fence would drain the
      // tensor pipe.)
      auto wait_slot = [&](int n) -> bool {  // n-th tile of the K0, V0, K1, V1, ... stream
        const int slot = n % kKVSlots;
        if (!mbar_wait(&ctl.kv_full[slot], (full_bits >> slot) & 1u, s_abort, status, FTB_ERR_TIMEOUT_TMA)) return false;
        full_bits ^= 1u << slot;
        return true;
      };
      // S_t(j) = Q_t . K_j^T
      auto issue_s = [&](int t, int j) {
        const uint64_t dq = dQ + static_cast<uint64_t>((t * kTileBytes) >> 4);
        const uint64_t dk = dK + static_cast<uint64_t>((((2 * j) % kKVSlots) * kTileBytes) >> 4);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
          umma_ss(tmem_base + t * 128, dq + off, dk + off, idesc_qk, k != 0 ? 1u : 0u);
        }
        umma_commit(&ctl.s_full[t]);
      };
      // O_t += P_t(j) . V_j: A = P_t from TMEM (16 keys = 8 packed columns per step; the two
      // key halves start 64 columns apart); B = V, MN-major: 16 keys = two 8-row groups
      // (1024 B apart), the two 64-column halves of d are 16 KB apart.
      auto issue_pv = [&](int t, int j, bool first) {
        const uint64_t dv = dV + static_cast<uint64_t>((((2 * j + 1) % kKVSlots) * kTileBytes) >> 4);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + (k >> 2) * 64 + (k & 3) * 8, dv + k * (2048 >> 4),
                  idesc_pv, (!first || k != 0) ? 1u : 0u);
        umma_commit(&ctl.pv_done[t]);
      };

      if (ok) ok = wait_slot(0);
      if (ok) {
        issue_s(0, 0);
        if (first1 == 0) issue_s(1, 0);
        umma_commit(&ctl.kv_empty[0]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const bool more = j + 1 < n_kv;
        if (!wait_slot(2 * j + 1)) break;            // V_j
        if (more && !wait_slot(2 * j + 2)) break;    // K_{j+1}
        for (int t = 0; t < 2 && ok; ++t) {
          const int first = t == 0 ? 0 : first1;
          const int last = t == 0 ? last0 : n_kv - 1;
          if (j >= first && j <= last) {
            // P_t(j) is in TMEM (and the softmax is done with S_t(j)).
            if (!mbar_wait(&ctl.p_full[t], (j - first) & 1, s_abort, status, FTB_ERR_TIMEOUT_EPI)) {
              ok = false;
              break;
            }
            tc_fence_after();
            FA_STAMP_MMA(t, j, 5);
            issue_pv(t, j, j == first);
          }
          // The tensor pipe runs MMAs in issue order: S_t(j+1) overwrites S_t / P_t only after
          // PV_t(j) has read P_t.
          if (more && j + 1 >= first && j + 1 <= last) issue_s(t, j + 1);
          FA_STAMP_MMA(t, j, 6);
        }
        if (!ok) break;
        umma_commit(&ctl.kv_empty[(2 * j + 1) % kKVSlots]);
        if (more) umma_commit(&ctl.kv_empty[(2 * j + 2) % kKVSlots]);
      }
    }
  } else {
    // ----------------------------------- softmax: query tile t, key half h, lane quadrant q
    const int t = (warp - 2) >> 3;
    const int h = ((warp - 2) >> 2) & 1;
    const int q = warp & 3;  // TMEM lane quadrant of this warp
    const int row = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t s_addr = lane_addr + t * 128 + h * 64;        // this thread's 64 scores; P over the first 32
    const uint32_t o_addr = lane_addr + 256 + t * 128 + h * 64;  // its 64 output columns (rescale, final pass)
    uint8_t* my_stage = sQ + t * kTileBytes;  // output staging: Q_t is dead once the last S MMA is done
    float* my_x = &ctl.xchg[t][h][row];
    const float* peer_x = &ctl.xchg[t][h ^ 1][row];
    uint64_t* pair = &ctl.pair_bar[t][q];
    float m_used = 0.f, l = 0.f;
    bool ok = true;
    const int j_first = t == 0 ? 0 : first1;
    const int j_last = t == 0 ? last0 : n_kv - 1;
    const int n_mine = j_last - j_first + 1;

    for (int j = j_first; j <= j_last && ok; ++j) {
      const int it = j - j_first;  // this tile's block count so far: the phase of its barriers
      if (!__all_sync(0xffffffffu, mbar_wait(&ctl.s_full[t], it & 1, s_abort, status, FTB_ERR_TIMEOUT_MMA))) {
        ok = false;
        break;
      }
      tc_fence_after();
      FA_STAMP(t, j, 0);
      uint32_t s[64];
      tmem_ld32p(s_addr + 0, s + 0);
      tmem_ld32p(s_addr + 32, s + 32);
      tmem_ld_wait();
      FA_STAMP(t, j, 1);
      if (kMasked) {
        // This thread's 64 keys start at key0; its query is `mine`.  Columns below lo_col are before
        // the window, columns above hi_col after it (for causal attention: after the query).
        const int key0 = (blk0 + j) * 128 + h * 64;
        const int mine = qpair * 256 + t * 128 + row;
        const int lo_col = left >= 0 ? mine - left - key0 : 0;
        const int hi_col = mine + right - key0;
        if (__any_sync(0xffffffffu, lo_col > 0)) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (i < lo_col) s[i] = 0xff800000u;  // -inf
        }
        if (__any_sync(0xffffffffu, hi_col < 63)) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (i > hi_col) s[i] = 0xff800000u;
        }
      }

      // Maximum of this half of the row: eight independent chains of three-input maxima.
      float mx8[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx8[i] = fmaxf(__uint_as_float(s[i]), __uint_as_float(s[8 + i]));
#pragma unroll
      for (int i = 16; i < 64; i += 16) {
#pragma unroll
        for (int k = 0; k < 8; ++k) mx8[k] = fmax3(mx8[k], __uint_as_float(s[i + k]), __uint_as_float(s[i + 8 + k]));
      }
      float mx = fmaxf(fmax3(mx8[0], mx8[1], mx8[2]), fmaxf(fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
      // Row maximum = the larger of the two halves.  The slot written here was last read by the
      // other thread before its arrival on p_full of the previous block, which the MMA warp waited
      // for before it issued the S this block started from: no second buffer is needed.
      *my_x = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(pair);
      if (!__all_sync(0xffffffffu, mbar_wait(pair, it & 1, s_abort, status, FTB_ERR_TIMEOUT_EPI))) {
        ok = false;
        break;
      }
      mx = fmaxf(mx, *peer_x);
      // A row can have no visible key in a block of its tile's walk: the floor keeps 2^(s - m) at 0
      // there instead of inf - inf, and the first real maximum rescales the (zero) accumulator by 0.
      const float m_new = kMasked ? fmaxf(mx * scale_log2, -1e30f) : mx * scale_log2;
      if (it == 0) {
        m_used = m_new;
      } else {
        // Both threads of a row see the same m_new and m_used, so both take the same branch.
        const bool need = (m_new - m_used) > kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // O_t must be at rest: the PV MMA of the previous block has to be done.
          if (!__all_sync(0xffffffffu,
                          mbar_wait(&ctl.pv_done[t], (it - 1) & 1, s_abort, status, FTB_ERR_TIMEOUT_MMA))) {
            ok = false;
            break;
          }
          tc_fence_after();
          const float alpha = need ? exp2_fast(m_used - m_new) : 1.f;
          if (need) m_used = m_new;
          l *= alpha;
#pragma unroll 1
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t o[16];
            tmem_ld16(o_addr + ch * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st16(o_addr + ch * 16, o);
          }
          tmem_st_wait();
        }
      }

      FA_STAMP(t, j, 2);
      // P_t(j) = 2^(scale*S - m) as 16-bit pairs over the first 32 of this thread's 64 S columns
      // (they are in registers now; the MMA that overwrites them next, S_t(j+1), is issued after
      // PV_t(j)); partial row sum for l.  (Packed fp16 exponentials, two per MUFU op, and a cubic
      // 2^x on the FMA pipes for every other element were both measured and are no faster.)
      {
        float sum8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const float p0 = exp2_fast(fmaf(__uint_as_float(s[32 * part + 2 * c]), scale_log2, -m_used));
            const float p1 = exp2_fast(fmaf(__uint_as_float(s[32 * part + 2 * c + 1]), scale_log2, -m_used));
            sum8[(2 * c) & 7] += p0;
            sum8[(2 * c + 1) & 7] += p1;
            pk[c] = Fmt<T>::pack2(p0, p1);
          }
          tmem_st16(s_addr + 16 * part, pk);
        }
        l += ((sum8[0] + sum8[1]) + (sum8[2] + sum8[3])) + ((sum8[4] + sum8[5]) + (sum8[6] + sum8[7]));
        FA_STAMP(t, j, 4);
        tmem_st_wait();
      }
      FA_STAMP(t, j, 3);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.p_full[t]);
    }

    // Row sum = the two halves' sums (same exchange, one more phase of the pair barrier).
    if (ok) {
      *my_x = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(pair);
      ok = __all_sync(0xffffffffu, mbar_wait(pair, n_mine & 1, s_abort, status, FTB_ERR_TIMEOUT_EPI));
      if (ok) l += *peer_x;
    }
    // Final: O_t / l -> 16-bit -> staging (the Q tile, dead once the last PV is done) -> TMA store.
    if (ok && __all_sync(0xffffffffu,
                         mbar_wait(&ctl.pv_done[t], (n_mine - 1) & 1, s_abort, status, FTB_ERR_TIMEOUT_MMA))) {
      tc_fence_after();
      const float inv_l = 1.f / l;
#pragma unroll 1
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t o[32];
        tmem_ld32(o_addr + ch * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 u;
          u.x = Fmt<T>::pack2(__uint_as_float(o[8 * c + 0]) * inv_l, __uint_as_float(o[8 * c + 1]) * inv_l);
          u.y = Fmt<T>::pack2(__uint_as_float(o[8 * c + 2]) * inv_l, __uint_as_float(o[8 * c + 3]) * inv_l);
          u.z = Fmt<T>::pack2(__uint_as_float(o[8 * c + 4]) * inv_l, __uint_as_float(o[8 * c + 5]) * inv_l);
          u.w = Fmt<T>::pack2(__uint_as_float(o[8 * c + 6]) * inv_l, __uint_as_float(o[8 * c + 7]) * inv_l);
          *reinterpret_cast<uint4*>(sw128_chunk_ptr(my_stage, row, (h * 2 + ch) * 4 + c)) = u;
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.o_staged[t]);
      // One thread per query tile stores it once all eight warps have staged their part.
      if (lane == 0 && h == 0 && q == 2 &&
          mbar_wait(&ctl.o_staged[t], 0, s_abort, status, FTB_ERR_TIMEOUT_EPI)) {
        tma_store_2d(&mapO, my_stage, 0, q_row0 + t * 128);
        tma_store_2d(&mapO, my_stage + kHalfBytes, 64, q_row0 + t * 128);
        tma_store_commit();
        tma_store_wait_read<0>();  // the staging tile has been read; the writes land before the grid ends
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (ctl.abort) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T, bool kMasked>
int launch(const CUtensorMap& mQ, const CUtensorMap& mK, const CUtensorMap& mV, const CUtensorMap& mO, int n_bh,
           int S, int left, int right, float scale_log2, int* status, cudaStream_t stream) {
  static std::atomic<unsigned long long> configured{0};
  auto kfn = flash_attn_kernel<T, kMasked>;
  if (!ensure_dynamic_smem(kfn, kSmemBytes, configured)) return FTB_ERR_LAUNCH;
  const int group = kCausalGroup;
  kfn<<<n_bh * (S / 256), kThreads, kSmemBytes, stream>>>(mQ, mK, mV, mO, S, n_bh, group, left, right, scale_log2, status);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
}

}  // namespace
}  // namespace ftb

using namespace ftb;

#ifdef FTB_TRACE
extern "C" int ftb_debug_fa_trace(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, g_fa_trace, sizeof(unsigned long long) * 2 * 32 * 8) == cudaSuccess ? 0 : 1;
}
#endif

namespace {
int flash_attn_entry(const void* q, const void* k, const void* v, void* o, int B, int heads, int S, int d,
                     float scale, int dtype, bool masked, int left, int right, void* workspace,
                     size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!q || !k || !v || !o || B <= 0 || heads <= 0 || S <= 0) return FTB_ERR_ARG;
  if (dtype != FTB_F16 && dtype != FTB_BF16) return FTB_ERR_ARG;
  if (d != 128 || S % 256 != 0) return FTB_ERR_ARG;
  if (masked && !(scale > 0.f)) return FTB_ERR_ARG;  // masked scores are -inf times the scale
  if (masked && right < 0) return FTB_ERR_ARG;
  if (left >= S) left = -1;  // every earlier key is inside the window
  if (right > S) right = S;
  const int64_t rows = static_cast<int64_t>(B) * heads * S;
  if (rows > 0x7fffffffLL) return FTB_ERR_ARG;
  if (workspace == nullptr || workspace_bytes < ftb_workspace_bytes()) return FTB_ERR_WORKSPACE;
  int rc = check_device_sm100();
  if (rc) return rc;
  // The status word is sticky: the caller zeroes the workspace once; after a device wait ran out
  // every later call on that workspace is a no-op until the caller clears the word.
  int* status = static_cast<int*>(workspace);

  CUtensorMap mQ, mK, mV, mO;
  if ((rc = make_tmap_2d(&mQ, q, dtype, rows, d, d, 128, 64))) return rc;
  if ((rc = make_tmap_2d(&mK, k, dtype, rows, d, d, 128, 64))) return rc;
  if ((rc = make_tmap_2d(&mV, v, dtype, rows, d, d, 128, 64))) return rc;
  if ((rc = make_tmap_2d(&mO, o, dtype, rows, d, d, 128, 64))) return rc;
  const int units = B * heads;
  const float scale_log2 = scale * 1.4426950408889634f;
  if (masked) {
    if (dtype == FTB_F16)
      return launch<__half, true>(mQ, mK, mV, mO, units, S, left, right, scale_log2, status, stream);
    return launch<__nv_bfloat16, true>(mQ, mK, mV, mO, units, S, left, right, scale_log2, status, stream);
  }
  if (dtype == FTB_F16) return launch<__half, false>(mQ, mK, mV, mO, units, S, -1, 0, scale_log2, status, stream);
  return launch<__nv_bfloat16, false>(mQ, mK, mV, mO, units, S, -1, 0, scale_log2, status, stream);
}
}  // namespace

extern "C" int ftb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, int B, int heads, int S,
                                  int d, float scale, int dtype, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  return flash_attn_entry(q, k, v, o, B, heads, S, d, scale, dtype, false, -1, 0, workspace, workspace_bytes, stream);
}

extern "C" int ftb_flash_attn_causal_fwd(const void* q, const void* k, const void* v, void* o, int B, int heads,
                                         int S, int d, float scale, int dtype, void* workspace,
                                         size_t workspace_bytes, void* stream) {
  return flash_attn_entry(q, k, v, o, B, heads, S, d, scale, dtype, true, -1, 0, workspace, workspace_bytes, stream);
}

extern "C" int ftb_flash_attn_window_fwd(const void* q, const void* k, const void* v, void* o, int B, int heads,
                                         int S, int d, int window, float scale, int dtype, void* workspace,
                                         size_t workspace_bytes, void* stream) {
  if (window <= 0) return FTB_ERR_ARG;
  return flash_attn_entry(q, k, v, o, B, heads, S, d, scale, dtype, true, window - 1, 0, workspace,
                          workspace_bytes, stream);
}

extern "C" int ftb_flash_attn_local_fwd(const void* q, const void* k, const void* v, void* o, int B, int heads,
                                        int S, int d, int left, int right, float scale, int dtype,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  if (left < 0 || right < 0) return FTB_ERR_ARG;
  return flash_attn_entry(q, k, v, o, B, heads, S, d, scale, dtype, true, left, right, workspace, workspace_bytes,
                          stream);
}
