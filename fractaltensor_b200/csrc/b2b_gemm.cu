// Back-to-back GEMM  D = (A . B) . C  for 16-bit inputs on sm_100a.
//
// Arithmetic follows KeBack2BackGemm (kaleido/core/device/kernels/cutlass_wmma.h:489-533):
// S = A.B accumulated in fp32, rounded to the 16-bit input type, D = S.C
// accumulated in fp32, rounded to the 16-bit type.  Unlike the reference, which
// re-reads the A tile for every N tile, every byte of A is read once: the shape
// is HBM-bound, so the kernel is organised around keeping TMA loads of A and TMA
// stores of D in flight while small MMAs and two conversions run per tile.
//
// Shapes: M % 128 == 0, K and P in {64, 128}, N in {128, 256, 512} (the reference's benchmark
// runs K = P = 64 with N = 256 and 512, benchmarks/fused_two_hgemms/fractaltensor/
// fused_two_hgemms.cu:152-174; the headline configuration is K = N = P = 128).
//
// One persistent CTA per SM owns a contiguous range of 128-row tiles.  N is walked in chunks of
// 128 columns: a "unit" is (tile, chunk), S of a unit is 128 x 128.
//   warp 0      TMA producer: B and C of the batch entry, ring of A tiles
//   warp 1      MMA issuer: S = A.B_chunk^T into TMEM, then O (+)= P.C_chunk^T into TMEM
//   warps 2..5  convert S -> P (16-bit pairs written with tcgen05.st over the TMEM columns
//               of the S tile just read; the second MMA takes its A operand from TMEM),
//               convert O -> D staging after the tile's last chunk, TMA store of D
// P never touches shared memory.  B and C of the next batch entry are prefetched into a second
// buffer pair when two pairs fit, so a CTA whose range crosses a batch boundary does not drain.
#include "../../include/ftb200.h"
#include "ptx.cuh"
#include "tmap.h"

namespace ftb {
namespace {

constexpr int kTile = 128;       // rows per tile; also the N chunk
constexpr int kSlabBytes = 128;  // one row of a 64-column, 128-byte-swizzled slab
constexpr int kAStages = 2;      // A tiles in flight per SM (2, 3 and 4 measured the same)
constexpr int kThreads = 192;
constexpr uint32_t kSmemBudget = 7 * 32768;  // tiles + buffers; the control block is static

struct Shape {
  int N, K, P;            // inner sizes
  int nchunks;            // N / 128
  int bc_pairs;           // 1 or 2 (B, C) buffer pairs
  uint32_t a_bytes;       // one A tile: 128 x K
  uint32_t b_bytes;       // B of a batch entry: N x K
  uint32_t c_bytes;       // C of a batch entry: P x N
  uint32_t d_bytes;       // one D tile: 128 x P
  int tiles_per_batch;
  int total_tiles;
};

// Writes 32 fp32 accumulator columns [col0, col0+32) of row `row` as 16-bit values into a tile
// of 128 rows laid out as 64-column slabs of 128-byte swizzled rows (16 KB per slab).
template <typename T>
__device__ __forceinline__ void write_row_chunk_sw128(uint8_t* tile, int row, int col0, const uint32_t (&r)[32]) {
  uint8_t* slab_row = tile + (col0 >> 6) * (kTile * kSlabBytes) + row * kSlabBytes;
  const int c0 = (col0 & 63) >> 3;  // first 16-byte chunk inside the 128-byte row
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 u;
    u.x = Fmt<T>::pack2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
    u.y = Fmt<T>::pack2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
    u.z = Fmt<T>::pack2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
    u.w = Fmt<T>::pack2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
    const int chunk = (c0 + j) ^ (row & 7);
    *reinterpret_cast<uint4*>(slab_row + chunk * 16) = u;
  }
}

#ifdef FTB_TRACE
__device__ unsigned long long g_b2b_wall[148][4];
#define B2B_WALL(k) if (blockIdx.x < 148) g_b2b_wall[blockIdx.x][k] = globaltimer_ns()
#else
#define B2B_WALL(k)
#endif

template <typename T, int KK, int PP, int NCH>
__global__ void __launch_bounds__(kThreads, 1)
b2b_gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CUtensorMap mapD,
                const Shape sh, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t a_full[kAStages], a_empty[kAStages];
  __shared__ uint64_t bc_full[2], bc_empty[2];
  __shared__ uint64_t s_full[2], p_full[2], o_full[2], o_empty[2];
  __shared__ uint64_t d_free, d_ready;  // staging tile handshakes between the epilogue warps and the storing thread
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

  if (threadIdx.x == 0) B2B_WALL(0);
  // The call behind this one may be scheduled as SMs free up; it touches no global memory
  // before its own grid_dependency_wait().
  grid_launch_dependents();

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // Layout: bc_pairs x (B, C), then the A ring, then the D staging tile.
  const uint32_t bc_pair_bytes = sh.b_bytes + sh.c_bytes;
  uint8_t* sBC = smem;
  uint8_t* sA = sBC + sh.bc_pairs * bc_pair_bytes;
  uint8_t* sD = sA + kAStages * sh.a_bytes;
  constexpr int nchunks = NCH;
  constexpr int k_halves = KK / 64, p_halves = PP / 64;

  if (threadIdx.x == 0) {
    prefetch_tmap(&mapA);
    prefetch_tmap(&mapB);
    prefetch_tmap(&mapC);
    prefetch_tmap(&mapD);
    for (int i = 0; i < kAStages; ++i) {
      mbar_init(&a_full[i], 1);
      mbar_init(&a_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bc_full[i], 1);
      mbar_init(&bc_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&o_full[i], 1);
      mbar_init(&o_empty[i], 4);
    }
    mbar_init(&d_free, 1);
    mbar_init(&d_ready, 4);
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
  // Set-up is done; from here on the kernel reads and writes global memory, so the call before it
  // in the stream must have finished.  A non-zero status word (sticky) turns the call into a no-op.
  grid_dependency_wait();
  const bool live = *reinterpret_cast<volatile int*>(status) == 0;
  // Contiguous tile range of this CTA.
  const int per = live ? sh.total_tiles / gridDim.x : 0, rem = live ? sh.total_tiles % gridDim.x : 0;
  const int first = blockIdx.x * per + (blockIdx.x < rem ? blockIdx.x : rem);
  const int count = per + (blockIdx.x < rem ? 1 : 0);
  const int units = count * nchunks;
  const int batch0 = count > 0 ? first / sh.tiles_per_batch : 0;
  const int batch_last = count > 0 ? (first + count - 1) / sh.tiles_per_batch : -1;

  // TMEM columns: S0 [0,128), S1 [128,256), O0 [256,256+P), O1 [384,384+P); P_u (16-bit pairs)
  // overlays the first 64 columns of S_u.

  // Batch entry n (counted from this CTA's first) lives in buffer pair n % bc_pairs, on its
  // use number n / bc_pairs.
  auto bc_pair = [&](int n) { return sh.bc_pairs == 2 ? (n & 1) : 0; };
  auto bc_use = [&](int n) { return sh.bc_pairs == 2 ? (n >> 1) : n; };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int next_bc = batch0;
      bool ok = true;
      auto load_bc = [&](int b) -> bool {
        const int n = b - batch0, pair = bc_pair(n);
        if (!mbar_wait(&bc_empty[pair], (bc_use(n) & 1) ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_SLOT)) return false;
        uint8_t* dB = sBC + pair * bc_pair_bytes;
        uint8_t* dC = dB + sh.b_bytes;
        mbar_arrive_expect_tx(&bc_full[pair], bc_pair_bytes);
        // B [N, K]: per 64-wide K slab, boxes of up to 256 rows.
        const int box_rows = sh.N < 256 ? sh.N : 256;
        for (int kh = 0; kh < k_halves; ++kh)
          for (int r0 = 0; r0 < sh.N; r0 += box_rows)
            tma_load_2d(dB + kh * (sh.N * kSlabBytes) + r0 * kSlabBytes, &mapB, &bc_full[pair], kh * 64, b * sh.N + r0);
        // C [P, N]: per 64-wide N slab, one box of P rows.
        for (int sl = 0; sl < sh.N / 64; ++sl)
          tma_load_2d(dC + sl * (PP * kSlabBytes), &mapC, &bc_full[pair], sl * 64, b * PP);
        return true;
      };
      for (int i = 0; i < count && ok; ++i) {
        const int tile = first + i;
        const int b = tile / sh.tiles_per_batch;
        while (ok && next_bc <= b) ok = load_bc(next_bc++);
        if (!ok) break;
        if (!mbar_wait(&a_empty[stage], phase ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_SLOT)) break;
        uint8_t* dst = sA + stage * sh.a_bytes;
        mbar_arrive_expect_tx(&a_full[stage], sh.a_bytes);
        for (int kh = 0; kh < k_halves; ++kh)
          tma_load_2d(dst + kh * (kTile * kSlabBytes), &mapA, &a_full[stage], kh * 64, tile * kTile);
        if (++stage == kAStages) {
          stage = 0;
          phase ^= 1u;
        }
        // Prefetch the next batch entry's B, C into the other buffer pair.  Only after this
        // tile's A is on its way: the pair frees up when the MMAs of the batch entry before this
        // one are done, and the MMA warp issues this tile's first product ahead of the previous
        // tile's last.
        if (sh.bc_pairs == 2)
          while (ok && next_bc <= batch_last && next_bc <= b + 1) ok = load_bc(next_bc++);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc1 = make_idesc_f16(128, 128, Fmt<T>::kind, 0, 0);
      constexpr uint32_t idesc2 = make_idesc_f16(128, PP, Fmt<T>::kind, 0, 0);
      const uint32_t aBC = smem_u32(sBC);
      int stage = 0;
      uint32_t a_phase = 0;
      int cur_batch = -1;
      bool ok = true;

      // First product of unit u = (tile i, chunk c): S[u&1] = A_i . B_c^T.  The buffer last held
      // S/P of unit u-2, whose second product was issued before this one and so runs before it on
      // the tensor pipe.
      auto gemm1 = [&](int u) -> bool {
        const int i = u / nchunks, c = u - i * nchunks;
        const int b = (first + i) / sh.tiles_per_batch;
        const int n = b - batch0;
        if (b != cur_batch) {
          if (!mbar_wait(&bc_full[bc_pair(n)], bc_use(n) & 1, &s_abort, status, FTB_ERR_TIMEOUT_TMA)) return false;
          cur_batch = b;
        }
        if (c == 0 && !mbar_wait(&a_full[stage], a_phase, &s_abort, status, FTB_ERR_TIMEOUT_TMA)) return false;
        // (No tcgen05 fence: TMA completes both barriers, and the accumulator's previous contents were
        // consumed by an MMA this thread issued earlier.)
        if (u == 0) B2B_WALL(1);
        const uint64_t dA = make_sdesc_sw128(smem_u32(sA + stage * sh.a_bytes), 16, 1024);
        const uint64_t dB = make_sdesc_sw128(aBC + bc_pair(n) * bc_pair_bytes + c * (kTile * kSlabBytes), 16, 1024);
        const uint32_t slabB = (sh.N * kSlabBytes) >> 4;
#pragma unroll
        for (int k = 0; k < KK / 16; ++k) {
          const uint32_t offA = ((k >> 2) * (kTile * kSlabBytes) + (k & 3) * 32) >> 4;
          const uint32_t offB = (k >> 2) * slabB + (k & 3) * 2;
          umma_ss(tmem_base + (u & 1) * 128, dA + offA, dB + offB, idesc1, k != 0 ? 1u : 0u);
        }
        if (c == nchunks - 1) {
          umma_commit(&a_empty[stage]);
          if (++stage == kAStages) {
            stage = 0;
            a_phase ^= 1u;
          }
        }
        umma_commit(&s_full[u & 1]);
        return true;
      };
      // Second product of unit u: O[i&1] (+)= P_u . C_c^T, P from TMEM (16 of the chunk's 128
      // inner positions = 8 packed columns per step).
      auto gemm2 = [&](int u, bool last_of_batch) -> bool {
        const int i = u / nchunks, c = u - i * nchunks;
        const int ob = i & 1;
        const int n = (first + i) / sh.tiles_per_batch - batch0;
        const uint32_t aC = aBC + bc_pair(n) * bc_pair_bytes + sh.b_bytes;
        if (c == 0 && !mbar_wait(&o_empty[ob], ((i >> 1) & 1) ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_EPI)) return false;
        // One barrier per S/P buffer: the converting warps can be a whole unit ahead of this wait
        // (S of the next unit is ready early), and a parity wait must not fall two phases behind.
        if (!mbar_wait(&p_full[u & 1], (u >> 1) & 1, &s_abort, status, FTB_ERR_TIMEOUT_EPI)) return false;
        tc_fence_after();
        const uint64_t dC = make_sdesc_sw128(aC + (2 * c) * (PP * kSlabBytes), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offC = ((kk >> 2) * (PP * kSlabBytes) + (kk & 3) * 32) >> 4;
          umma_ts(tmem_base + 256 + ob * 128, tmem_base + (u & 1) * 128 + kk * 8, dC + offC, idesc2,
                  (c | kk) != 0 ? 1u : 0u);
        }
        if (c == nchunks - 1) {
          umma_commit(&o_full[ob]);
          if (last_of_batch) umma_commit(&bc_empty[bc_pair(n)]);
        }
        return true;
      };

      if (units > 0) ok = gemm1(0);
      for (int u = 0; u < units && ok; ++u) {
        const int i = u / nchunks;
        const bool has_next = u + 1 < units;
        const bool tile_ends = (u + 1) % nchunks == 0;
        const bool next_new_batch =
            has_next && tile_ends && ((first + i + 1) / sh.tiles_per_batch != (first + i) / sh.tiles_per_batch);
        const bool last_of_batch = tile_ends && (next_new_batch || !has_next);
        // Run ahead with the next unit's first product, unless it needs a B that can only be
        // loaded once this batch entry's MMAs are done (a single buffer pair).
        const bool ahead = has_next && !(next_new_batch && sh.bc_pairs == 1);
        if (ahead) ok = gemm1(u + 1);
        if (ok) ok = gemm2(u, last_of_batch);
        if (ok && has_next && !ahead) ok = gemm1(u + 1);
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const bool issuer = (warp == 2 && lane == 0);
    uint32_t d_phase = 0;
    bool ok = true;

    auto convert_s = [&](int u) -> bool {
      const int sb = u & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[sb], (u >> 1) & 1, &s_abort, status, FTB_ERR_TIMEOUT_MMA)))
        return false;
      tc_fence_after();
      // 32 fp32 columns in, 16 columns of 16-bit pairs out, in place: the columns written at step
      // ch lie below the ones still to be read.
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t r[32];
        tmem_ld32(lane_addr + sb * 128 + ch * 32, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) pk[c] = Fmt<T>::pack2(__uint_as_float(r[2 * c]), __uint_as_float(r[2 * c + 1]));
        tmem_st16(lane_addr + sb * 128 + ch * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[sb]);
      return true;
    };
    auto output_o = [&](int i) -> bool {
      const int ob = i & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&o_full[ob], (i >> 1) & 1, &s_abort, status, FTB_ERR_TIMEOUT_MMA)))
        return false;
      tc_fence_after();
      // The previous TMA store must have finished reading the staging tile.
      if (issuer) {
        tma_store_wait_read<0>();
        mbar_arrive(&d_free);
      }
      if (!__all_sync(0xffffffffu, mbar_wait(&d_free, d_phase, &s_abort, status, FTB_ERR_TIMEOUT_EPI))) return false;
#pragma unroll 1
      for (int ch = 0; ch < PP / 32; ++ch) {
        uint32_t r[32];
        tmem_ld32(lane_addr + 256 + ob * 128 + ch * 32, r);
        tmem_ld_wait();
        write_row_chunk_sw128<T>(sD, row, ch * 32, r);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&o_empty[ob]);
        mbar_arrive(&d_ready);
      }
      const bool staged = !issuer || mbar_wait(&d_ready, d_phase, &s_abort, status, FTB_ERR_TIMEOUT_EPI);
      d_phase ^= 1u;
      if (issuer && staged) {
        const int tile = first + i;
        for (int ph = 0; ph < p_halves; ++ph) tma_store_2d(&mapD, sD + ph * (kTile * kSlabBytes), ph * 64, tile * kTile);
        tma_store_commit();
      }
      return true;
    };

    // After a tile's first unit is converted, the previous tile's result is on its way (or done):
    // put it out while the MMA warp works on this tile.
    for (int u = 0; u < units && ok; ++u) {
      ok = convert_s(u);
      if (ok && u % nchunks == 0 && u > 0) ok = output_o(u / nchunks - 1);
    }
    if (ok && count > 0) ok = output_o(count - 1);
    if (issuer) B2B_WALL(2);
    if (issuer) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (s_abort) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
    if (lane == 0) B2B_WALL(3);
  }
}

template <typename T, int KK, int PP, int NCH>
int launch(const CUtensorMap& mA, const CUtensorMap& mB, const CUtensorMap& mC, const CUtensorMap& mD, const Shape& sh,
           uint32_t smem_bytes, int* status, int sm_count, cudaStream_t stream) {
  static std::atomic<unsigned long long> configured{0};
  auto kfn = b2b_gemm_kernel<T, KK, PP, NCH>;
  if (!ensure_dynamic_smem(kfn, kSmemBudget + 1024, configured)) return FTB_ERR_LAUNCH;
  const int grid = sh.total_tiles < sm_count ? sh.total_tiles : sm_count;
  const cudaError_t err = launch_dependent(kfn, dim3(grid), dim3(kThreads), smem_bytes, stream, mA, mB, mC, mD, sh, status);
  count_launch();
  if (err != cudaSuccess) cudaGetLastError();
  return err == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
}

}  // namespace
}  // namespace ftb

using namespace ftb;

#ifdef FTB_TRACE
extern "C" int ftb_debug_b2b_wall(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, g_b2b_wall, sizeof(unsigned long long) * 148 * 4) == cudaSuccess ? 0 : 1;
}
#endif

extern "C" int ftb_b2b_gemm(const void* A, const void* B, const void* C, void* Dout, int batch, int M, int N, int K,
                            int P, int dtype, void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!A || !B || !C || !Dout || batch <= 0 || M <= 0) return FTB_ERR_ARG;
  if (dtype != FTB_F16 && dtype != FTB_BF16) return FTB_ERR_ARG;
  if (M % 128 != 0 || (N != 128 && N != 256 && N != 512) || (K != 64 && K != 128) || (P != 64 && P != 128))
    return FTB_ERR_ARG;
  if (static_cast<int64_t>(batch) * M > 0x7fffffffLL) return FTB_ERR_ARG;
  if (workspace == nullptr || workspace_bytes < ftb_workspace_bytes()) return FTB_ERR_WORKSPACE;

  Shape sh;
  sh.N = N;
  sh.K = K;
  sh.P = P;
  sh.nchunks = N / 128;
  sh.a_bytes = 128u * K * 2;
  sh.b_bytes = static_cast<uint32_t>(N) * K * 2;
  sh.c_bytes = static_cast<uint32_t>(P) * N * 2;
  sh.d_bytes = 128u * P * 2;
  sh.tiles_per_batch = M / 128;
  sh.total_tiles = batch * sh.tiles_per_batch;
  const uint32_t fixed = kAStages * sh.a_bytes + sh.d_bytes;
  const uint32_t pair = sh.b_bytes + sh.c_bytes;
  if (fixed + pair > kSmemBudget) return FTB_ERR_ARG;  // B and C of one batch entry must fit next to the ring
  sh.bc_pairs = (fixed + 2 * pair <= kSmemBudget) ? 2 : 1;
  const uint32_t smem_bytes = fixed + sh.bc_pairs * pair + 1024;

  int rc = check_device_sm100();
  if (rc) return rc;
  // The status word is sticky: the caller zeroes the workspace once; after a device wait ran out
  // every later call on that workspace is a no-op until the caller clears the word.
  int* status = static_cast<int*>(workspace);

  CUtensorMap mA, mB, mC, mD;
  const uint64_t rowsA = static_cast<uint64_t>(batch) * M;
  if ((rc = make_tmap_2d(&mA, A, dtype, rowsA, K, K, 128, 64))) return rc;
  if ((rc = make_tmap_2d(&mB, B, dtype, static_cast<uint64_t>(batch) * N, K, K, N < 256 ? N : 256, 64))) return rc;
  if ((rc = make_tmap_2d(&mC, C, dtype, static_cast<uint64_t>(batch) * P, N, N, P, 64))) return rc;
  if ((rc = make_tmap_2d(&mD, Dout, dtype, rowsA, P, P, 128, 64))) return rc;
  const int sms = current_sm_count();
#define FTB_B2B_LAUNCH(TT, KK, PP)                                                                          \
  (sh.nchunks == 1 ? launch<TT, KK, PP, 1>(mA, mB, mC, mD, sh, smem_bytes, status, sms, stream)                 \
                   : (sh.nchunks == 2 ? launch<TT, KK, PP, 2>(mA, mB, mC, mD, sh, smem_bytes, status, sms, stream) \
                                      : launch<TT, KK, PP, 4>(mA, mB, mC, mD, sh, smem_bytes, status, sms, stream)))
#define FTB_B2B_BY_SHAPE(TT)                                                                      \
  (K == 128 ? (P == 128 ? FTB_B2B_LAUNCH(TT, 128, 128) : FTB_B2B_LAUNCH(TT, 128, 64))             \
            : (P == 128 ? FTB_B2B_LAUNCH(TT, 64, 128) : FTB_B2B_LAUNCH(TT, 64, 64)))
  if (dtype == FTB_F16) return FTB_B2B_BY_SHAPE(__half);
  return FTB_B2B_BY_SHAPE(__nv_bfloat16);
#undef FTB_B2B_BY_SHAPE
#undef FTB_B2B_LAUNCH
}
