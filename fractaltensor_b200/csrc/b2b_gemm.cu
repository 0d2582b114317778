// Back-to-back GEMM  D = (A . B) . C  for 16-bit inputs on sm_100a.
//
// Arithmetic follows KeBack2BackGemm (kaleido/core/device/kernels/cutlass_wmma.h:489-533):
// S = A.B accumulated in fp32, rounded to the 16-bit input type, D = S.C
// accumulated in fp32, rounded to the 16-bit type.  Unlike the reference, which
// re-reads the A tile for every N tile, every byte of A is read once: the shape
// is HBM-bound, so the kernel is organised around keeping TMA loads of A and TMA
// stores of D in flight while two small MMAs and two conversions run per tile.
//
// One persistent CTA per SM owns a contiguous range of 128-row tiles.
//   warp 0      TMA producer: B and C of the current batch entry, ring of A tiles
//   warp 1      MMA issuer: S = A.B^T into TMEM, then O = P.C^T into TMEM
//   warps 2..5  convert S -> P (16-bit pairs written with tcgen05.st over the TMEM columns
//               of the S tile just read; the second MMA takes its A operand from TMEM),
//               convert O -> D staging, TMA store of D
// P never touches shared memory, which leaves room for a fourth A tile in flight: the shape
// is bound by how many bytes each SM keeps outstanding against DRAM latency.
#include "../../include/ftb200.h"
#include "ptx.cuh"
#include "tmap.h"

namespace ftb {
namespace {

constexpr int kTile = 128;              // rows per tile; also N, K, P
constexpr int kHalfBytes = 128 * 128;   // one 64-column half of a 128x128 16-bit tile
constexpr int kTileBytes = 2 * kHalfBytes;
#ifndef FTB_B2B_STAGES
#define FTB_B2B_STAGES 2
#endif
constexpr int kAStages = FTB_B2B_STAGES;  // A tiles in flight per SM (2, 3 and 4 measured the same)
constexpr int kThreads = 192;
constexpr uint32_t kSmemBytes = (4 + kAStages + 1) * kTileBytes + 1024;  // two (B, C) pairs, A ring, D staging

// Writes 32 fp32 accumulator columns [col0, col0+32) of row `row` as 16-bit
// values into a 128x128 tile laid out as two 64-column halves of 128-byte
// swizzled rows.
template <typename T>
__device__ __forceinline__ void write_row_chunk_sw128(uint8_t* tile, int row, int col0, const uint32_t (&r)[32]) {
  uint8_t* half_base = tile + (col0 >> 6) * kHalfBytes + row * 128;
  const int c0 = (col0 & 63) >> 3;  // first 16-byte chunk inside the 128-byte row
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 u;
    u.x = Fmt<T>::pack2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
    u.y = Fmt<T>::pack2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
    u.z = Fmt<T>::pack2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
    u.w = Fmt<T>::pack2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
    const int chunk = (c0 + j) ^ (row & 7);
    *reinterpret_cast<uint4*>(half_base + chunk * 16) = u;
  }
}

#ifdef FTB_TRACE
__device__ unsigned long long g_b2b_trace[16][8];
#define B2B_STAMP(i, k) if (blockIdx.x == 5 && (i) < 16) g_b2b_trace[i][k] = clock64()
__device__ unsigned long long g_b2b_wall[148][4];
#define B2B_WALL(k) if (blockIdx.x < 148) g_b2b_wall[blockIdx.x][k] = globaltimer_ns()
#else
#define B2B_WALL(k)
#define B2B_STAMP(i, k)
#endif

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
b2b_gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CUtensorMap mapD,
                int total_tiles, int tiles_per_batch, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t a_full[kAStages], a_empty[kAStages];
  __shared__ uint64_t bc_full[2], bc_empty[2];
  __shared__ uint64_t s_full[2], p_full[2], o_full[2], o_empty[2];
  __shared__ uint64_t d_free, d_ready;  // staging tile handshakes between the epilogue warps and the storing thread
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

  if (threadIdx.x == 0) B2B_WALL(0);
  if (*reinterpret_cast<volatile int*>(status) != 0) return;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sBC = smem;  // pair p: B at p * 2 tiles, C one tile further
  uint8_t* sA = sBC + 4 * kTileBytes;
  uint8_t* sD = sA + kAStages * kTileBytes;

  // Contiguous tile range of this CTA.
  const int per = total_tiles / gridDim.x, rem = total_tiles % gridDim.x;
  const int first = blockIdx.x * per + (blockIdx.x < rem ? blockIdx.x : rem);
  const int count = per + (blockIdx.x < rem ? 1 : 0);

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
    }
    mbar_init(&d_free, 1);
    mbar_init(&d_ready, 4);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&o_full[i], 1);
      mbar_init(&o_empty[i], 4);
    }
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
  // TMEM columns: S0 [0,128), S1 [128,256), O0 [256,384), O1 [384,512); P_i (16-bit pairs)
  // overlays the first 64 columns of S_i.

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      // B and C of a batch entry travel together into one of two buffer pairs, one batch entry
      // ahead of the tiles: a CTA whose range crosses into the next batch entry finds its B and C
      // already there instead of draining its pipeline at the boundary.
      const int batch0 = count > 0 ? first / tiles_per_batch : 0;
      const int batch_last = count > 0 ? (first + count - 1) / tiles_per_batch : -1;
      int next_bc = batch0;
      bool ok = true;
      auto load_bc = [&](int b) -> bool {
        const int n = b - batch0, pair = n & 1;
        if (!mbar_wait(&bc_empty[pair], ((n >> 1) & 1) ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_SLOT)) return false;
        uint8_t* dB = sBC + pair * 2 * kTileBytes;
        uint8_t* dC = dB + kTileBytes;
        mbar_arrive_expect_tx(&bc_full[pair], 2 * kTileBytes);
        tma_load_2d(dB, &mapB, &bc_full[pair], 0, b * kTile);
        tma_load_2d(dB + kHalfBytes, &mapB, &bc_full[pair], 64, b * kTile);
        tma_load_2d(dC, &mapC, &bc_full[pair], 0, b * kTile);
        tma_load_2d(dC + kHalfBytes, &mapC, &bc_full[pair], 64, b * kTile);
        return true;
      };
      for (int i = 0; i < count && ok; ++i) {
        const int tile = first + i;
        const int b = tile / tiles_per_batch;
        while (ok && next_bc <= b) ok = load_bc(next_bc++);
        if (!ok) break;
        if (!mbar_wait(&a_empty[stage], phase ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_SLOT)) break;
        uint8_t* dst = sA + stage * kTileBytes;
        mbar_arrive_expect_tx(&a_full[stage], kTileBytes);
        tma_load_2d(dst, &mapA, &a_full[stage], 0, tile * kTile);
        tma_load_2d(dst + kHalfBytes, &mapA, &a_full[stage], 64, tile * kTile);
        if (++stage == kAStages) {
          stage = 0;
          phase ^= 1u;
        }
        // Prefetch the next batch entry's B, C.  Only after this tile's A is on its way: the
        // buffer pair frees up when the MMAs of the batch entry before this one are done, and the
        // MMA warp issues this tile's first product ahead of the previous tile's second.
        while (ok && next_bc <= batch_last && next_bc <= b + 1) ok = load_bc(next_bc++);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(128, 128, Fmt<T>::kind, 0, 0);
      const uint32_t aBC = smem_u32(sBC);
      const int batch0 = count > 0 ? first / tiles_per_batch : 0;
      int stage = 0;
      uint32_t a_phase = 0;
      uint32_t o_phase[2] = {0, 0}, p_phase[2] = {0, 0};
      int cur_batch = -1;
      bool ok = true;

      // GEMM 1 of tile i: S[i&1] = A . B^T.  The buffer last held S/P of tile i-2, whose GEMM 2 was
      // issued before this one and so runs before it on the tensor pipe.
      auto gemm1 = [&](int i) -> bool {
        const int b = (first + i) / tiles_per_batch;
        const int n = b - batch0;
        if (b != cur_batch) {
          if (!mbar_wait(&bc_full[n & 1], (n >> 1) & 1, &s_abort, status, FTB_ERR_TIMEOUT_TMA)) return false;
          cur_batch = b;
        }
        const uint32_t aB = aBC + (n & 1) * 2 * kTileBytes;
        const int sb = i & 1;
        if (!mbar_wait(&a_full[stage], a_phase, &s_abort, status, FTB_ERR_TIMEOUT_TMA)) return false;
        tc_fence_after();
        B2B_STAMP(i, 0);
        if (i == 0) B2B_WALL(1);
        const uint32_t aA = smem_u32(sA + stage * kTileBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
          umma_ss(tmem_base + sb * 128, make_sdesc_sw128(aA + off, 16, 1024), make_sdesc_sw128(aB + off, 16, 1024),
                  idesc, k != 0 ? 1u : 0u);
        }
        umma_commit(&a_empty[stage]);
        umma_commit(&s_full[sb]);
        if (++stage == kAStages) {
          stage = 0;
          a_phase ^= 1u;
        }
        return true;
      };
      // GEMM 2 of tile i: O[i&1] = P . C^T, P from TMEM (16 of the 128 inner positions = 8 packed
      // columns per step).
      auto gemm2 = [&](int i, bool last_of_batch) -> bool {
        const int ob = i & 1;
        const int n = (first + i) / tiles_per_batch - batch0;
        const uint32_t aC = aBC + ((n & 1) * 2 + 1) * kTileBytes;
        if (!mbar_wait(&o_empty[ob], o_phase[ob] ^ 1u, &s_abort, status, FTB_ERR_TIMEOUT_EPI)) return false;
        o_phase[ob] ^= 1u;
        // One barrier per S/P buffer: the converting warps can be a whole tile ahead of this wait
        // (S of the next tile is ready early), and a parity wait must not fall two phases behind.
        if (!mbar_wait(&p_full[ob], p_phase[ob], &s_abort, status, FTB_ERR_TIMEOUT_EPI)) return false;
        p_phase[ob] ^= 1u;
        tc_fence_after();
        B2B_STAMP(i, 3);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
          umma_ts(tmem_base + 256 + ob * 128, tmem_base + ob * 128 + k * 8, make_sdesc_sw128(aC + off, 16, 1024),
                  idesc, k != 0 ? 1u : 0u);
        }
        umma_commit(&o_full[ob]);
        if (last_of_batch) umma_commit(&bc_empty[n & 1]);
        return true;
      };

      if (count > 0) ok = gemm1(0);
      for (int i = 0; i < count && ok; ++i) {
        const bool has_next = i + 1 < count;
        const bool next_new_batch = has_next && ((first + i + 1) / tiles_per_batch != (first + i) / tiles_per_batch);
        // Run ahead with GEMM 1 of the next tile (its B sits in the other buffer pair if it
        // belongs to the next batch entry).
        if (has_next) ok = gemm1(i + 1);
        if (ok) ok = gemm2(i, next_new_batch || !has_next);
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const bool issuer = (warp == 2 && lane == 0);
    uint32_t s_phase[2] = {0, 0}, o_phase[2] = {0, 0}, d_phase = 0;
    bool ok = true;

    auto convert_s = [&](int i) -> bool {
      const int sb = i & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[sb], s_phase[sb], &s_abort, status, FTB_ERR_TIMEOUT_MMA)))
        return false;
      s_phase[sb] ^= 1u;
      tc_fence_after();
      if (threadIdx.x == 64) B2B_STAMP(i, 1);
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
      if (threadIdx.x == 64) B2B_STAMP(i, 2);
      return true;
    };
    auto output_o = [&](int i) -> bool {
      const int ob = i & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&o_full[ob], o_phase[ob], &s_abort, status, FTB_ERR_TIMEOUT_MMA)))
        return false;
      o_phase[ob] ^= 1u;
      tc_fence_after();
      if (threadIdx.x == 64) B2B_STAMP(i, 4);
      // The previous TMA store must have finished reading the staging tile.
      if (issuer) {
        tma_store_wait_read<0>();
        mbar_arrive(&d_free);
      }
      if (!__all_sync(0xffffffffu, mbar_wait(&d_free, d_phase, &s_abort, status, FTB_ERR_TIMEOUT_EPI))) return false;
      if (threadIdx.x == 64) B2B_STAMP(i, 5);
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
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
      if (threadIdx.x == 64) B2B_STAMP(i, 6);
      const bool staged = !issuer || mbar_wait(&d_ready, d_phase, &s_abort, status, FTB_ERR_TIMEOUT_EPI);
      d_phase ^= 1u;
      if (issuer && staged) {
        const int tile = first + i;
        tma_store_2d(&mapD, sD, 0, tile * kTile);
        tma_store_2d(&mapD, sD + kHalfBytes, 64, tile * kTile);
        tma_store_commit();
        B2B_STAMP(i, 7);
      }
      return true;
    };

    for (int i = 0; i < count && ok; ++i) {
      ok = convert_s(i);
      if (ok && i > 0) ok = output_o(i - 1);
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

template <typename T>
int launch(const CUtensorMap& mA, const CUtensorMap& mB, const CUtensorMap& mC, const CUtensorMap& mD, int total,
           int tiles_per_batch, int* status, int sm_count, cudaStream_t stream) {
  static bool configured = false;
  auto kfn = b2b_gemm_kernel<T>;
  if (!configured) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
      return FTB_ERR_LAUNCH;
    configured = true;
  }
  const int grid = total < sm_count ? total : sm_count;
  kfn<<<grid, kThreads, kSmemBytes, stream>>>(mA, mB, mC, mD, total, tiles_per_batch, status);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
}

}  // namespace
}  // namespace ftb

using namespace ftb;

#ifdef FTB_TRACE
extern "C" int ftb_debug_b2b_trace(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, g_b2b_trace, sizeof(unsigned long long) * 16 * 8) == cudaSuccess ? 0 : 1;
}
extern "C" int ftb_debug_b2b_wall(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, g_b2b_wall, sizeof(unsigned long long) * 148 * 4) == cudaSuccess ? 0 : 1;
}
#endif

extern "C" int ftb_b2b_gemm(const void* A, const void* B, const void* C, void* Dout, int batch, int M, int N, int K,
                            int P, int dtype, void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!A || !B || !C || !Dout || batch <= 0 || M <= 0) return FTB_ERR_ARG;
  if (dtype != FTB_F16 && dtype != FTB_BF16) return FTB_ERR_ARG;
  if (N != 128 || K != 128 || P != 128 || M % 128 != 0) return FTB_ERR_ARG;
  if (static_cast<int64_t>(batch) * M > 0x7fffffffLL) return FTB_ERR_ARG;
  if (workspace == nullptr || workspace_bytes < ftb_workspace_bytes()) return FTB_ERR_WORKSPACE;
  int rc = check_device_sm100();
  if (rc) return rc;
  // The status word is sticky: the caller zeroes the workspace once; after a device wait ran out
  // every later call on that workspace is a no-op until the caller clears the word.
  int* status = static_cast<int*>(workspace);

  CUtensorMap mA, mB, mC, mD;
  const uint64_t rowsA = static_cast<uint64_t>(batch) * M;
  if ((rc = make_tmap_2d(&mA, A, dtype, rowsA, K, K, 128, 64))) return rc;
  if ((rc = make_tmap_2d(&mB, B, dtype, static_cast<uint64_t>(batch) * N, K, K, 128, 64))) return rc;
  if ((rc = make_tmap_2d(&mC, C, dtype, static_cast<uint64_t>(batch) * P, N, N, 128, 64))) return rc;
  if ((rc = make_tmap_2d(&mD, Dout, dtype, rowsA, P, P, 128, 64))) return rc;
  const int tiles_per_batch = M / 128;
  const int total = batch * tiles_per_batch;
  const int sms = current_sm_count();
  if (dtype == FTB_F16) return launch<__half>(mA, mB, mC, mD, total, tiles_per_batch, status, sms, stream);
  return launch<__nv_bfloat16>(mA, mB, mC, mD, total, tiles_per_batch, status, sms, stream);
}
