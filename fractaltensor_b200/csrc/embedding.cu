// Embedding lookup: out[t, :] = table[ids[t], :].
//
// Stands in for the lookup the reference's RNN examples run before the recurrence,
//   ops.map(lambda words: ops.map(lambda word: ops.index(ops.slices(embedding, dim=0), word), words), batch)
// (examples/stacked_rnn/rnn_utils.py:80-90, with Slices / Index of
// kaleido/frontend/operations/fractaltensor/access.py), which copies one table row per word
// into the flat buffer of a FractalTensor of [1, H] tensors: a gather of T rows.
//
// HBM-bound byte work: 2 * H * element size bytes per row plus 8 for the index.  A warp moves
// one row at a time with 16-byte accesses (rows that are not a multiple of 16 bytes long fall
// back to element-wise copies); the grid is a whole number of CTAs per SM striding over rows.
// An index outside [0, V) writes a row of zeros and records FTB_ERR_INDEX in the status word.
#include "../../include/ftb200.h"
#include "ptx.cuh"
#include "tmap.h"

namespace ftb {
namespace {

constexpr int kGatherThreads = 256;

__global__ void __launch_bounds__(kGatherThreads)
embedding_gather_kernel(const unsigned char* __restrict__ table, const long long* __restrict__ ids,
                        unsigned char* __restrict__ out, long long T, long long V, int row_bytes, int vec16,
                        int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * kGatherThreads + threadIdx.x) >> 5;
  const long long n_warps = (static_cast<long long>(gridDim.x) * kGatherThreads) >> 5;
  grid_launch_dependents();
  grid_dependency_wait();
  for (long long t = warp; t < T; t += n_warps) {
    const long long id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && lane == 0) atomicCAS(status, 0, FTB_ERR_INDEX);
    unsigned char* dst = out + t * row_bytes;
    const unsigned char* src = table + (ok ? id : 0) * row_bytes;
    if (vec16) {
      const uint4* s4 = reinterpret_cast<const uint4*>(src);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      for (int i = lane; i < row_bytes / 16; i += 32) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (ok) v = __ldg(s4 + i);  // table rows are re-used across words: let them stay in cache
        __stcs(d4 + i, v);          // the output streams out
      }
    } else {
      for (int i = lane; i < row_bytes; i += 32) dst[i] = ok ? src[i] : static_cast<unsigned char>(0);
    }
  }
}

}  // namespace
}  // namespace ftb

using namespace ftb;

extern "C" int ftb_embedding_gather(const void* table, const long long* ids, void* out, long long T, long long V,
                                    int H, int dtype, void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!table || !ids || !out || T < 0 || V <= 0 || H <= 0) return FTB_ERR_ARG;
  if (dtype != FTB_F32 && dtype != FTB_F16 && dtype != FTB_BF16) return FTB_ERR_ARG;
  if (workspace == nullptr || workspace_bytes < ftb_workspace_bytes()) return FTB_ERR_WORKSPACE;
  if (T == 0) return FTB_OK;
  int rc = check_device_sm100();
  if (rc) return rc;
  const int es = dtype == FTB_F32 ? 4 : 2;
  const long long row_bytes = static_cast<long long>(H) * es;
  if (row_bytes > 0x7fffffffLL) return FTB_ERR_ARG;
  const bool vec16 = row_bytes % 16 == 0 && ((reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  // The status word is sticky, as for the other single-kernel entry points.
  int* status = static_cast<int*>(workspace);
  const long long warps_needed = T;
  const long long ctas_needed = (warps_needed * 32 + kGatherThreads - 1) / kGatherThreads;
  const long long full = static_cast<long long>(current_sm_count()) * 8;  // 8 CTAs of 256 threads per SM
  const int grid = static_cast<int>(ctas_needed < full ? ctas_needed : full);
  const cudaError_t err = launch_light(embedding_gather_kernel, dim3(grid), dim3(kGatherThreads), 0, stream,
                                           static_cast<const unsigned char*>(table), ids, static_cast<unsigned char*>(out),
                                           T, V, static_cast<int>(row_bytes), vec16 ? 1 : 0, status);
  count_launch();
  if (err != cudaSuccess) cudaGetLastError();
  return err == cudaSuccess ? FTB_OK : FTB_ERR_LAUNCH;
}
