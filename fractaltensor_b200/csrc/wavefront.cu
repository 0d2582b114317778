// Host side of the RNN hot path: wavefront schedulers that turn the
// fold/scan/map nests of the reference programs into levels of independent
// cells, one kernel launch per level, plus the C-ABI entry points.
//
// The reference derives the same schedules by hand per benchmark
// (benchmarks/rnn/fractaltensor/stacked_lstm/regions/region3.h:11-28 for the
// stacked skew m = d + t, dilated_lstm/regions/region2.h:34-93 for the dilated
// steps, grid_lstm/regions/region8.h:26-53 for m = d + i + j) and executes each
// hyperplane as gather -> batched GEMM -> elementwise -> scatter.  Here a level
// is one launch of a fused cell kernel that addresses the hyperplane in place.
#include <algorithm>
#include <initializer_list>
#include <map>
#include <mutex>
#include <vector>

#include "../../include/ftb200.h"
#include "cell.h"
#include "ptx.cuh"
#include "tmap.h"

namespace ftb {

int launch_cell_gemm(int dtype, int epi, int bn, int pair, const CUtensorMap* maps, const CUtensorMap& mapW,
                     const CUtensorMap& mapC, const CellBatch& batch, int* status, int sm_count,
                     cudaStream_t stream);
int launch_cell_gemm_persistent(int dtype, int epi, int bn, int pair, const CUtensorMap* maps,
                                const CUtensorMap& mapW, const CUtensorMap& mapC, const CellBatch& header,
                                const PlanView& plan, int* status, int sm_count, cudaStream_t stream);
bool lstm_simt_static_supported(int D, int N, int I, int H, int sm_count);
int launch_lstm_simt_static(const float* x, const float* Wp, const float* bias_p, float* hs, float* c, int D, int L,
                            int N, int I, int H, int* done, int* status, int sm_count, cudaStream_t stream);
bool lstm_static_supported(int dtype, int D, int N, int I, int H, int G, int sm_count);
int launch_lstm_static(int dtype, const void* x, const void* Wp, const float* bias_p, void* hs, float* c, int D, int L,
                       int N, int I, int H, int G, int* done, int* status, unsigned long long* trace,
                       cudaStream_t stream);
bool lstm_wmajor_supported(int dtype, int D, int N, int I, int H, int G, int sm_count);
int launch_lstm_wmajor(int dtype, const void* x, const void* Wp, const float* bias_p, void* hs, float* c, int D, int L,
                       int N, int I, int H, int G, int resident, int* done, int* status, unsigned long long* trace,
                       cudaStream_t stream);
bool lstm_dilated_cluster_supported(int dtype, int D, int N, int H, int sm_count);
size_t lstm_dilated_cluster_flag_ints(int D, int L);
int launch_lstm_dilated_cluster(int dtype, const void* x, const void* Wp, const float* bias_p, void* hs, float* c,
                                const int* dilations, int D, int L, int N, int H, int* flags, int* status,
                                cudaStream_t stream);
bool grid_rnn_cluster_supported(int dtype, int D, int A, int B, int N, int H, int sm_count);
int launch_grid_rnn_cluster(int dtype, const void* X, const void* Y, const void* Wpx, const void* Wpy,
                            const float* bias_x, const float* bias_y, void* hx, void* hy, int D, int A, int B, int N,
                            int H, int* flags, int* status, cudaStream_t stream);
int launch_cell_simt(int epi, const float* const* act, const int* ld_act, const float* const* w, int ldw,
                     const CellBatch& batch, cudaStream_t stream);
int pack_lstm(const void* W, const void* U, const void* bias, void* Wp, float* bias_p, int D, int I, int H, int dtype,
              cudaStream_t s);
int pack_grid(const void* i2h, const void* h2h, void* Wp, int H, int dtype, cudaStream_t s);
int pack_projection(const void* P, void* Pt, int H, int V, int Vp, int dtype, cudaStream_t s);
int pack_rnn(const void* W, const void* U, void* Wp, int I, int H, int dtype, cudaStream_t s);
int rnn_attention_max_src_len();
int launch_enc_scores(int dtype, const void* enc, const void* proj, float* scores, long long n_rows, int H,
                      cudaStream_t stream);
int launch_attn_step(int dtype, const void* enc, const float* enc_scores, const void* dec_t, const void* dec_proj,
                     const int* src_lens, void* out_t, int Ls, int N, int H, cudaStream_t stream);
int online_softmax_rows(const float* x, float* y, int rows, int width, int ld, cudaStream_t stream);

namespace {

constexpr size_t kWorkspaceBytes = 256;

// Launch context for one family of cells (up to two weight buffers, up to four
// activation buffers).
struct CellLauncher {
  int dtype = FTB_BF16;
  int epi = EPI_STORE;
  int bn = 128;
  int pair = 0;  // 16-bit path: run CTAs as pairs on 256-row blocks
  int n_cols = 0, ld_out = 0, ld_c = 0;
  int sm_count = 0;
  int* status = nullptr;
  cudaStream_t stream = nullptr;
  // 16-bit path
  CUtensorMap maps[kNumActMaps];
  CUtensorMap mapW;
  CUtensorMap mapC;  // fp32 cell state (LSTM); otherwise the second weight buffer's map (or a copy of mapW)
  // fp32 path
  const float* act[kNumActMaps] = {nullptr, nullptr, nullptr, nullptr};
  int ld_act[kNumActMaps] = {0, 0, 0, 0};
  const float* w = nullptr;   // weight buffer 0
  const float* w2 = nullptr;  // weight buffer 1 (cells with w_map == 1), same row length
  int ldw = 0;

  int rows_per_tile() const { return dtype == FTB_F32 ? 32 : 128; }
  int m_tiles_for(int rows) const {
    if (dtype != FTB_F32 && pair) return 2 * ((rows + 255) / 256);
    return (rows + rows_per_tile() - 1) / rows_per_tile();
  }
  int w_box_rows() const { return pair ? bn / 2 : bn; }
  int cols_per_tile() const { return dtype == FTB_F32 ? 32 : bn; }

  // Launches the cells of one level (any number; split into chunks).
  int run(std::vector<CellItem>& items) const {
    const int n_tiles_n = (n_cols + cols_per_tile() - 1) / cols_per_tile();
    for (size_t off = 0; off < items.size(); off += kMaxItems) {
      CellBatch b;
      b.n_items = static_cast<int>(std::min<size_t>(kMaxItems, items.size() - off));
      b.n_cols = n_cols;
      b.ld_out = ld_out;
      b.ld_c = ld_c;
      b.pad_ = 0;
      int tiles = 0;
      for (int i = 0; i < b.n_items; ++i) {
        CellItem it = items[off + i];
        it.m_tiles = m_tiles_for(it.rows);
        it.tile0 = tiles;
        tiles += it.m_tiles * n_tiles_n;
        b.items[i] = it;
      }
      b.total_tiles = tiles;
      int rc;
      if (dtype == FTB_F32) {
        const float* ws[kNumWeightMaps] = {w, w2 ? w2 : w};
        rc = launch_cell_simt(epi, act, ld_act, ws, ldw, b, stream);
      } else {
        rc = launch_cell_gemm(dtype, epi, bn, pair, maps, mapW, mapC, b, status, sm_count, stream);
      }
      if (rc) return rc;
    }
    return FTB_OK;
  }
};

// Runs a whole wavefront as one persistent launch: `items` in an order in which every item
// only depends on earlier ones, `deps[i]` = per segment the inclusive range of item indices the
// segment reads (-1 = external).  Tables go to the workspace with stream-ordered copies.
int run_persistent(const CellLauncher& cl, std::vector<CellItem>& items, const std::vector<int32_t>& deps,
                   char* ws, const struct PlanLayout& lay);

CellItem blank_item() {
  CellItem it;
  it.out = nullptr;
  it.c = nullptr;
  it.bias = nullptr;
  for (int s = 0; s < kMaxSeg; ++s) it.seg_row[s] = it.seg_kb[s] = it.seg_wk[s] = it.seg_map[s] = 0;
  it.nseg = 0;
  it.w_row0 = 0;
  it.rows = 0;
  it.c_zero = 0;
  it.tile0 = 0;
  it.m_tiles = 0;
  it.out_row0 = 0;
  it.c_row0 = 0;
  it.out_map = 1;
  it.w_map = 0;
  it.skip = 0;
  it.pad_ = 0;
  return it;
}

void add_seg(CellItem& it, int map, int64_t row, int k_elems, int wk) {
  const int s = it.nseg++;
  it.seg_map[s] = map;
  it.seg_row[s] = static_cast<int32_t>(row);
  it.seg_kb[s] = k_elems / 64;
  it.seg_wk[s] = wk;
}

int begin_call(void* workspace, size_t workspace_bytes, cudaStream_t stream, int** status) {
  if (workspace == nullptr || workspace_bytes < kWorkspaceBytes) return FTB_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0) return FTB_ERR_ALIGN;
  int rc = check_device_sm100();
  if (rc) return rc;
  if (cudaMemsetAsync(workspace, 0, kWorkspaceBytes, stream) != cudaSuccess) return FTB_ERR_LAUNCH;
  *status = static_cast<int*>(workspace);
  return FTB_OK;
}

bool valid_dtype(int dt) { return dt == FTB_F32 || dt == FTB_F16 || dt == FTB_BF16; }

// Every kernel reads and writes 16 bytes at a time (the fp32 path as float4, the 16-bit path by TMA).
bool aligned16(std::initializer_list<const void*> ptrs) {
  for (const void* p : ptrs)
    if ((reinterpret_cast<uintptr_t>(p) & 15) != 0) return false;
  return true;
}

// Optional tuning knobs of the wavefront entry points (0 = automatic).
struct Tuning {
  int layers_per_group = 0, bn = 0, schedule = 0, skew = 0, pair = 0, fine_deps = 0, resident = 0;
  explicit Tuning(const int* t) {
    if (t != nullptr) {
      layers_per_group = t[0];
      bn = t[1];
      schedule = t[2];
      skew = t[3];
      pair = t[4];
      fine_deps = t[5];
      resident = t[6];
    }
  }
  // pair: 0 = automatic (pairs when a cell has more than 128 rows), 1 = never, 2 = always.
  int use_pair(int rows) const { return pair == 2 || (pair == 0 && rows > 128); }
};

// ---------------------------------------------------------- persistent schedule
// Workspace layout of a persistent stacked-LSTM call: status block, then the
// item table, the dependency table, the completion targets and the counters.
constexpr int kMaxCtas = 1024;  // entries of the per-CTA first-item table
struct PlanLayout {
  size_t items, dep, target, cta_first, done, tile_done, c_done, counters_end, trace, total;
};
PlanLayout plan_layout(int n_items, int max_tiles_per_item = 64) {
  PlanLayout p;
  auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
  p.items = kWorkspaceBytes;
  p.dep = up(p.items + sizeof(CellItem) * n_items);
  p.target = up(p.dep + sizeof(int32_t) * 2 * kMaxSeg * n_items);
  p.cta_first = up(p.target + sizeof(int32_t) * n_items);
  p.done = up(p.cta_first + sizeof(int32_t) * kMaxCtas);
  const size_t max_tiles = static_cast<size_t>(n_items) * max_tiles_per_item;
  p.tile_done = up(p.done + sizeof(int32_t) * 2 * n_items);
  p.c_done = up(p.tile_done + sizeof(int32_t) * max_tiles);
  p.counters_end = up(p.c_done + sizeof(int32_t) * max_tiles);
  p.trace = p.counters_end;
#ifdef FTB_TRACE
  p.total = up(p.trace + 8 * 4 * max_tiles);
#else
  p.total = p.trace;
#endif
  return p;
}

int run_persistent(const CellLauncher& cl, std::vector<CellItem>& items, const std::vector<int32_t>& deps,
                   char* ws, const PlanLayout& lay, size_t ws_bytes = 0) {
  const int n = static_cast<int>(items.size());
  const int n_tiles_n = (cl.n_cols + cl.cols_per_tile() - 1) / cl.cols_per_tile();
  std::vector<int32_t> target(n);
  int tiles = 0;
  for (int i = 0; i < n; ++i) {
    items[i].m_tiles = cl.m_tiles_for(items[i].rows);
    items[i].tile0 = tiles;
    tiles += items[i].m_tiles * n_tiles_n;
    target[i] = 8 * items[i].m_tiles * n_tiles_n;  // eight epilogue warps per tile
  }
  // Tile -> item lookups without a table walk on the device (the grid size computed here is
  // the one launch_cell_gemm_persistent uses): for every item the item that holds the tile one
  // grid stride further, and for every CTA the item of its first tile.
  int grid = std::min(tiles, cl.sm_count);
  if (cl.pair) grid &= ~1;
  if (grid <= 0) return FTB_OK;
  if (grid > kMaxCtas) return FTB_ERR_ARG;
  {
    int j = 0;
    for (int i = 0; i < n; ++i) {
      const int t = items[i].tile0 + grid;
      while (j + 1 < n && t >= items[j + 1].tile0) ++j;
      items[i].skip = j;
    }
  }
  std::vector<int32_t> cta_first(grid);
  {
    int j = 0;
    for (int c = 0; c < grid; ++c) {
      while (j + 1 < n && c >= items[j + 1].tile0) ++j;
      cta_first[c] = j;
    }
  }
  // The host vectors die with this call; cudaMemcpyAsync from pageable memory returns once the
  // bytes are staged.
  if (cudaMemcpyAsync(ws + lay.items, items.data(), sizeof(CellItem) * n, cudaMemcpyHostToDevice, cl.stream) !=
          cudaSuccess ||
      cudaMemcpyAsync(ws + lay.dep, deps.data(), sizeof(int32_t) * 2 * kMaxSeg * n, cudaMemcpyHostToDevice,
                      cl.stream) != cudaSuccess ||
      cudaMemcpyAsync(ws + lay.target, target.data(), sizeof(int32_t) * n, cudaMemcpyHostToDevice, cl.stream) !=
          cudaSuccess ||
      cudaMemcpyAsync(ws + lay.cta_first, cta_first.data(), sizeof(int32_t) * grid, cudaMemcpyHostToDevice,
                      cl.stream) != cudaSuccess ||
      cudaMemsetAsync(ws + lay.done, 0, sizeof(int32_t) * 2 * n, cl.stream) != cudaSuccess)
    return FTB_ERR_LAUNCH;
  CellBatch header;
  header.n_items = n;
  header.n_cols = cl.n_cols;
  header.ld_out = cl.ld_out;
  header.ld_c = cl.ld_c;
  header.total_tiles = tiles;
  header.pad_ = 0;
  PlanView pv = {reinterpret_cast<const CellItem*>(ws + lay.items), reinterpret_cast<const int32_t*>(ws + lay.dep),
                 reinterpret_cast<const int32_t*>(ws + lay.target), reinterpret_cast<int32_t*>(ws + lay.done),
                 nullptr, nullptr, 0, 0, 0, 0, reinterpret_cast<const int32_t*>(ws + lay.cta_first), nullptr};
#ifdef FTB_TRACE
  // Debug build: four time stamps per tile behind the tables, when the caller left room.
  if (ws_bytes >= lay.total + static_cast<size_t>(32) * tiles)
    pv.trace = reinterpret_cast<unsigned long long*>(ws + lay.total);
#endif
  return launch_cell_gemm_persistent(cl.dtype, cl.epi, cl.bn, cl.pair, cl.maps, cl.mapW, cl.mapC, header, pv,
                                     cl.status, cl.sm_count, cl.stream);
}

struct StackedPlanArgs {
  int D, L, N, I, H, G, skew, es, tiles_per_item, m_tiles;
  char* hs;
  float* c;
  const float* bias_p;
  CellItem* items;
  int32_t* dep;
  int32_t* target;
};

// Position of cell (l, t) in the launch order: groups of G layers one after the
// other; inside a group level by level, level m = skew * j + t with j the layer's
// index in the group, lower layers first.  A cell reads (l, t-1), one level back,
// and (l-1, t), `skew` levels back (or in an earlier group): with skew >= 2 the
// input half of a cell's K loop can run while the cells of the previous level,
// which feed its recurrent half, are still finishing.
__device__ int stacked_item_index(const StackedPlanArgs& a, int l, int t) {
  const int g0 = (l / a.G) * a.G;
  const int Lg = min(a.G, a.D - g0);
  const int j = l - g0;
  const int m = a.skew * j + t;
  int before = 0;
  for (int q = 0; q < m; ++q) {
    const int j_lo = (max(0, q - a.L + 1) + a.skew - 1) / a.skew;
    const int j_hi = min(Lg - 1, q / a.skew);
    before += max(0, j_hi - j_lo + 1);
  }
  const int j_min = (max(0, m - a.L + 1) + a.skew - 1) / a.skew;
  return g0 * a.L + before + (j - j_min);
}

__global__ void plan_stacked_kernel(const StackedPlanArgs a) {
  const int id = blockIdx.x * blockDim.x + threadIdx.x;
  if (id >= a.D * a.L) return;
  const int l = id / a.L, t = id - l * a.L;
  const int pos = stacked_item_index(a, l, t);
  CellItem it;
  for (int s = 0; s < kMaxSeg; ++s) it.seg_row[s] = it.seg_kb[s] = it.seg_wk[s] = it.seg_map[s] = 0;
  int32_t dep[kMaxSeg][2] = {{-1, -1}, {-1, -1}, {-1, -1}};
  int ns = 0;
  if (l == 0) {
    it.seg_map[ns] = 0; it.seg_row[ns] = t * a.N; it.seg_kb[ns] = a.I / 64; it.seg_wk[ns] = 0;
  } else {
    it.seg_map[ns] = 1; it.seg_row[ns] = ((l - 1) * a.L + t) * a.N; it.seg_kb[ns] = a.H / 64; it.seg_wk[ns] = 0;
    dep[ns][0] = dep[ns][1] = stacked_item_index(a, l - 1, t);
  }
  ++ns;
  if (t > 0) {
    it.seg_map[ns] = 2; it.seg_row[ns] = (l * a.L + t - 1) * a.N; it.seg_kb[ns] = a.H / 64; it.seg_wk[ns] = a.I;
    dep[ns][0] = dep[ns][1] = stacked_item_index(a, l, t - 1);
    ++ns;
  }
  it.nseg = ns;
  it.w_row0 = l * 4 * a.H;
  it.rows = a.N;
  it.c_zero = (t == 0);
  it.out = a.hs + (static_cast<size_t>(l) * a.L + t) * a.N * a.H * a.es;
  it.out_row0 = (l * a.L + t) * a.N;
  it.out_map = 1;
  it.w_map = 0;
  it.skip = 0;
  it.pad_ = 0;
  it.c = a.c + static_cast<size_t>(l) * a.N * a.H;
  it.c_row0 = l * a.N;
  it.bias = a.bias_p ? a.bias_p + static_cast<size_t>(l) * 4 * a.H : nullptr;
  it.m_tiles = a.m_tiles;
  it.tile0 = pos * a.tiles_per_item;
  a.items[pos] = it;
  for (int s = 0; s < kMaxSeg; ++s) {
    a.dep[(pos * kMaxSeg + s) * 2 + 0] = dep[s][0];
    a.dep[(pos * kMaxSeg + s) * 2 + 1] = dep[s][1];
  }
  a.target[pos] = 8 * a.tiles_per_item;  // eight epilogue warps per tile
}

// Accumulator tile width.  The last column tile of a cell may be partial (the
// epilogue skips 32-column groups past n_cols), so n_cols % 32 == 0 is enough.
int pick_bn(int n_cols, int want) {
  if (n_cols % 32 != 0) return 0;
  if (want == 128 || want == 256) return want;
  if (want != 0) return 0;
  return (n_cols % 256 == 0 && n_cols >= 2048) ? 256 : 128;
}

}  // namespace
}  // namespace ftb

using namespace ftb;

extern "C" {

int ftb_version(void) { return 1; }

const char* ftb_status_str(int code) {
  switch (code) {
    case FTB_OK: return "ok";
    case FTB_ERR_ARG: return "bad argument (shape, pointer or dtype)";
    case FTB_ERR_ALIGN: return "pointer or stride not 16-byte aligned";
    case FTB_ERR_WORKSPACE: return "workspace missing or too small";
    case FTB_ERR_DRIVER: return "tensor-map encode failed or driver entry point missing";
    case FTB_ERR_LAUNCH: return "kernel launch failed";
    case FTB_ERR_ARCH: return "device is not sm_100";
    case FTB_ERR_SCRATCH_LIMIT: return "problem needs more scratch than the built-in static buffer holds";
    case FTB_ERR_TIMEOUT_TMA: return "device wait ran out: TMA stage never arrived";
    case FTB_ERR_TIMEOUT_MMA: return "device wait ran out: MMA never committed";
    case FTB_ERR_TIMEOUT_EPI: return "device wait ran out: epilogue never drained";
    case FTB_ERR_TIMEOUT_SLOT: return "device wait ran out: no free pipeline stage";
    case FTB_ERR_TIMEOUT_DEP: return "device wait ran out: a cell's inputs never completed";
    case FTB_ERR_TMEM_LAYOUT: return "the two CTAs of a pair got different TMEM columns";
    case FTB_ERR_INDEX: return "an index was outside its table";
    default: return "unknown status";
  }
}

size_t ftb_workspace_bytes(void) { return kWorkspaceBytes; }

long long ftb_launch_count(void) { return launches_so_far(); }

int ftb_read_status(const void* workspace, int* status_out, void* stream) {
  if (workspace == nullptr || status_out == nullptr) return FTB_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(status_out, workspace, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return FTB_ERR_LAUNCH;
  if (cudaStreamSynchronize(s) != cudaSuccess) return FTB_ERR_LAUNCH;
  return FTB_OK;
}

int ftb_lstm_pack_weights(const void* W, const void* U, const void* bias, void* Wp, float* bias_p, int D, int I,
                          int H, int dtype, void* stream) {
  if (!W || !U || !Wp || D <= 0 || I <= 0 || H <= 0 || !valid_dtype(dtype)) return FTB_ERR_ARG;
  if (bias != nullptr && bias_p == nullptr) return FTB_ERR_ARG;
  return pack_lstm(W, U, bias, Wp, bias_p, D, I, H, dtype, static_cast<cudaStream_t>(stream));
}

int ftb_grid_pack_weights(const void* i2h, const void* h2h, void* Wp, int H, int dtype, void* stream) {
  if (!i2h || !h2h || !Wp || H <= 0 || !valid_dtype(dtype)) return FTB_ERR_ARG;
  return pack_grid(i2h, h2h, Wp, H, dtype, static_cast<cudaStream_t>(stream));
}

// Upper bound of tiles per cell over the tile shapes the library may pick.
static int stacked_max_tiles_per_cell(int N, int H) { return 2 * ((N + 255) / 256) * ((4 * H + 127) / 128); }

size_t ftb_lstm_stacked_workspace_bytes(int D, int L, int N, int H) {
  if (D <= 0 || L <= 0 || N <= 0 || H <= 0) return kWorkspaceBytes;
  return plan_layout(D * L, stacked_max_tiles_per_cell(N, H)).total;
}

int ftb_lstm_stacked_fwd(const void* x, const void* Wp, const float* bias_p, void* hs, float* c, int D, int L,
                         int N, int I, int H, int dtype, const int* tuning, void* workspace, size_t workspace_bytes,
                         void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const Tuning tune(tuning);
  const int layers_per_group = tune.layers_per_group, bn = tune.bn, schedule = tune.schedule, skew = tune.skew;
  if (!x || !Wp || !hs || !c || D <= 0 || L <= 0 || N <= 0 || !valid_dtype(dtype)) return FTB_ERR_ARG;
  if (H <= 0 || I <= 0 || H % 64 != 0 || I % 64 != 0) return FTB_ERR_ARG;
  if (D > 1 && I != H) return FTB_ERR_ARG;
  if (static_cast<int64_t>(D) * L * N > 0x7fffffffLL) return FTB_ERR_ARG;
  if (!aligned16({x, Wp, bias_p, hs, c})) return FTB_ERR_ALIGN;
  int* status = nullptr;
  int rc = begin_call(workspace, workspace_bytes, stream, &status);
  if (rc) return rc;

  const int K = I + H;
  const size_t es = dtype_size(dtype);
  CellLauncher cl;
  cl.dtype = dtype;
  cl.epi = EPI_LSTM;
  cl.n_cols = 4 * H;
  cl.ld_out = H;
  cl.ld_c = H;
  cl.status = status;
  cl.stream = stream;
  cl.sm_count = current_sm_count();
  if (dtype == FTB_F32) {
    cl.act[0] = static_cast<const float*>(x);
    cl.ld_act[0] = I;
    cl.act[1] = cl.act[2] = static_cast<const float*>(hs);
    cl.ld_act[1] = cl.ld_act[2] = H;
    cl.w = static_cast<const float*>(Wp);
    cl.ldw = K;
  } else {
    cl.bn = pick_bn(4 * H, bn);
    if (cl.bn == 0) return FTB_ERR_ARG;
    cl.pair = tune.use_pair(N);
    rc = make_tmap_2d(&cl.maps[0], x, dtype, static_cast<uint64_t>(L) * N, I, I, 128, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.maps[1], hs, dtype, static_cast<uint64_t>(D) * L * N, H, H, 128, 64);
    if (rc) return rc;
    cl.maps[2] = cl.maps[1];
    cl.maps[3] = cl.maps[0];
    rc = make_tmap_2d(&cl.mapW, Wp, dtype, static_cast<uint64_t>(D) * 4 * H, K, K, cl.w_box_rows(), 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.mapC, c, FTB_F32, static_cast<uint64_t>(D) * N, H, H, 128, 32);
    if (rc) return rc;
  }

  int G = layers_per_group;
  if (G <= 0) {
    // Keep a group's packed weights within about half of L2.
    int dev = 0, l2 = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev);
    const double per_layer = 4.0 * H * K * es;
    G = static_cast<int>((0.55 * l2) / per_layer);
    G = std::max(1, std::min(G, D));
    if (per_layer * D <= 0.55 * l2) G = D;
  }
  G = std::min(G, D);

  const int n_cells = D * L;
  const PlanLayout lay = plan_layout(n_cells, stacked_max_tiles_per_cell(N, H));
  if (dtype == FTB_F32 && schedule != 1 && (schedule >= 2 || workspace_bytes >= lay.total)) {
    // fp32: one persistent launch, a CTA per accumulator tile with its weights in shared memory
    // (csrc/lstm_simt_static.cu), when a layer's tiles fit on the device.
    if (workspace_bytes < lay.total) return FTB_ERR_WORKSPACE;
    const bool can = lstm_simt_static_supported(D, N, I, H, cl.sm_count);
    if (schedule >= 2 && !can) return FTB_ERR_ARG;
    if (can) {
      rc = launch_lstm_simt_static(static_cast<const float*>(x), static_cast<const float*>(Wp), bias_p,
                                   static_cast<float*>(hs), c, D, L, N, I, H,
                                   reinterpret_cast<int*>(static_cast<char*>(workspace) + lay.done), status,
                                   cl.sm_count, stream);
      // A refused cooperative launch falls back to one launch per level under the automatic choice.
      if (rc != FTB_ERR_LAUNCH || schedule != 0) return rc;
    }
  }
  const bool persistent = dtype != FTB_F32 && schedule != 1 && (schedule >= 2 || workspace_bytes >= lay.total);
  if (persistent) {
    if (workspace_bytes < lay.total) return FTB_ERR_WORKSPACE;
    char* ws = static_cast<char*>(workspace);
    // Static tile ownership (schedule 3, and the automatic choice when it applies): CTA pairs
    // keep their slice of a layer, cell state in registers, for a whole sweep over time.
    // Weights-major static ownership (schedule 4, and the automatic choice for batches of at most
    // 128 sequences): the batch is the N side of the MMA, so a small batch wastes no tensor work.
    const bool can_wmajor = lstm_wmajor_supported(dtype, D, N, I, H, G, cl.sm_count);
    if (schedule == 4 && !can_wmajor) return FTB_ERR_ARG;
    if (schedule == 4 || (schedule == 0 && can_wmajor && tune.pair == 0 && bn == 0 && !tune.fine_deps)) {
      // tuning[6]: 0 = as many recurrent weight blocks on chip as fit, -1 = none, n = n blocks
      const int resident = tune.resident == 0 ? -1 : (tune.resident < 0 ? 0 : tune.resident);
      unsigned long long* trace = nullptr;
#ifdef FTB_TRACE
      trace = reinterpret_cast<unsigned long long*>(ws + lay.trace);
#endif
      // one flag per (cell, tile), in the per-tile counter area (at least 4H/128 ints per cell)
      rc = launch_lstm_wmajor(dtype, x, Wp, bias_p, hs, c, D, L, N, I, H, G, resident,
                              reinterpret_cast<int*>(ws + lay.tile_done), status, trace, stream);
      if (rc != FTB_ERR_LAUNCH || schedule != 0) return rc;
      goto level_schedule;
    }
    const bool can_static = tune.pair != 1 && (bn == 0 || bn == 256) && !tune.fine_deps &&
                            lstm_static_supported(dtype, D, N, I, H, G, cl.sm_count);
    if (schedule == 3 && !can_static) return FTB_ERR_ARG;
    if ((schedule == 3 || schedule == 0) && can_static) {
      unsigned long long* trace = nullptr;
#ifdef FTB_TRACE
      trace = reinterpret_cast<unsigned long long*>(ws + lay.trace);
#endif
      rc = launch_lstm_static(dtype, x, Wp, bias_p, hs, c, D, L, N, I, H, G,
                              reinterpret_cast<int*>(ws + lay.done), status, trace, stream);
      // A cooperative launch can be refused (device shared through MPS, SMs reserved, ...).
      // With an explicit schedule that is the caller's error to see; the automatic choice
      // falls back to one launch per level, which needs no co-residency.
      if (rc != FTB_ERR_LAUNCH || schedule != 0) return rc;
      goto level_schedule;
    }
    StackedPlanArgs pa;
    pa.D = D; pa.L = L; pa.N = N; pa.I = I; pa.H = H; pa.G = G; pa.es = static_cast<int>(es);
    pa.skew = skew > 0 ? skew : 1;
    pa.m_tiles = cl.m_tiles_for(N);
    pa.tiles_per_item = pa.m_tiles * ((4 * H + cl.bn - 1) / cl.bn);
    pa.hs = static_cast<char*>(hs);
    pa.c = c;
    pa.bias_p = bias_p;
    pa.items = reinterpret_cast<CellItem*>(ws + lay.items);
    pa.dep = reinterpret_cast<int32_t*>(ws + lay.dep);
    pa.target = reinterpret_cast<int32_t*>(ws + lay.target);
    int32_t* done = reinterpret_cast<int32_t*>(ws + lay.done);
    if (cudaMemsetAsync(done, 0, lay.counters_end - lay.done, stream) != cudaSuccess) return FTB_ERR_LAUNCH;
    plan_stacked_kernel<<<(n_cells + 127) / 128, 128, 0, stream>>>(pa);
    if (cudaGetLastError() != cudaSuccess) return FTB_ERR_LAUNCH;
    count_launch();
    CellBatch header;
    header.n_items = n_cells;
    header.n_cols = 4 * H;
    header.ld_out = H;
    header.ld_c = H;
    header.total_tiles = n_cells * pa.tiles_per_item;
    header.pad_ = 0;
    PlanView pv = {pa.items, pa.dep, pa.target, done, reinterpret_cast<int32_t*>(ws + lay.tile_done),
                   reinterpret_cast<int32_t*>(ws + lay.c_done), tune.fine_deps == 1 ? 1 : 0, cl.bn / 4,
                   pa.tiles_per_item, 0, nullptr, nullptr};
#ifdef FTB_TRACE
    pv.trace = reinterpret_cast<unsigned long long*>(ws + lay.trace);
#endif
    rc = launch_cell_gemm_persistent(dtype, EPI_LSTM, cl.bn, cl.pair, cl.maps, cl.mapW, cl.mapC, header, pv,
                                     status, cl.sm_count, stream);
    if (rc != FTB_ERR_LAUNCH || schedule != 0) return rc;
  }

level_schedule:
  std::vector<CellItem> items;
  for (int g0 = 0; g0 < D; g0 += G) {
    const int Lg = std::min(G, D - g0);
    for (int m = 0; m < Lg + L - 1; ++m) {
      items.clear();
      for (int l = g0; l < g0 + Lg; ++l) {
        const int t = m - (l - g0);
        if (t < 0 || t >= L) continue;
        CellItem it = blank_item();
        if (l == 0)
          add_seg(it, 0, static_cast<int64_t>(t) * N, I, 0);
        else
          add_seg(it, 1, (static_cast<int64_t>(l - 1) * L + t) * N, H, 0);
        if (t > 0) add_seg(it, 2, (static_cast<int64_t>(l) * L + t - 1) * N, H, I);
        it.w_row0 = l * 4 * H;
        it.rows = N;
        it.c_zero = (t == 0);
        it.out = static_cast<char*>(hs) + (static_cast<size_t>(l) * L + t) * N * H * es;
        it.out_row0 = static_cast<int32_t>((static_cast<int64_t>(l) * L + t) * N);
        it.out_map = 1;
        it.c = c + static_cast<size_t>(l) * N * H;
        it.c_row0 = l * N;
        it.bias = bias_p ? bias_p + static_cast<size_t>(l) * 4 * H : nullptr;
        items.push_back(it);
      }
      rc = cl.run(items);
      if (rc) return rc;
    }
  }
  return FTB_OK;
}

int ftb_lstm_stacked_varlen_fwd(const void* x, const void* Wp, const float* bias_p, void* hs, float* c,
                                const int* active_rows, int D, int L, int I, int H, int dtype, const int* tuning,
                                void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const Tuning tune(tuning);
  if (!x || !Wp || !hs || !c || !active_rows || D <= 0 || L <= 0 || !valid_dtype(dtype)) return FTB_ERR_ARG;
  if (H <= 0 || I <= 0 || H % 64 != 0 || I % 64 != 0) return FTB_ERR_ARG;
  if (D > 1 && I != H) return FTB_ERR_ARG;
  // Row offset of every step in the packed buffers; the batch must be sorted by decreasing length.
  std::vector<int64_t> off(L + 1, 0);
  for (int t = 0; t < L; ++t) {
    if (active_rows[t] <= 0 || (t > 0 && active_rows[t] > active_rows[t - 1])) return FTB_ERR_ARG;
    off[t + 1] = off[t] + active_rows[t];
  }
  const int64_t T = off[L];
  const int N = active_rows[0];
  if (static_cast<int64_t>(D) * T > 0x7fffffffLL) return FTB_ERR_ARG;
  if (!aligned16({x, Wp, bias_p, hs, c})) return FTB_ERR_ALIGN;
  int* status = nullptr;
  int rc = begin_call(workspace, workspace_bytes, stream, &status);
  if (rc) return rc;

  const int K = I + H;
  const size_t es = dtype_size(dtype);
  CellLauncher cl;
  cl.dtype = dtype;
  cl.epi = EPI_LSTM;
  cl.n_cols = 4 * H;
  cl.ld_out = H;
  cl.ld_c = H;
  cl.status = status;
  cl.stream = stream;
  cl.sm_count = current_sm_count();
  if (dtype == FTB_F32) {
    cl.act[0] = static_cast<const float*>(x);
    cl.ld_act[0] = I;
    cl.act[1] = cl.act[2] = static_cast<const float*>(hs);
    cl.ld_act[1] = cl.ld_act[2] = H;
    cl.w = static_cast<const float*>(Wp);
    cl.ldw = K;
  } else {
    cl.bn = pick_bn(4 * H, tune.bn);
    if (cl.bn == 0) return FTB_ERR_ARG;
    cl.pair = tune.use_pair(N);
    rc = make_tmap_2d(&cl.maps[0], x, dtype, static_cast<uint64_t>(T), I, I, 128, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.maps[1], hs, dtype, static_cast<uint64_t>(D) * T, H, H, 128, 64);
    if (rc) return rc;
    cl.maps[2] = cl.maps[1];
    cl.maps[3] = cl.maps[0];
    rc = make_tmap_2d(&cl.mapW, Wp, dtype, static_cast<uint64_t>(D) * 4 * H, K, K, cl.w_box_rows(), 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.mapC, c, FTB_F32, static_cast<uint64_t>(D) * N, H, H, 128, 32);
    if (rc) return rc;
  }

  // Layers run in groups whose packed weights stay in L2, as in the rectangular entry point.
  int G = tune.layers_per_group;
  if (G <= 0) {
    int dev = 0, l2 = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev);
    const double per_layer = 4.0 * H * K * es;
    G = static_cast<int>((0.55 * l2) / per_layer);
    G = std::max(1, G);
  }
  G = std::min(G, D);

  // Cell (l, t) holds the active_rows[t] sequences still running: it reads the layer below (or
  // x) at step t and the first active_rows[t] rows of its own layer's step t-1.
  auto make_item = [&](int l, int t) {
    CellItem it = blank_item();
    if (l == 0)
      add_seg(it, 0, off[t], I, 0);
    else
      add_seg(it, 1, static_cast<int64_t>(l - 1) * T + off[t], H, 0);
    if (t > 0) add_seg(it, 2, static_cast<int64_t>(l) * T + off[t - 1], H, I);
    it.w_row0 = l * 4 * H;
    it.rows = active_rows[t];
    it.c_zero = (t == 0);
    it.out = static_cast<char*>(hs) + (static_cast<size_t>(l) * T + off[t]) * H * es;
    it.out_row0 = static_cast<int32_t>(static_cast<int64_t>(l) * T + off[t]);
    it.out_map = 1;
    it.c = c + static_cast<size_t>(l) * N * H;
    it.c_row0 = l * N;
    it.bias = bias_p ? bias_p + static_cast<size_t>(l) * 4 * H : nullptr;
    return it;
  };

  const int n_cells = D * L;
  const PlanLayout lay = plan_layout(n_cells, 0);
  bool persistent = dtype != FTB_F32 && tune.schedule != 1 && (tune.schedule >= 2 || workspace_bytes >= lay.total);
  if (persistent) {
    if (workspace_bytes < lay.total) return FTB_ERR_WORKSPACE;
    // One persistent launch over the steps [t0, t1) of every layer.  Launch order: group by
    // group, level by level (level = layer-in-group + step), so every cell comes after the two
    // it reads; cells of earlier steps belong to an earlier launch on the stream and count as
    // inputs.
    auto run_range = [&](const CellLauncher& launcher, int t0, int t1) -> int {
      const int Lr = t1 - t0;
      std::vector<CellItem> order;
      order.reserve(static_cast<size_t>(D) * Lr);
      std::vector<int> index_of(static_cast<size_t>(D) * Lr, -1);
      for (int g0 = 0; g0 < D; g0 += G) {
        const int Lg = std::min(G, D - g0);
        for (int m = 0; m < Lg + Lr - 1; ++m)
          for (int l = g0; l < g0 + Lg; ++l) {
            const int t = m - (l - g0);
            if (t < 0 || t >= Lr) continue;
            index_of[l * Lr + t] = static_cast<int>(order.size());
            order.push_back(make_item(l, t0 + t));
          }
      }
      std::vector<int32_t> deps(order.size() * kMaxSeg * 2, -1);
      for (int l = 0; l < D; ++l)
        for (int t = 0; t < Lr; ++t) {
          const int me = index_of[l * Lr + t];
          if (l > 0)
            deps[(me * kMaxSeg + 0) * 2 + 0] = deps[(me * kMaxSeg + 0) * 2 + 1] = index_of[(l - 1) * Lr + t];
          if (t > 0) deps[(me * kMaxSeg + 1) * 2 + 0] = deps[(me * kMaxSeg + 1) * 2 + 1] = index_of[l * Lr + t - 1];
        }
      return run_persistent(launcher, order, deps, static_cast<char*>(workspace), lay, workspace_bytes);
    };
    // Once the batch has shrunk to one 128-row tile, a CTA pair would multiply 128 rows of
    // padding with every weight tile.  From that step on the cells run as single CTAs on
    // 128-column tiles (same bytes per CTA and K block, half the tensor work, twice the tiles):
    // the time axis is cut there into two launches.  Only when the caller left the tile shape open.
    int t_split = L;
    if (cl.pair && tune.pair == 0 && tune.bn == 0 && tune.schedule == 0)
      for (int t = 0; t < L; ++t)
        if (active_rows[t] <= 128) {
          t_split = t;
          break;
        }
    rc = FTB_OK;
    if (t_split > 0) rc = run_range(cl, 0, t_split);
    if (rc == FTB_OK && t_split < L) {
      CellLauncher single = cl;
      single.pair = 0;
      single.bn = 128;
      rc = make_tmap_2d(&single.mapW, Wp, dtype, static_cast<uint64_t>(D) * 4 * H, K, K, single.w_box_rows(), 64);
      if (rc) return rc;
      rc = run_range(single, t_split, L);
    }
    if (rc != FTB_ERR_LAUNCH || tune.schedule != 0) return rc;
    // A refused cooperative launch falls back to one launch per level (which recomputes every cell).
  }

  std::vector<CellItem> items;
  for (int g0 = 0; g0 < D; g0 += G) {
    const int Lg = std::min(G, D - g0);
    for (int m = 0; m < Lg + L - 1; ++m) {
      items.clear();
      for (int l = g0; l < g0 + Lg; ++l) {
        const int t = m - (l - g0);
        if (t < 0 || t >= L) continue;
        items.push_back(make_item(l, t));
      }
      rc = cl.run(items);
      if (rc) return rc;
    }
  }
  return FTB_OK;
}

size_t ftb_lstm_stacked_varlen_workspace_bytes(int D, int L) {
  if (D <= 0 || L <= 0) return kWorkspaceBytes;
  return plan_layout(D * L, 0).total;
}

int ftb_lstm_dilated_fwd(const void* x, const void* Wp, const float* bias_p, void* hs, float* c,
                         const int* dilations, int D, int L, int N, int H, int dtype, const int* tuning,
                         void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const Tuning tune(tuning);
  const int bn = tune.bn;
  if (!x || !Wp || !hs || !c || !dilations || D <= 0 || L <= 0 || N <= 0 || !valid_dtype(dtype)) return FTB_ERR_ARG;
  if (H <= 0 || H % 64 != 0) return FTB_ERR_ARG;
  int max_dil = 1;
  for (int l = 0; l < D; ++l) {
    if (dilations[l] <= 0) return FTB_ERR_ARG;
    max_dil = std::max(max_dil, dilations[l]);
  }
  if (static_cast<int64_t>(D) * L * N > 0x7fffffffLL) return FTB_ERR_ARG;
  if (!aligned16({x, Wp, bias_p, hs, c})) return FTB_ERR_ALIGN;
  int* status = nullptr;
  int rc = begin_call(workspace, workspace_bytes, stream, &status);
  if (rc) return rc;

  const int K = 2 * H;
  const size_t es = dtype_size(dtype);
  CellLauncher cl;
  cl.dtype = dtype;
  cl.epi = EPI_LSTM;
  cl.n_cols = 4 * H;
  cl.ld_out = H;
  cl.ld_c = H;
  cl.status = status;
  cl.stream = stream;
  cl.sm_count = current_sm_count();
  if (dtype == FTB_F32) {
    cl.act[0] = static_cast<const float*>(x);
    cl.act[1] = cl.act[2] = static_cast<const float*>(hs);
    cl.ld_act[0] = cl.ld_act[1] = cl.ld_act[2] = H;
    cl.w = static_cast<const float*>(Wp);
    cl.ldw = K;
  } else {
    cl.bn = pick_bn(4 * H, bn);
    if (cl.bn == 0) return FTB_ERR_ARG;
    cl.pair = tune.pair == 2;  // cells here are latency-bound: single CTAs measured faster than pairs
    rc = make_tmap_2d(&cl.maps[0], x, dtype, static_cast<uint64_t>(L) * N, H, H, 128, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.maps[1], hs, dtype, static_cast<uint64_t>(D) * L * N, H, H, 128, 64);
    if (rc) return rc;
    cl.maps[2] = cl.maps[1];
    cl.maps[3] = cl.maps[0];
    rc = make_tmap_2d(&cl.mapW, Wp, dtype, static_cast<uint64_t>(D) * 4 * H, K, K, cl.w_box_rows(), 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.mapC, c, FTB_F32, static_cast<uint64_t>(D) * max_dil * N, H, H, 128, 32);
    if (rc) return rc;
  }

  // Cluster schedule (schedule 4, and the automatic choice when it applies): one thread-block
  // cluster per (layer, batch slice), weights resident in tensor memory, the state of a layer with
  // dilation 1 handed on through the cluster's shared memory.  Its flags sit behind the tables of
  // the generic persistent schedule in the workspace.
  {
    const size_t flags_off = plan_layout(D * L, 0).total;
    const size_t need = flags_off + sizeof(int) * lstm_dilated_cluster_flag_ints(D, L);
    const bool can = lstm_dilated_cluster_supported(dtype, D, N, H, cl.sm_count) && tune.pair == 0 && bn == 0;
    if (tune.schedule == 4 && (!can || workspace_bytes < need)) return can ? FTB_ERR_WORKSPACE : FTB_ERR_ARG;
    if ((tune.schedule == 4 || tune.schedule == 0) && can && workspace_bytes >= need) {
      rc = launch_lstm_dilated_cluster(dtype, x, Wp, bias_p, hs, c, dilations, D, L, N, H,
                                       reinterpret_cast<int*>(static_cast<char*>(workspace) + flags_off), status,
                                       stream);
      // a refused cooperative cluster launch falls back to the generic wavefront
      if (rc != FTB_ERR_LAUNCH || tune.schedule != 0) return rc;
    }
  }

  // Layer l advances in steps of dilations[l] consecutive timesteps: those
  // timesteps only depend on the step before (same layer) and on the layer
  // below, so one step is one cell of batch dilation*N.  Earliest-start levels.
  std::map<int, std::vector<CellItem>> levels;
  std::map<int, std::vector<std::pair<int, int>>> level_ids;  // (layer, step) of each item, same order
  std::vector<std::vector<int>> level_of(D);
  for (int l = 0; l < D; ++l) {
    const int dl = dilations[l];
    const int steps = (L + dl - 1) / dl;
    level_of[l].resize(steps);
    for (int s = 0; s < steps; ++s) {
      const int t0 = s * dl;
      const int t1 = std::min(L, t0 + dl);
      int lv = 0;
      if (s > 0) lv = level_of[l][s - 1] + 1;
      if (l > 0) {
        const int below = (t1 - 1) / dilations[l - 1];
        lv = std::max(lv, level_of[l - 1][below] + 1);
      }
      level_of[l][s] = lv;
      CellItem it = blank_item();
      if (l == 0)
        add_seg(it, 0, static_cast<int64_t>(t0) * N, H, 0);
      else
        add_seg(it, 1, (static_cast<int64_t>(l - 1) * L + t0) * N, H, 0);
      if (s > 0) add_seg(it, 2, (static_cast<int64_t>(l) * L + t0 - dl) * N, H, H);
      it.w_row0 = l * 4 * H;
      it.rows = (t1 - t0) * N;
      it.c_zero = (s == 0);
      it.out = static_cast<char*>(hs) + (static_cast<size_t>(l) * L + t0) * N * H * es;
      it.out_row0 = static_cast<int32_t>((static_cast<int64_t>(l) * L + t0) * N);
      it.out_map = 1;
      it.c = c + static_cast<size_t>(l) * max_dil * N * H;
      it.c_row0 = l * max_dil * N;
      it.bias = bias_p ? bias_p + static_cast<size_t>(l) * 4 * H : nullptr;
      levels[lv].push_back(it);
      level_ids[lv].push_back(std::make_pair(l, s));
    }
  }
  int n_items = 0;
  for (auto& kv : levels) n_items += static_cast<int>(kv.second.size());
  const PlanLayout lay = plan_layout(n_items, 0);
  const bool persistent = dtype != FTB_F32 && tune.schedule != 1 && (tune.schedule >= 2 || workspace_bytes >= lay.total);
  if (persistent) {
    if (workspace_bytes < lay.total) return FTB_ERR_WORKSPACE;
    // Launch order = level order.  A step of layer l reads the layer below up to the step that
    // holds its last timestep (the steps of a layer complete in order, so waiting for that one
    // is enough) and the step before it in its own layer.
    std::vector<CellItem> order;
    std::vector<std::vector<int>> index_of(D);
    for (int l = 0; l < D; ++l) index_of[l].resize(level_of[l].size());
    for (auto& kv : levels)
      for (size_t i = 0; i < kv.second.size(); ++i) {
        const std::pair<int, int> id = level_ids[kv.first][i];
        index_of[id.first][id.second] = static_cast<int>(order.size());
        order.push_back(kv.second[i]);
      }
    std::vector<int32_t> deps(static_cast<size_t>(n_items) * kMaxSeg * 2, -1);
    for (int l = 0; l < D; ++l)
      for (size_t s = 0; s < index_of[l].size(); ++s) {
        const int me = index_of[l][s];
        const int dl = dilations[l];
        const int t1 = std::min(L, static_cast<int>(s + 1) * dl);
        if (l > 0) {
          const int below = index_of[l - 1][(t1 - 1) / dilations[l - 1]];
          deps[(me * kMaxSeg + 0) * 2 + 0] = deps[(me * kMaxSeg + 0) * 2 + 1] = below;
        }
        if (s > 0) {
          const int prev = index_of[l][s - 1];
          deps[(me * kMaxSeg + 1) * 2 + 0] = deps[(me * kMaxSeg + 1) * 2 + 1] = prev;
        }
      }
    rc = run_persistent(cl, order, deps, static_cast<char*>(workspace), lay, workspace_bytes);
    // A refused cooperative launch falls back to one launch per level, as in the other entries;
    // an explicitly requested persistent schedule reports the refusal.
    if (rc != FTB_ERR_LAUNCH || tune.schedule != 0) return rc;
  }
  for (auto& kv : levels) {
    rc = cl.run(kv.second);
    if (rc) return rc;
  }
  return FTB_OK;
}

size_t ftb_lstm_dilated_workspace_bytes(int D, int L) {
  if (D <= 0 || L <= 0) return kWorkspaceBytes;
  // tables of the generic persistent schedule, then the flags of the cluster schedule
  return plan_layout(D * L, 0).total + sizeof(int) * lstm_dilated_cluster_flag_ints(D, L);
}

int ftb_grid_rnn_fwd(const void* X, const void* Y, const void* Wpx, const void* Wpy, const float* bias_x,
                     const float* bias_y, void* hx, void* hy, int D, int A, int B, int N, int H, int dtype,
                     void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!X || !Y || !Wpx || !Wpy || !hx || !hy || D <= 0 || A <= 0 || B <= 0 || N <= 0 || !valid_dtype(dtype))
    return FTB_ERR_ARG;
  if (H <= 0 || H % 64 != 0) return FTB_ERR_ARG;
  if (static_cast<int64_t>(D) * A * B * N > 0x7fffffffLL) return FTB_ERR_ARG;
  if (!aligned16({X, Y, Wpx, Wpy, bias_x, bias_y, hx, hy})) return FTB_ERR_ALIGN;
  int* status = nullptr;
  int rc = begin_call(workspace, workspace_bytes, stream, &status);
  if (rc) return rc;

  const int K = 3 * H;
  const size_t es = dtype_size(dtype);
  // One launch context for both directions: activation buffers 0..3 = X, Y, hx, hy; weight
  // buffer 0 = direction x, 1 = direction y.  Direction x reads (hx | hy | X or hx below),
  // direction y reads (hx | hy | Y or hy below).
  CellLauncher cl;
  cl.dtype = dtype;
  cl.epi = EPI_TANH;
  cl.n_cols = H;
  cl.ld_out = H;
  cl.ld_c = H;
  cl.status = status;
  cl.stream = stream;
  cl.sm_count = current_sm_count();
  if (dtype == FTB_F32) {
    cl.act[0] = static_cast<const float*>(X);
    cl.act[1] = static_cast<const float*>(Y);
    cl.act[2] = static_cast<const float*>(hx);
    cl.act[3] = static_cast<const float*>(hy);
    cl.ld_act[0] = cl.ld_act[1] = cl.ld_act[2] = cl.ld_act[3] = H;
    cl.w = static_cast<const float*>(Wpx);
    cl.w2 = static_cast<const float*>(Wpy);
    cl.ldw = K;
  } else {
    cl.bn = pick_bn(H, 128);
    if (cl.bn == 0) return FTB_ERR_ARG;
    const uint64_t grid_rows = static_cast<uint64_t>(A) * B * N;
    rc = make_tmap_2d(&cl.maps[0], X, dtype, grid_rows, H, H, 128, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.maps[1], Y, dtype, grid_rows, H, H, 128, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.maps[2], hx, dtype, grid_rows * D, H, H, 128, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.maps[3], hy, dtype, grid_rows * D, H, H, 128, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.mapW, Wpx, dtype, static_cast<uint64_t>(D) * H, K, K, cl.bn, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.mapC, Wpy, dtype, static_cast<uint64_t>(D) * H, K, K, cl.bn, 64);
    if (rc) return rc;
  }

  // Cell (d, a, b) of direction dirn, and which earlier cell each of its K segments reads
  // (-1: an input of the call).  Anti-diagonal level = d + a + b.
  auto cell_index = [&](int d, int a, int b) { return (static_cast<int64_t>(d) * A + a) * B + b; };
  auto make_item = [&](int d, int a, int b, int dirn, int64_t (&src)[kMaxSeg]) {
    CellItem it = blank_item();
    const int64_t cell = cell_index(d, a, b);
    for (int s = 0; s < kMaxSeg; ++s) src[s] = -1;
    // The cell's own input first: it is an input of the call (layer 0) or was finished two
    // levels ago, so its K blocks run while the two neighbours of the previous level finish.
    if (d == 0) {
      add_seg(it, dirn, (static_cast<int64_t>(a) * B + b) * N, H, 2 * H);
    } else {
      src[it.nseg] = cell_index(d - 1, a, b) * 2 + dirn;
      add_seg(it, 2 + dirn, cell_index(d - 1, a, b) * N, H, 2 * H);
    }
    if (a > 0) {
      src[it.nseg] = cell_index(d, a - 1, b) * 2 + 0;
      add_seg(it, 2, cell_index(d, a - 1, b) * N, H, 0);
    }
    if (b > 0) {
      src[it.nseg] = (cell - 1) * 2 + 1;
      add_seg(it, 3, (cell - 1) * N, H, H);
    }
    it.w_row0 = d * H;
    it.w_map = dirn;
    it.rows = N;
    it.out = static_cast<char*>(dirn == 0 ? hx : hy) + static_cast<size_t>(cell) * N * H * es;
    const float* bias = dirn == 0 ? bias_x : bias_y;
    it.bias = bias ? bias + static_cast<size_t>(d) * H : nullptr;
    return it;
  };

  const int n_items = 2 * D * A * B;
  const int levels = (D - 1) + (A - 1) + (B - 1) + 1;
  const PlanLayout lay = plan_layout(n_items, 0);
  // Cluster schedule (the choice when it applies and the workspace has room for its flags behind the
  // tables): one thread-block cluster per grid row and batch slice, weights resident in tensor
  // memory, h_y handed to the next column through the cluster's shared memory.
  if (grid_rnn_cluster_supported(dtype, D, A, B, N, H, cl.sm_count) &&
      workspace_bytes >= ftb_grid_rnn_workspace_bytes(D, A, B)) {
    rc = launch_grid_rnn_cluster(dtype, X, Y, Wpx, Wpy, bias_x, bias_y, hx, hy, D, A, B, N, H,
                                 reinterpret_cast<int*>(static_cast<char*>(workspace) + lay.total), status, stream);
    if (rc != FTB_ERR_LAUNCH) return rc;  // a refused cooperative cluster launch falls back to the generic wavefront
  }
  const bool persistent = dtype != FTB_F32 && workspace_bytes >= lay.total;
  if (persistent) {
    // One cooperative launch for the whole grid: items in level order, each K segment waiting
    // for the one earlier cell it reads.
    std::vector<CellItem> order;
    order.reserve(n_items);
    std::vector<int> index_of(n_items, -1);
    std::vector<int64_t> srcs;
    srcs.reserve(static_cast<size_t>(n_items) * kMaxSeg);
    for (int m = 0; m < levels; ++m)
      for (int d = 0; d < D; ++d)
        for (int a = 0; a < A; ++a) {
          const int b = m - d - a;
          if (b < 0 || b >= B) continue;
          for (int dirn = 0; dirn < 2; ++dirn) {
            int64_t src[kMaxSeg];
            index_of[cell_index(d, a, b) * 2 + dirn] = static_cast<int>(order.size());
            order.push_back(make_item(d, a, b, dirn, src));
            for (int s = 0; s < kMaxSeg; ++s) srcs.push_back(src[s]);
          }
        }
    std::vector<int32_t> deps(static_cast<size_t>(n_items) * kMaxSeg * 2, -1);
    for (int i = 0; i < n_items; ++i)
      for (int s = 0; s < kMaxSeg; ++s) {
        const int64_t src = srcs[static_cast<size_t>(i) * kMaxSeg + s];
        if (src >= 0) deps[(i * kMaxSeg + s) * 2 + 0] = deps[(i * kMaxSeg + s) * 2 + 1] = index_of[src];
      }
    rc = run_persistent(cl, order, deps, static_cast<char*>(workspace), lay, workspace_bytes);
    if (rc != FTB_ERR_LAUNCH) return rc;  // a refused cooperative launch falls back to levels
  }

  std::vector<CellItem> items;
  for (int m = 0; m < levels; ++m) {
    items.clear();
    for (int d = 0; d < D; ++d)
      for (int a = 0; a < A; ++a) {
        const int b = m - d - a;
        if (b < 0 || b >= B) continue;
        for (int dirn = 0; dirn < 2; ++dirn) {
          int64_t src[kMaxSeg];
          items.push_back(make_item(d, a, b, dirn, src));
        }
      }
    rc = cl.run(items);
    if (rc) return rc;
  }
  return FTB_OK;
}

int ftb_rnn_pack_weights(const void* W, const void* U, void* Wp, int I, int H, int dtype, void* stream) {
  if (!W || !U || !Wp || I <= 0 || H <= 0 || !valid_dtype(dtype)) return FTB_ERR_ARG;
  return pack_rnn(W, U, Wp, I, H, dtype, static_cast<cudaStream_t>(stream));
}

int ftb_rnn_attention_fwd(const void* src, const void* trg, const void* Wp_src, const void* Wp_trg,
                          const float* bias_src, const float* bias_trg, const void* enc_proj, const void* dec_proj,
                          const int* src_lens, void* enc, float* enc_scores, void* dec, void* out, int Ls, int Lt,
                          int N, int H, int dtype, void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!src || !trg || !Wp_src || !Wp_trg || !enc_proj || !dec_proj || !enc || !enc_scores || !dec || !out)
    return FTB_ERR_ARG;
  if (Ls <= 0 || Lt <= 0 || N <= 0 || H <= 0 || H % 64 != 0 || !valid_dtype(dtype)) return FTB_ERR_ARG;
  if (Ls > rnn_attention_max_src_len()) return FTB_ERR_ARG;
  if (static_cast<int64_t>(std::max(Ls, Lt)) * N > 0x7fffffffLL) return FTB_ERR_ARG;
  if (!aligned16({src, trg, Wp_src, Wp_trg, bias_src, bias_trg, enc, dec, out})) return FTB_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(enc_scores) & 3) != 0 || (reinterpret_cast<uintptr_t>(src_lens) & 3) != 0)
    return FTB_ERR_ALIGN;
  int* status = nullptr;
  int rc = begin_call(workspace, workspace_bytes, stream, &status);
  if (rc) return rc;

  const int K = 2 * H;
  const size_t es = dtype_size(dtype);
  // One launch context for both cells: activation buffers 0..3 = src, trg, enc, out (the attention
  // vectors, which are the decoder's recurrent input); weight buffer 0 = encoder, 1 = decoder.
  CellLauncher cl;
  cl.dtype = dtype;
  cl.epi = EPI_TANH;
  cl.n_cols = H;
  cl.ld_out = H;
  cl.ld_c = H;
  cl.status = status;
  cl.stream = stream;
  cl.sm_count = current_sm_count();
  if (dtype == FTB_F32) {
    cl.act[0] = static_cast<const float*>(src);
    cl.act[1] = static_cast<const float*>(trg);
    cl.act[2] = static_cast<const float*>(enc);
    cl.act[3] = static_cast<const float*>(out);
    cl.ld_act[0] = cl.ld_act[1] = cl.ld_act[2] = cl.ld_act[3] = H;
    cl.w = static_cast<const float*>(Wp_src);
    cl.w2 = static_cast<const float*>(Wp_trg);
    cl.ldw = K;
  } else {
    cl.bn = pick_bn(H, 128);
    if (cl.bn == 0) return FTB_ERR_ARG;
    const uint64_t src_rows = static_cast<uint64_t>(Ls) * N, trg_rows = static_cast<uint64_t>(Lt) * N;
    rc = make_tmap_2d(&cl.maps[0], src, dtype, src_rows, H, H, 128, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.maps[1], trg, dtype, trg_rows, H, H, 128, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.maps[2], enc, dtype, src_rows, H, H, 128, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.maps[3], out, dtype, trg_rows, H, H, 128, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.mapW, Wp_src, dtype, H, K, K, cl.bn, 64);
    if (rc) return rc;
    rc = make_tmap_2d(&cl.mapC, Wp_trg, dtype, H, K, K, cl.bn, 64);
    if (rc) return rc;
  }

  std::vector<CellItem> items(1);
  // Encoder: e_j = tanh(x_j W + e_{j-1} U + b), one level per source position.
  for (int j = 0; j < Ls; ++j) {
    CellItem it = blank_item();
    add_seg(it, 0, static_cast<int64_t>(j) * N, H, 0);
    if (j > 0) add_seg(it, 2, static_cast<int64_t>(j - 1) * N, H, H);
    it.rows = N;
    it.w_map = 0;
    it.bias = bias_src;
    it.out = static_cast<char*>(enc) + static_cast<size_t>(j) * N * H * es;
    items[0] = it;
    rc = cl.run(items);
    if (rc) return rc;
  }
  rc = launch_enc_scores(dtype, enc, enc_proj, enc_scores, static_cast<long long>(Ls) * N, H, stream);
  if (rc) return rc;
  // Decoder: the cell, then the attention over the encoder rows; its result is both the step's
  // output and the next step's recurrent input.
  for (int t = 0; t < Lt; ++t) {
    CellItem it = blank_item();
    add_seg(it, 1, static_cast<int64_t>(t) * N, H, 0);
    if (t > 0) add_seg(it, 3, static_cast<int64_t>(t - 1) * N, H, H);
    it.rows = N;
    it.w_map = 1;
    it.bias = bias_trg;
    char* dec_t = static_cast<char*>(dec) + static_cast<size_t>(t) * N * H * es;
    it.out = dec_t;
    items[0] = it;
    rc = cl.run(items);
    if (rc) return rc;
    rc = launch_attn_step(dtype, enc, enc_scores, dec_t, dec_proj, src_lens,
                          static_cast<char*>(out) + static_cast<size_t>(t) * N * H * es, Ls, N, H, stream);
    if (rc) return rc;
  }
  return FTB_OK;
}

size_t ftb_grid_rnn_tables_bytes(int D, int A, int B) {
  if (D <= 0 || A <= 0 || B <= 0) return kWorkspaceBytes;
  return plan_layout(2 * D * A * B, 0).total;
}

size_t ftb_grid_rnn_workspace_bytes(int D, int A, int B) {
  if (D <= 0 || A <= 0 || B <= 0) return kWorkspaceBytes;
  // tables of the generic persistent schedule, then the flags of the cluster schedule: one per cell,
  // batch slice and CTA of a cluster; clusters x CTAs never exceed the SM count (taken as <= 256)
  const size_t per_column = std::max<size_t>(static_cast<size_t>(D) * A * 4, 256);
  return plan_layout(2 * D * A * B, 0).total + sizeof(int) * per_column * B;
}

int ftb_gemm_nt(const void* A, const void* Bt, void* out, int M, int N, int K, int dtype, const int* tuning,
                void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const Tuning tune(tuning);
  if (!A || !Bt || !out || M <= 0 || N <= 0 || K <= 0 || !valid_dtype(dtype)) return FTB_ERR_ARG;
  if (K % 64 != 0) return FTB_ERR_ARG;
  if (dtype == FTB_F32 ? (N % 64 != 0) : (N % 128 != 0)) return FTB_ERR_ARG;
  if (!aligned16({A, Bt, out})) return FTB_ERR_ALIGN;
  int* status = nullptr;
  int rc = begin_call(workspace, workspace_bytes, stream, &status);
  if (rc) return rc;
  CellLauncher cl;
  cl.dtype = dtype;
  cl.epi = EPI_STORE;
  cl.n_cols = N;
  cl.ld_out = N;
  cl.status = status;
  cl.stream = stream;
  cl.sm_count = current_sm_count();
  if (dtype == FTB_F32) {
    cl.act[0] = cl.act[1] = cl.act[2] = static_cast<const float*>(A);
    cl.ld_act[0] = cl.ld_act[1] = cl.ld_act[2] = K;
    cl.w = static_cast<const float*>(Bt);
    cl.ldw = K;
  } else {
    cl.bn = tune.bn ? tune.bn : ((N % 256 == 0) ? 256 : 128);
    if (cl.bn != 128 && cl.bn != 256) return FTB_ERR_ARG;
    cl.pair = tune.use_pair(M);
    rc = make_tmap_2d(&cl.maps[0], A, dtype, M, K, K, 128, 64);
    if (rc) return rc;
    cl.maps[1] = cl.maps[2] = cl.maps[3] = cl.maps[0];
    rc = make_tmap_2d(&cl.mapW, Bt, dtype, N, K, K, cl.w_box_rows(), 64);
    if (rc) return rc;
    cl.mapC = cl.maps[0];
  }
  std::vector<CellItem> items(1, blank_item());
  add_seg(items[0], 0, 0, K, 0);
  items[0].rows = M;
  items[0].out = out;
  return cl.run(items);
}

int ftb_projection_padded_cols(int V) { return V <= 0 ? 0 : ((V + 127) / 128) * 128; }

int ftb_projection_pack(const void* P, void* Pt, int H, int V, int dtype, void* stream) {
  if (!P || !Pt || H <= 0 || V <= 0 || (dtype != FTB_F16 && dtype != FTB_BF16)) return FTB_ERR_ARG;
  if (!aligned16({P, Pt})) return FTB_ERR_ALIGN;
  return pack_projection(P, Pt, H, V, ftb_projection_padded_cols(V), dtype, static_cast<cudaStream_t>(stream));
}

int ftb_lstm_project_softmax(const void* h, const void* Pt, float* probs, long long T, int V, int H, int dtype,
                             void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!h || !Pt || !probs || T <= 0 || T > 0x7fffffffLL || V <= 0 || H <= 0 || H % 64 != 0) return FTB_ERR_ARG;
  if (dtype != FTB_F16 && dtype != FTB_BF16) return FTB_ERR_ARG;
  if (V > 48 * 1024) return FTB_ERR_ARG;  // the softmax runs in place on rows that fit its on-chip row cache
  if (!aligned16({h, Pt, probs})) return FTB_ERR_ALIGN;
  const int Vp = ftb_projection_padded_cols(V);
  if (static_cast<int64_t>(T) * Vp > 0x7fffffffffLL) return FTB_ERR_ARG;
  int* status = nullptr;
  int rc = begin_call(workspace, workspace_bytes, stream, &status);
  if (rc) return rc;
  // 1. logits = h . Pt^T, fp32, written straight into `probs` (row stride Vp)
  CellLauncher cl;
  cl.dtype = dtype;
  cl.epi = EPI_STORE_F32;
  cl.n_cols = Vp;
  cl.ld_out = Vp;
  cl.status = status;
  cl.stream = stream;
  cl.sm_count = current_sm_count();
  cl.bn = (Vp % 256 == 0) ? 256 : 128;
  cl.pair = 0;
  rc = make_tmap_2d(&cl.maps[0], h, dtype, static_cast<uint64_t>(T), H, H, 128, 64);
  if (rc) return rc;
  cl.maps[1] = cl.maps[2] = cl.maps[3] = cl.maps[0];
  rc = make_tmap_2d(&cl.mapW, Pt, dtype, Vp, H, H, cl.w_box_rows(), 64);
  if (rc) return rc;
  cl.mapC = cl.maps[0];
  std::vector<CellItem> items(1, blank_item());
  add_seg(items[0], 0, 0, H, 0);
  items[0].rows = static_cast<int32_t>(T);
  items[0].out = probs;
  rc = cl.run(items);
  if (rc) return rc;
  // 2. softmax over the first V logits of every row, in place, one read and one write per logit
  return online_softmax_rows(probs, probs, static_cast<int>(T), V, Vp, stream);
}

// ------------------------------------------------------------------------------
// Stacked LSTM forward for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a
// forward pass: a real-time loop that must not enter the allocator, a
// plugin whose host application owns the allocator and hands out nothing but the
// input and output buffers, or a process whose memory pool is already carved up.
// ftb_lstm_stacked_fwd needs a caller-provided workspace for its schedule tables,
// completion counters and status word; this variant keeps that scratch in a
// fixed-size array that is part of the library image instead.
//
// Cost and limits: every GPU that loads the library holds FTB_STATIC_SCRATCH_BYTES
// of device memory for the array until the process exits.  Problems whose
// ftb_lstm_stacked_workspace_bytes(D, L, N, H) exceeds that size are rejected with
// FTB_ERR_SCRATCH_LIMIT.  Only the persistent schedule (16-bit dtypes) is offered.
// All calls on a device share the one array, and it keeps whatever the previous
// call left in it: each call re-zeroes the status word and the counters it uses on
// its stream before launching, so back-to-back calls on one stream are fine, but two
// calls whose kernels can overlap on the GPU (different streams, or different host
// threads) race on the tables and counters and must be serialised by the caller.
//
// The first call on each device resolves the array's device address
// (cudaGetSymbolAddress; the array's name is only a host-side handle, not an
// address a kernel could use) and caches it; make that first call outside any
// stream capture.
#define FTB_STATIC_SCRATCH_BYTES (4u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[FTB_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_scratch_mu;
void* g_static_scratch_ptr[64] = {};
}  // namespace

int ftb_lstm_stacked_fwd_noalloc(const void* x, const void* Wp, const float* bias_p, void* hs, float* c, int D,
                                 int L, int N, int I, int H, int dtype, const int* tuning, void** scratch_out,
                                 void* stream) {
  if (D <= 0 || L <= 0 || N <= 0 || H <= 0) return FTB_ERR_ARG;
  if (dtype != FTB_F16 && dtype != FTB_BF16) return FTB_ERR_ARG;
  if (ftb_lstm_stacked_workspace_bytes(D, L, N, H) > FTB_STATIC_SCRATCH_BYTES) return FTB_ERR_SCRATCH_LIMIT;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FTB_ERR_ARCH;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_scratch_mu);
    if (g_static_scratch_ptr[dev] == nullptr) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
        cudaGetLastError();
        return FTB_ERR_DRIVER;
      }
      g_static_scratch_ptr[dev] = p;
    }
    scratch = g_static_scratch_ptr[dev];
  }
  if (scratch_out != nullptr) *scratch_out = scratch;
  int t[FTB_TUNING_INTS] = {0, 0, 0, 0, 0, 0};
  if (tuning != nullptr)
    for (int i = 0; i < FTB_TUNING_INTS; ++i) t[i] = tuning[i];
  // A single-launch schedule: their host side builds nothing on the heap (the one-launch-per-level
  // schedule keeps its cell lists in std::vector).  2 = generic persistent kernel, 3 = static tile
  // ownership; anything else the caller asked for becomes 2.
  if (t[2] != 3) t[2] = 2;
  return ftb_lstm_stacked_fwd(x, Wp, bias_p, hs, c, D, L, N, I, H, dtype, t, scratch, FTB_STATIC_SCRATCH_BYTES,
                              stream);
}

}  // extern "C"
