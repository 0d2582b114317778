// Work-item description shared by the wavefront schedulers (host) and the cell
// kernels (device).  One launch executes every cell of one wavefront level: the
// cells of a level are independent, so no CTA ever waits on another CTA.
//
// A cell computes  acc[rows, n_cols] = sum_s  A_s[rows, K_s] * Wp[w_row0 .. , wk_s ..]^T
// where the A_s are up to three activation row-blocks (the cell's input, its
// recurrent state(s)), each read from one of four activation buffers, and Wp (one of
// two packed weight buffers, `w_map`) holds the cell's weights K-major, one row per
// output column.  The epilogue turns acc into the cell's outputs.
#pragma once
#include <stdint.h>

namespace ftb {

constexpr int kMaxSeg = 3;     // activation sources concatenated along K
constexpr int kMaxItems = 24;  // cells per launch (a level with more is split)
constexpr int kNumActMaps = 4;
constexpr int kNumWeightMaps = 2;

enum Epilogue : int {
  EPI_STORE = 0,  // out = acc
  EPI_LSTM = 1,   // columns are gate-interleaved (i,f,o,g per unit): c = f*c + i*g, h = o*tanh(c)
  EPI_TANH = 2,   // out = tanh(acc + bias)
  EPI_STORE_F32 = 3,  // out = acc as fp32 (16-bit inputs; one launch per level, single CTAs only)
};

struct CellItem {
  void* out;          // first output row of this cell: [rows, ld_out]
  float* c;           // LSTM only: fp32 cell state rows, updated in place: [rows, ld_c]
  const float* bias;  // one value per accumulator column (packed order) or nullptr
  int32_t seg_row[kMaxSeg];  // first activation row of segment s in its tensor map / buffer
  int32_t seg_kb[kMaxSeg];   // length of segment s in 64-element K blocks
  int32_t seg_wk[kMaxSeg];   // K offset of segment s inside the packed weight rows
  int32_t seg_map[kMaxSeg];  // which activation tensor map / buffer the segment reads
  int32_t nseg;
  int32_t w_row0;  // first packed weight row of this cell
  int32_t rows;    // valid activation rows (batch entries) of this cell
  int32_t c_zero;  // LSTM only: 1 when the previous cell state is zero (c is not read)
  int32_t tile0;   // index of this cell's first tile inside the launch
  int32_t m_tiles; // row tiles of this cell (128 rows each; even when CTAs run as pairs)
  int32_t out_row0;  // 16-bit LSTM path: row of `out` in the tensor map `out_map` (TMA stores)
  int32_t c_row0;    // 16-bit LSTM path: row of `c` in the cell-state tensor map
  int32_t out_map;   // activation map index that covers `out`
  int32_t w_map;     // which packed weight buffer the cell reads (0 or 1)
  int32_t skip;      // persistent schedule: index of the item that holds tile (tile0 + grid size)
  int32_t pad_;
};

struct CellBatch {
  int32_t n_items;
  int32_t n_cols;       // accumulator columns per cell (4H for LSTM, H for tanh cells)
  int32_t ld_out;       // elements between output rows
  int32_t ld_c;         // elements between cell-state rows
  int32_t total_tiles;
  int32_t pad_;
  CellItem items[kMaxItems];
};

// Device-resident schedule for the persistent (single-launch) wavefront: the
// same CellItem records in launch order (tile0 increasing) plus, per item and
// per activation segment, the inclusive range of items whose output the segment
// reads (-1 = external input).
//
// Completion counters (all zero before the launch):
//   coarse (fine == 0)  done[i] counts epilogue warps of item i that have written
//       their part of the item's output; complete at target[i] (8 warps x tiles).
//       done[n_items + i] counts tiles of item i whose new LSTM cell state is
//       written (complete at target[i] / 8).
//   fine (fine == 1)    for schedules in which a cell and the cells it reads share
//       one row tiling and each segment reads exactly one item: tile_done[t] counts
//       the epilogue warps of tile t (complete at 8) and c_done[t] is 1 once the
//       tile's cell state is written.  K block kb of a segment then waits only
//       for the producer tile(s) that hold those 64 activation columns, so a cell's
//       K loop follows the cells it reads tile by tile instead of waiting for all
//       of them.
struct PlanView {
  const CellItem* items;
  const int32_t* dep;     // [n_items][kMaxSeg][2]
  const int32_t* target;  // [n_items]
  int32_t* done;          // [2 * n_items]
  int32_t* tile_done;     // [total_tiles] (fine)
  int32_t* c_done;        // [total_tiles] (fine)
  int32_t fine;
  int32_t units_per_tile; // activation columns produced by one tile (fine)
  // Finding the item of a tile without walking the table (every step of a walk is a dependent
  // load from L2): either all items have the same number of tiles (tiles_per_item > 0), or
  // cta_first[cta] is the item of the CTA's first tile and CellItem::skip leads from the item
  // of one of its tiles to (at most a few items before) the item of its next tile.
  int32_t tiles_per_item;
  int32_t pad_;
  const int32_t* cta_first;
  unsigned long long* trace;  // debug builds (FTB_TRACE): [total_tiles][4] globaltimer stamps, else nullptr
};

}  // namespace ftb
