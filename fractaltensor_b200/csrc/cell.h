// Work-item description shared by the wavefront schedulers (host) and the cell
// kernels (device).  One launch executes every cell of one wavefront level: the
// cells of a level are independent, so no CTA ever waits on another CTA.
//
// A cell computes  acc[rows, n_cols] = sum_s  A_s[rows, K_s] * Wp[w_row0 .. , wk_s ..]^T
// where the A_s are up to three activation row-blocks (the cell's input, its
// recurrent state(s)) and Wp holds the cell's weights K-major, one row per
// output column.  The epilogue turns acc into the cell's outputs.
#pragma once
#include <stdint.h>

namespace ftb {

constexpr int kMaxSeg = 3;     // activation sources concatenated along K
constexpr int kMaxItems = 32;  // cells per launch (a level with more is split)
constexpr int kNumActMaps = 3;

enum Epilogue : int {
  EPI_STORE = 0,  // out = acc
  EPI_LSTM = 1,   // columns are gate-interleaved (i,f,o,g per unit): c = f*c + i*g, h = o*tanh(c)
  EPI_TANH = 2,   // out = tanh(acc + bias)
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
  int32_t m_tiles; // ceil(rows / 128)
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
// reads (-1 = external input).  done[i] counts finished epilogue warps of item
// i; item i is complete when done[i] == target[i] (4 warps x tiles of the item).
struct PlanView {
  const CellItem* items;
  const int32_t* dep;     // [n_items][kMaxSeg][2]
  const int32_t* target;  // [n_items]
  int32_t* done;          // [n_items], zero before the launch
};

}  // namespace ftb
