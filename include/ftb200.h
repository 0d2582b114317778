/* C ABI of libftb200: sm_100a kernels for FractalTensor's nested data-parallel
 * hot path (RNN cell wavefronts, back-to-back GEMM, flash attention).
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer owned by the caller unless stated
 *    otherwise; the library allocates nothing in these calls.
 *  - Matrices are row-major with the last dimension contiguous; base pointers
 *    must be 16-byte aligned.
 *  - `dtype`: 0 = fp32, 1 = fp16, 2 = bf16.  16-bit types run on tcgen05 tensor
 *    cores with fp32 accumulation; fp32 runs on CUDA cores.
 *  - `stream` is a cudaStream_t passed as void*.  Calls are asynchronous,
 *    stream-ordered, re-entrant and safe to capture in a CUDA graph.
 *  - `workspace` is at least ftb_workspace_bytes() bytes, zero-filled by the caller
 *    before its first use.  Its first word is the device status word: 0, or the
 *    code of the first bounded device wait that ran out.  Read it with
 *    ftb_read_status() after the stream synced.  The RNN entry points clear it at
 *    the start of every call; for ftb_b2b_gemm and ftb_flash_attn_fwd it is sticky
 *    (a call on a workspace whose status is non-zero does nothing) until the
 *    caller zeroes it again.
 *  - Return value: 0, or an FTB_ERR_* code (ftb_status_str() names it).
 *
 * The reference exposes this path as C++ host functors with compile-time tile
 * shapes and raw device pointers (kaleido/core/device/kernels/lstm.h,
 * gemm.h) and as Python programs over kaleido.operations; each entry point
 * cites what it stands in for.
 */
#ifndef FTB200_H_
#define FTB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FTB_DTYPE_F32 0
#define FTB_DTYPE_F16 1
#define FTB_DTYPE_BF16 2

int ftb_version(void);
const char* ftb_status_str(int code);
size_t ftb_workspace_bytes(void);
/* Number of kernels this library has launched in this process so far. */
long long ftb_launch_count(void);
/* Copies the status word out of `workspace` (synchronises `stream`). */
int ftb_read_status(const void* workspace, int* status_out, void* stream);

/* Packs LSTM parameters for the cell kernels.
 * W: [D,4,I,H], U: [D,4,H,H] in the reference's x@W + h@U orientation and gate
 * order i,f,o,c~ (examples/stacked_rnn/stacked_rnn.py:12-36); bias: [D,4,H] or
 * NULL.  Wp: [D,4H,I+H] K-major with row u*4+g = gate g of unit u (the reference
 * kernels take W,U as [4H,K] row-major, kaleido/core/device/kernels/lstm_kernels.h:24-48).
 * bias_p: fp32 [D,4H] in the same row order (may be NULL when bias is NULL). */
int ftb_lstm_pack_weights(const void* W, const void* U, const void* bias, void* Wp, float* bias_p, int D, int I,
                          int H, int dtype, void* stream);

/* Optional tuning knobs of the wavefront entry points: NULL (all automatic) or a
 * HOST array of FTB_TUNING_INTS ints, 0 = automatic for each:
 *  [0] layers_per_group  stacked LSTM: sweep the wavefront over groups of this many
 *                        layers so that a group's weights stay in L2
 *  [1] bn                accumulator tile width, 128 or 256
 *  [2] schedule          1 = one kernel launch per wavefront level; 2 = one persistent
 *                        cooperative kernel, cells chained through completion counters
 *                        in the workspace (16-bit dtypes; for the fp32 stacked LSTM 2 and 3 both
 *                        name its one persistent kernel: a CTA keeps a 32 x 32 tile of one layer
 *                        with its weights in shared memory and its cell state in registers over
 *                        the whole sweep, the automatic choice when [I + H] x 32 weights and 32
 *                        rows of operands fit in shared memory and a layer's tiles fit on the
 *                        device); 3 = persistent with static
 *                        tile ownership (stacked LSTM: every CTA pair keeps its slice of a
 *                        layer, cell state in registers, over a whole sweep; needs a layer
 *                        group's tiles to fit on the device; the automatic choice when so and
 *                        the batch exceeds 128 sequences); 4 = static tile ownership with the
 *                        weights as the M side of the MMA and the batch (at most 128 sequences)
 *                        as its N side, cell state in registers, recurrent weights resident in
 *                        tensor memory (stacked LSTM; the automatic choice for such batches: it
 *                        is the kernel a batch of 256 sharded over 2, 4 or 8 GPUs runs); every
 *                        schedule gives the same bits
 *  [3] skew              persistent schedule: layer j of a group runs `skew` levels
 *                        behind layer j-1
 *  [4] pair              1 = single CTAs, 2 = CTA pairs (tcgen05 cta_group::2) on
 *                        256-row blocks; automatic = pairs when a cell has > 128 rows
 *  [5] fine_deps         persistent schedule: 1 = each K block waits only for the producer
 *                        tile that holds its columns; otherwise a cell waits for whole cells
 *  [6] resident          weights-major schedule: 64-wide K blocks of each CTA's recurrent weights
 *                        kept in tensor memory for a whole sweep over time; 0 = as many as fit
 *                        beside the accumulators (14, 12 or 8 for batches up to 32, 64 or 128),
 *                        -1 = none (stream everything), n = at most n */
#define FTB_TUNING_INTS 7

/* Stacked LSTM forward as a depth x time wavefront.
 * Stands in for stacked_lstm() (examples/stacked_rnn/stacked_lstm1.py:66-76) and
 * for StackedLstmRegion1/2/3 (kaleido/core/device/kernels/lstm/stacked_lstm/region{1,2,3}.h,
 * benchmarks/rnn/fractaltensor/stacked_lstm/lstm.cu:19-60).
 * x: [L,N,I]; Wp/bias_p from ftb_lstm_pack_weights; hs (out): [D,L,N,H] hidden
 * states of every layer (top layer = hs[D-1]); c (out): fp32 [D,N,H] final cell
 * state.  I == H is required for D > 1.  The persistent schedule needs
 * ftb_lstm_stacked_workspace_bytes(D, L, N, H) bytes of workspace; with less, one kernel
 * is launched per level. */
size_t ftb_lstm_stacked_workspace_bytes(int D, int L, int N, int H);
int ftb_lstm_stacked_fwd(const void* x, const void* Wp, const float* bias_p, void* hs, float* c, int D, int L,
                         int N, int I, int H, int dtype, const int* tuning, void* workspace, size_t workspace_bytes,
                         void* stream);

/* Stacked LSTM forward without a caller workspace.  No counterpart in the reference: it exists
 * for hosts that cannot allocate device memory where they call the forward pass (in a
 * real-time loop, in a plugin that is only handed input and output buffers, under a
 * fully committed memory pool).  Same arguments and results as ftb_lstm_stacked_fwd with the
 * persistent schedule, but the schedule tables, completion counters and status word live in
 * a 4 MiB array inside the library image (held on every GPU that loads the library).
 * Returns FTB_ERR_SCRATCH_LIMIT (7) when ftb_lstm_stacked_workspace_bytes(D, L, N, H) exceeds
 * 4 MiB; fp16/bf16 only.  The array is shared by all calls on a device: calls that can
 * overlap on the GPU race and must be serialised by the caller; consecutive calls on one
 * stream are safe.  The first call on a device looks the array's address up and should be
 * made outside stream capture.  `scratch_out` (may be NULL) receives the array's device
 * address, usable as the `workspace` argument of ftb_read_status(). */
int ftb_lstm_stacked_fwd_noalloc(const void* x, const void* Wp, const float* bias_p, void* hs, float* c, int D,
                                 int L, int N, int I, int H, int dtype, const int* tuning, void** scratch_out,
                                 void* stream);

/* Stacked LSTM forward over a length-sorted batch of variable-length sequences in the
 * time-major packed layout of a ragged FractalTensor [L][active_rows[t]] (flat buffer:
 * the rows of step t follow those of step t-1).  Stands in for batched_cell()/lstm_layer()/
 * stacked_lstm() of the time-major program (examples/stacked_rnn/stacked_rnn.py:40-79, which
 * carries hs_prev[0:xs.length]) on batches built like gen_dataset_time_major()
 * (examples/utils/data_utils.py:42-66), and for the variable-length mode of the reference's
 * cuDNN baseline (benchmarks/rnn/cuDNN/utils.h:44-61).
 * `active_rows` is a HOST array of L ints, non-increasing, active_rows[L-1] >= 1: the number
 * of sequences still running at step t (sequence n occupies row n of every step it is in).
 * With T = sum(active_rows) and N = active_rows[0]: x: [T,I]; hs (out): [D,T,H] in the same
 * packed order; c (out): fp32 [D,N,H], the cell state of each sequence after its own last step.
 * Only tiles that hold active rows are computed.  With ftb_lstm_stacked_varlen_workspace_bytes(D, L)
 * bytes of workspace (16-bit dtypes) the wavefront runs as one persistent launch whose schedule
 * tables are copied from host memory on `stream`; with less it runs one launch per level. */
size_t ftb_lstm_stacked_varlen_workspace_bytes(int D, int L);
int ftb_lstm_stacked_varlen_fwd(const void* x, const void* Wp, const float* bias_p, void* hs, float* c,
                                const int* active_rows, int D, int L, int I, int H, int dtype, const int* tuning,
                                void* workspace, size_t workspace_bytes, void* stream);

/* Dilated stacked LSTM forward: layer l reads its own state dilations[l] steps
 * back.  Stands in for dilated_layer()/model() (examples/dilated_rnn/dilated_rnn.py:16-41)
 * and DilatedLstmRegion1/2 (kaleido/core/device/kernels/lstm/dilated_lstm/region{1,2}.h).
 * x: [L,N,H]; hs (out): [D,L,N,H]; c (scratch/out): fp32 [D, max_dilation*N, H].
 * `dilations` is a HOST array of D ints.  With ftb_lstm_dilated_workspace_bytes(D, L) bytes of
 * workspace (16-bit dtypes) the whole forward pass is one launch.  For H of 64, 128 or 256 that is the
 * cluster schedule (tuning[2] = 4, and the automatic choice): one thread-block cluster per layer and
 * slice of 128 sequences, each CTA's slice of the weights resident in tensor memory for the whole
 * launch, the state of a layer with dilation 1 handed to its next step through the cluster's
 * shared memory.  Otherwise (or with tuning[2] = 2) it is the generic persistent wavefront, whose
 * schedule tables are copied from host memory on `stream`, so that form is not for stream capture.
 * All schedules give the same bits. */
size_t ftb_lstm_dilated_workspace_bytes(int D, int L);
int ftb_lstm_dilated_fwd(const void* x, const void* Wp, const float* bias_p, void* hs, float* c,
                         const int* dilations, int D, int L, int N, int H, int dtype, const int* tuning,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Packs one direction of a grid-RNN block: i2h [2H,H], h2h [H,H] (x@W
 * orientation, examples/grid_rnn/grid_rnn.py:21-30,42-50) into Wp [H,3H]
 * K-major with K order [state_x | state_y | input]. */
int ftb_grid_pack_weights(const void* i2h, const void* h2h, void* Wp, int H, int dtype, void* stream);

/* Stacked 2-D grid RNN forward (vanilla tanh cells, recurrence along both
 * axes), anti-diagonal wavefront.  Stands in for stacked_grid_rnns()
 * (examples/grid_rnn/grid_rnn.py:42-122) and the grid regions
 * (benchmarks/rnn/fractaltensor/grid_lstm/regions/region{1..8}.h).
 * X,Y: [A,B,N,H] inputs of the x and y directions at grid point (a,b);
 * Wpx,Wpy: [D,H,3H] from ftb_grid_pack_weights; bias_x,bias_y: fp32 [D,H] or NULL;
 * hx,hy (out): [D,A,B,N,H].  state_x = hx[a-1][b], state_y = hy[a][b-1].
 * Both directions of a level run in one launch.  With ftb_grid_rnn_workspace_bytes(D, A, B)
 * bytes of workspace (16-bit dtypes) the whole grid runs as one launch: for H of 128 or 256 and
 * D*A*ceil(N/64)*(H/64) <= the SM count, the cluster schedule (one thread-block cluster per grid
 * row and slice of 64 sequences walks the columns; weights resident in tensor memory; h_y handed to
 * the next column through the cluster's shared memory; h_x of the row above through global flags);
 * otherwise, or with a workspace of at least ftb_grid_rnn_tables_bytes(D, A, B) but less than
 * ftb_grid_rnn_workspace_bytes(D, A, B) bytes, the generic persistent wavefront, whose schedule
 * tables are copied from host memory on `stream`; with less than that, one launch per level.
 * All schedules give the same bits. */
size_t ftb_grid_rnn_workspace_bytes(int D, int A, int B);
size_t ftb_grid_rnn_tables_bytes(int D, int A, int B);
int ftb_grid_rnn_fwd(const void* X, const void* Y, const void* Wpx, const void* Wpy, const float* bias_x,
                     const float* bias_y, void* hx, void* hy, int D, int A, int B, int N, int H, int dtype,
                     void* workspace, size_t workspace_bytes, void* stream);

/* Back-to-back GEMM D = (A.B).C per batch entry, fp32 accumulation, the
 * intermediate rounded to the 16-bit input type.  Stands in for B2BGemm /
 * KeBack2BackGemm (kaleido/core/device/kernels/gemm.h:233-269,
 * cutlass_wmma.h:440-540).  A: [batch,M,K] row-major; B: [batch,N,K]
 * (column-major [K,N]); C: [batch,P,N] (column-major [N,P]); Dout: [batch,M,P].
 * M % 128 == 0; K and P 64 or 128; N 128, 256 or 512, with B and C of one batch entry
 * (N.(K+P) 16-bit elements) at most 128 KB; dtype fp16 or bf16. */
int ftb_b2b_gemm(const void* A, const void* B, const void* C, void* Dout, int batch, int M, int N, int K, int P,
                 int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* Flash attention forward with online softmax, non-causal.  Stands in for
 * flash_attention() (examples/flash_attention/flash_attention.py:14-88) with the
 * (max, sum, out) carry started at (-inf, 0, 0).  q,k,v,o: [B,heads,S,d];
 * d = 128, S % 256 == 0 (a CTA takes two 128-row query tiles); dtype fp16 or bf16;
 * softmax(scale * q.k^T). */
int ftb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, int B, int heads, int S, int d,
                       float scale, int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* The same with a causal mask: query i attends to keys 0..i only (scores of later keys
 * are -inf before the softmax).  The reference has no causal program; this is the
 * blockwise program above with the key walk of each query tile cut at its diagonal
 * block, as every other implementation of that example's algorithm defines it.
 * Same shapes and types; scale > 0. */
int ftb_flash_attn_causal_fwd(const void* q, const void* k, const void* v, void* o, int B, int heads, int S,
                              int d, float scale, int dtype, void* workspace, size_t workspace_bytes,
                              void* stream);

/* Causal attention inside a sliding window: query i attends to keys i-window+1 .. i
 * (window >= 1; window >= S is plain causal attention).  Each query tile starts its key
 * walk at the block of the first key its first row sees.  The windowed part of the
 * reference's sparse attention example (examples/sparse_attention/sparse_attention.py:44-46,
 * ops.shifted_slide) is token-level, two-sided and dilated; this entry is the one-sided
 * block form only. */
int ftb_flash_attn_window_fwd(const void* q, const void* k, const void* v, void* o, int B, int heads, int S,
                              int d, int window, float scale, int dtype, void* workspace,
                              size_t workspace_bytes, void* stream);

/* Two-sided local attention: query i attends to keys i-left .. i+right (both >= 0, cut at
 * the ends of the sequence).  left = right = w is the block form of a window of 2w+1 keys
 * centred on the query, as ops.shifted_slide builds it with dilation 1
 * (examples/sparse_attention/sparse_attention.py:44-46). */
int ftb_flash_attn_local_fwd(const void* q, const void* k, const void* v, void* o, int B, int heads, int S,
                             int d, int left, int right, float scale, int dtype, void* workspace,
                             size_t workspace_bytes, void* stream);

/* Token-level sparse attention: dilated window + random + global keys, per head.  Stands in for
 * per_head_attn / sparse_attn (examples/sparse_attention/sparse_attention.py:24-76).  The first and
 * last n_global tokens of a head attend to each other only.  Every other token i attends to the
 * `window` (odd) keys at i - half + j * dilation, half = (window - 1) * dilation / 2, wrapped as
 * ops.shifted_slide wraps them (a position x < 0 becomes x + S - 1, x >= S becomes x - S;
 * kaleido/frontend/operations/fractaltensor/access.py:389-410), and to the keys at the R positions
 * rand_pos[b, head, i - n_global, :].  The example uses window 5, dilation 2, n_global 3, R 3,
 * d 64, scale 1, fp32.
 * q, k, v, o: [B, heads, S, d] of `dtype` (fp32, fp16 or bf16; the arithmetic is fp32), d 32, 64,
 * 128 or 256; rand_pos: int32 [B, heads, S - 2 * n_global, R] on the device (NULL when R = 0);
 * window + R <= 64, 2 * n_global <= min(S, 64), half < S.  A random position outside [0, S) is
 * read as 0 and sets the (sticky) status word to 22.
 * as_shipped: the example calls ops.softmax without a dimension, and the reference's softmax then
 * normalises dimension 0 (kaleido/frontend/operations/tensor/arithmetic/reduction.py:26): every
 * weight of a windowed token becomes 1 (the output is the sum of the gathered values) and the
 * global block is normalised over the queries.  Non-zero reproduces exactly what that program
 * returns; 0 gives softmax(scale * q.k^T) over the keys. */
int ftb_sparse_attn_fwd(const void* q, const void* k, const void* v, const int* rand_pos, void* o, int B,
                        int heads, int S, int d, int window, int dilation, int n_global, int R, float scale,
                        int as_shipped, int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* Packs the weights of a tanh RNN cell h = tanh(x.W + s.U + b) (cell(),
 * examples/rnn_attention/rnn_attention.py:40-48): W [I, H], U [H, H] of `dtype` ->
 * Wp [H, I + H], row u = (W[:, u] | U[:, u]). */
int ftb_rnn_pack_weights(const void* W, const void* U, void* Wp, int I, int H, int dtype, void* stream);

/* Attention RNN forward: model() of examples/rnn_attention/rnn_attention.py:86-110 behind the word
 * lookups.  Encoder: e_j = tanh(x_j.Ws + e_{j-1}.Us + bs) scanned over the source from zeros.
 * Decoder scan (attn_func, lines 52-70), carried value v: dec_t = tanh(y_t.Wt + v_{t-1}.Ut + bt),
 * score_j = e_j.enc_proj + dec_t.dec_proj, w = softmax over the source positions, v_t = sum_j w_j e_j;
 * the program's result is the v_t.
 * Time-major padded batches: src [Ls, N, H], trg [Lt, N, H] of `dtype` (fp32: CUDA cores; fp16 /
 * bf16: tensor cores, fp32 accumulation); Wp_src, Wp_trg from ftb_rnn_pack_weights with I = H;
 * bias_src, bias_trg: fp32 [H] or NULL; enc_proj, dec_proj: [H] of `dtype`; src_lens: int32 [N] on
 * the device, sequence n attends to source positions j < src_lens[n] (NULL: all Ls).
 * Outputs (caller-owned): enc [Ls, N, H] encoder states, enc_scores fp32 [Ls, N] (e_j.enc_proj),
 * dec [Lt, N, H] decoder states, out [Lt, N, H] the attention vectors.  Rows of a sequence past its
 * own source / target length hold values nobody should read.  H % 64 == 0, Ls <= 12288.
 * One launch per source position, one for the scores, two per target position. */
int ftb_rnn_attention_fwd(const void* src, const void* trg, const void* Wp_src, const void* Wp_trg,
                          const float* bias_src, const float* bias_trg, const void* enc_proj, const void* dec_proj,
                          const int* src_lens, void* enc, float* enc_scores, void* dec, void* out, int Ls, int Lt,
                          int N, int H, int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* Embedding lookup out[t, :] = table[ids[t], :] for t < T.  Stands in for the lookup in front of
 * the reference's RNN examples, ops.index(ops.slices(embedding, dim=0), word) mapped over a batch
 * of word sequences (examples/stacked_rnn/rnn_utils.py:80-90): `ids` is the flat int64 buffer of
 * the words FractalTensor in any nesting (batch-major or time-major, ragged or not), `out` the flat
 * buffer of the resulting FractalTensor of [1, H] tensors in the same order.  table: [V, H] of
 * `dtype`; ids: int64 [T] on the device; out: [T, H].  An id outside [0, V) gives a row of zeros
 * and sets the (sticky) status word to 22. */
int ftb_embedding_gather(const void* table, const long long* ids, void* out, long long T, long long V, int H,
                         int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* Row-wise softmax of an fp32 matrix x [rows, width] (row-major, contiguous) with the online
 * (maximum, normaliser) reduction: y = e^(max(x - m, -64)) / d per row, m the row maximum, d the sum
 * of e^(x - m).  Stands in for KeOnlineNormalizedSoftMax / OnlineNormalizedSoftmaxOp
 * (kaleido/core/device/kernels/online_softmax.h:15-183,
 * kaleido/core/operators/online_softmax_op.cu:13-38; the reference instantiates fp32 only and
 * normalises along dimension 0 of its [height, width] view, i.e. over each row's `width`
 * elements).  Needs no workspace. */
int ftb_online_softmax(const float* x, float* y, int rows, int width, void* stream);

/* The projection onto the vocabulary that follows the recurrent layers in the reference's RNN
 * examples (prev_softmax_proj [H, vocab], examples/stacked_rnn/rnn_utils.py:39-62): for every word
 * position, probs = softmax(h . P) over the vocabulary.
 * ftb_projection_pack: P [H,V] (the reference's x @ P orientation) -> Pt [Vp,H] K-major, one row per
 * vocabulary entry, Vp = ftb_projection_padded_cols(V) = V rounded up to 128, padding rows zero.
 * ftb_lstm_project_softmax: h [T,H] = the top layer's hidden states in any flat order (the hs[D-1]
 * of a wavefront entry point as it is); probs (out): fp32 [T,Vp], row t holds softmax(h[t] . P) in its
 * first V columns (columns V..Vp-1 hold 0).  One tcgen05 GEMM writes the fp32 logits into `probs`
 * and the online softmax (ftb_online_softmax's kernel, same clamp) normalises them in place: each
 * logit is written once, read once and written once.  H % 64 == 0; V <= 49152; dtype fp16 or bf16. */
int ftb_projection_padded_cols(int V);
int ftb_projection_pack(const void* P, void* Pt, int H, int V, int dtype, void* stream);
int ftb_lstm_project_softmax(const void* h, const void* Pt, float* probs, long long T, int V, int H, int dtype,
                             void* workspace, size_t workspace_bytes, void* stream);

/* Plain GEMM out[M,N] = A[M,K] . Bt[N,K]^T through the cell kernel's main loop
 * (support op; the reference's KeCuteGemm, kaleido/core/device/kernels/cutlass_wmma.h:115-181).
 * 16-bit dtypes: K % 64 == 0, N % 128 == 0.  fp32: K % 64 == 0, N % 64 == 0. */
int ftb_gemm_nt(const void* A, const void* Bt, void* out, int M, int N, int K, int dtype, const int* tuning,
                void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FTB200_H_ */
