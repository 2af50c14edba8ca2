// Launch interfaces of the hand-written sm_100a kernels for the Zoph_RNN inference forward path.
// Everything is column-major fp32 as in the reference (activations H x B, one column per sentence).
#pragma once
#include <cuda_runtime.h>

namespace zrnn {

// thread-local launch counter (each launcher increments it once per kernel launch)
void count_launch(int n = 1);

// ---- input preparation (replaces vocab_to_01 / vocab_to_nonM1, src/custom_kernels.h:9-32)
cudaError_t launch_prep_ids(const int* raw, int n, int* nonm1, int* mask01, cudaStream_t st);

// ---- embedding column gather (replaces sparse_lookup_kernel, src/custom_kernels.h:340-348)
// V > 0: an id >= V reads column 0 instead of memory past the table and sets *err (if given) to kErrBadTokenId
constexpr int kErrBadTokenId = 100;
cudaError_t launch_gather_columns(const float* W, int H, int V, const int* ids, int n_cols, float* x, int* err,
                                  cudaStream_t st);
// same for rows of `row_bytes` bytes (a multiple of 16) of any element type: dst row n = src row ids[n]; n_src_rows > 0
// bounds the ids the same way
cudaError_t launch_gather_rows16(const void* src, size_t row_bytes, int n_src_rows, const int* ids, int n_rows,
                                 void* dst, int* err, cudaStream_t st);

// ---- generic column gather over several H x ncols arrays at once: dst[a][:,c] = src[a][:,map[c]]
// (replaces the per-column cudaMemcpy loops of swap_states_decoding / transfer_decoding_states_GPU,
// src/Input_To_Hidden_Layer.hpp:1231-1260, src/model.hpp:2715-2719)
struct ColGatherArgs {
  enum { MAX_ARRAYS = 40 };  // 8 layers x (h: fp32 + two operand parts, c) + the fed-back attention vector
  const float* src[MAX_ARRAYS];
  float* dst[MAX_ARRAYS];
  int h_arr[MAX_ARRAYS];  // floats per column of each array; 0 = H
  int n_arrays;
  int H, n_cols;
  const int* map;  // n_cols source column indices
};
cudaError_t launch_col_gather(const ColGatherArgs& a, cudaStream_t st);

// ---- fused multi-source GEMM:  acc[M x N] = sum_s A_s[M x K_s] * B_s[K_s x N]
// With gates == 4 the M rows are 4 interleaved H-row blocks (one per LSTM gate i,f,g,o) and each
// thread owns all four gates of its hidden units, so the cell update happens in registers and the
// gate pre-activations never reach HBM.
struct GemmSrc {
  const float* A[4];  // one base pointer per gate block (A[0] only when gates == 1); column-major, ld = lda
  int lda;
  const float* B;  // K x N column-major
  int ldb;
  int K;
};
enum { EPI_STORE = 0, EPI_LSTM = 1, EPI_LSE = 2 };
struct GemmArgs {
  GemmSrc src[3];
  int nsrc;
  int M;  // rows per gate block
  int N;
  // EPI_STORE: C = act(acc + bias[row]) * mask[col]
  float* C;
  int ldc;
  const float* bias[4];  // per gate block; may be null
  const int* mask;       // per column; may be null
  int act;               // 0 none, 1 tanh
  int act_rows;          // act applies to rows < act_rows only (0 = all rows)
  // EPI_LSTM (gates i,f,g,o): c = f*c_prev + i*g ; h = o*tanh(c) ; (h,c) *= mask
  const float* c_prev;
  float* h_out;
  float* c_out;
  float* h_out2;  // optional second copy of h (e.g. the attention memory slot)
  // EPI_LSE: per (row tile, column) max and sum exp(z - max) of z = acc + bias, plus the logit of target[col]
  const int* target;  // global row index; target - target_offset outside [0,M) is ignored
  int target_offset;  // first global row held by this matrix (vocabulary sharding)
  float* part_max;    // [n_row_tiles x N]
  float* part_sum;
  float* tgt_logit;  // [N], must be zero-filled by the caller when targets may fall outside [0,M)
};
// tile = 0: 64 x 64 CTA tile (4x4 per thread); tile = 1: 128 x 128 (8x8 per thread)
cudaError_t launch_fused_gemm(const GemmArgs& a, int gates, int epi, int tile, cudaStream_t st);
int gemm_rows_per_tile(int gates, int tile);

// ---- small layers: a whole sequence of LSTM steps in one launch with the recurrent weights resident on chip
// For hidden sizes whose four H x H recurrent matrices fit the shared memory of a cluster of up to 8 CTAs (H <= 320),
// one layer's S steps run as ONE kernel: each CTA keeps the weight rows of its slice of hidden units in shared memory
// for the whole sequence, h_t is exchanged through distributed shared memory and c_t never leaves registers, so a step
// costs a cluster barrier instead of a kernel launch and no weight byte is read twice.  The input half of the
// pre-activations (M x for every step; it does not depend on the recurrence) is formed first by one batched kernel.
// Exact fp32 FMA arithmetic.  Replaces the per-step loop of src/model.hpp:1581-1600 / :1765-1795 over
// LSTM_IH_Node / LSTM_HH_Node::forward_prop_GPU (src/LSTM.hpp:76-421, src/LSTM_HH.hpp:103-333) for layers without
// feed-input.
// one launch for the start of a scoring pass: id preparation of up to three arrays + zero fills (16-byte aligned
// regions whose sizes are multiples of 4 bytes)
struct PrologueArgs {
  const int* raw[3];
  int n[3];
  int* ids[3];
  int* mask[3];
  void* zero_ptr[12];
  size_t zero_bytes[12];
  int n_zero;
};
cudaError_t launch_score_prologue(const PrologueArgs& a, cudaStream_t st);

struct SeqArgs {
  int H, B, S;           // hidden size, columns, steps
  const float* Mx;       // 4 x (H x H) input matrices, gate order i,f,g,o, each column-major
  const float* Wh;       // 4 x (H x H) recurrent matrices
  const float* bias;     // 4 x H
  // layer input: either x_seq (H x (S*B), the layer below) or an embedding gather (emb H x V, ids [S*B], -1 free)
  const float* x_seq;
  const float* emb;
  const int* ids;
  int V;                 // rows of the embedding table (ids >= V read column 0 and set *err)
  int* err;
  const int* mask;       // [S*B] 0/1
  const float* h0;       // H x B state before step 0
  const float* c0;
  float* h_seq;          // H x (S*B) out
  float* c_out;          // H x B: cell state after the last step
  float* xp;             // scratch: 4 floats per (step, column, hidden unit)
  // optional operand-form copies of h_seq for the tensor-core consumers (row n at + n*ld_op), as AttArgs
  void* op_b16;
  float* op_hi;
  float* op_lo;
  void* op_h_hi;
  void* op_h_lo;
  int ld_op;
};
// false when the shape does not fit (H > 320, B > 32, ...): the caller keeps its per-step path
bool lstm_seq_resident_supported(int H, int B);
cudaError_t launch_lstm_seq_resident(const SeqArgs& a, cudaStream_t st);

// ---- softmax partial combine: logp[n] = (tgt - M) - log(sum_i s_i exp(m_i - M)); 0 where mask==0
cudaError_t launch_lse_combine(const float* part_max, const float* part_sum, const float* tgt_logit, int n_parts,
                               int N, const int* mask, float* logp, cudaStream_t st);
// same with the target logit summed over G shard rows of tgt_logit[G x N] (exactly one shard holds it, the others 0);
// shard_stride (floats, 0 = N) is the distance between two shards' rows in each of the three arrays
cudaError_t launch_lse_combine_shards(const float* part_max, const float* part_sum, const float* tgt_logit, int G,
                                      int N, const int* mask, float* logp, cudaStream_t st, size_t shard_stride = 0);
// reduce n_parts row-tile partials to one (max, sum exp(z-max)) per column
cudaError_t launch_lse_reduce(const float* part_max, const float* part_sum, int n_parts, int N, float* out_max,
                              float* out_sum, cudaStream_t st);

// ---- decode: per column the k largest log-probabilities (sorted) from logits z[V x N] + normaliser
// part_max / part_sum (optional): n_parts row-tile partials per column [part][N] produced by the logits GEMM, which
// save the kernel its first pass over the column; with both and part_width (rows of z per tile) the second pass
// reads only the tiles whose maximum reaches the selection bound
// eos_row: the row of `logits` that holds <EOF> (1 for a whole vocabulary; -1 for a shard that does not hold it, whose
// logp_eos is then -inf); lse_out (optional): log of the column's normaliser, for merging vocabulary shards
cudaError_t launch_topk_logp(const float* logits, int V, int N, int k, float* val_out, int* idx_out, float* logp_eos,
                             cudaStream_t st, const float* part_max = nullptr, const float* part_sum = nullptr,
                             int n_parts = 0, int part_width = 0, int eos_row = 1, float* lse_out = nullptr);
// Merge of G vocabulary shards' top-k lists (each [G][N][k], lse / eos [G][N], shard_lo[G] on the device) into the k
// best of the whole vocabulary per column, as log-probabilities under the global normaliser; G * k <= 288.
// cand_stride / col_stride (4-byte words, 0 = dense) are the distances between two shards' val / idx and lse / eos
// blocks, so the lists can be read straight out of an all-gather's receive buffer.
cudaError_t launch_topk_merge(const float* val, const int* idx, const float* lse, const float* eos, const int* shard_lo,
                              int G, int N, int k, float* val_out, int* idx_out, float* eos_out, cudaStream_t st,
                              size_t cand_stride = 0, size_t col_stride = 0);

// ---- attention
struct AttArgs {
  int H, B, D, S_max, B_src, cols_per_sent;
  const float* hs;  // S_max slots of H x B_src
  const int* len;   // per source column
  const int* offset;
  const int* mask;   // per target column
  const float* h_t;  // H x B
  // local-p only
  const float* tanh1;  // tanh(W_p h), column b at tanh1 + b*ld_tq
  const float* v_p;    // H
  const float* q;      // W_a^T h, column b at q + b*ld_tq
  int ld_tq;
  float* c_t;          // context out, H x B
  float* align_out;    // optional
  // local-p only: 0 = align_out holds the (2D+1) window weights [j*B+b]; 1 = S_max x B weights by source position
  // [s*B+b] with zeros outside the window (what BZ_CUDA::alignment_scores holds, src/attention_node.hpp:236-262)
  int align_by_pos;
  // optional: per target column the source position with the largest weight, -1 for a masked column
  // (get_viterbi_alignment_kernel, src/custom_kernels.h:1621-1635)
  int* viterbi_out;
  // start value of the running maximum: -1 in the kernel itself; 0 in the decoder, where ensembles_models re-derives
  // the alignment from the weights with a maximum that starts at 0 (src/ensemble_factory.hpp:812-834), so a column
  // whose weights are all zero reports -1
  float viterbi_init;
  // optional copies of the context in tensor-core operand form (row b at + b*ld_op)
  void* op_b16;
  float* op_hi;
  float* op_lo;
  void* op_h_hi;  // fp16 split operands: fp16 hi part and scaled fp16 lo part
  void* op_h_lo;
  int ld_op;
};
cudaError_t launch_att_local(const AttArgs& a, cudaStream_t st);
cudaError_t launch_att_global(const AttArgs& a, cudaStream_t st);

// ---- ensemble decoding: out[v + n*V] = log( mean_k softmax(logits_k[:, n])[v] ), the log of the averaged
// distribution of ensemble_factory::ensembles_models (src/ensemble_factory.hpp:768-795).  The renormalisation the
// reference applies after averaging is the log-softmax the top-k kernel performs on `out`.
#define ZR_ENSEMBLE_MAX 8
#define ZR_BEAM_MAX 32  // beam width (every hypothesis proposes beam + 1 <= 33 candidates per step)
#define ZR_SHARD_MAX 8  // vocabulary shards (ranks) a top-k merge takes
struct EnsembleArgs {
  const float* logits[ZR_ENSEMBLE_MAX];  // each V x N, column-major
  int K, V, N;
  float* out;  // V x N
};
cudaError_t launch_ensemble_logmean(const EnsembleArgs& a, cudaStream_t st);
// Alignment voting of an ensemble (ensembles_models, src/ensemble_factory.hpp:798-834): per column the source position
// with the largest sum over the models of the attention weight at that position; the running maximum starts at 0,
// so a column whose weights are all zero reports -1.  align[k] is S_max[k] x N by position.
struct EnsembleVitArgs {
  const float* align[ZR_ENSEMBLE_MAX];
  int S_max[ZR_ENSEMBLE_MAX];
  int K, N;
  int* viterbi_out;  // [N]
};
cudaError_t launch_ensemble_viterbi(const EnsembleVitArgs& a, cudaStream_t st);

// ---- beam bookkeeping (replaces decoder::expand_hypothesis_without_fsa / finish_current_hypotheses /
// output_k_best_hypotheses, src/decoder.h:1157-1315, 672-688, 1386-1463, run on the host there)
struct BeamArgs {
  int n_sent, beam, k_cand, Lmax, k_best, step;
  float min_ratio, penalty;
  const float* cand_val;   // [n_sent*beam][k_cand] log-probs, sorted descending
  const int* cand_idx;     // [n_sent*beam][k_cand]
  const float* logp_eos;   // [n_sent*beam]
  const int* src_len;      // [n_sent]
  const int* max_steps;    // [n_sent]
  int* top_sent;           // [n_sent][beam][Lmax]
  int* top_tmp;            // same size: the step writes the surviving rows here; the caller swaps the two after it
  float* scores;           // [n_sent][beam]
  int* cur_ids;            // [n_sent*beam] current word per column (-1 invalid)
  int* col_map;            // [n_sent*beam] source column for the state reorder
  int* best_ids;           // [n_sent][k_best][Lmax]
  int* best_len;           // [n_sent][k_best]
  float* best_score;       // [n_sent][k_best]
  // optional viterbi-alignment tracking for UNK replacement (all null when off): the attention step's alignment per
  // column, the alignment stored with every position of every beam entry (top_sentences_viterbi, src/decoder.h:230,
  // initialised to -20, :1335) and with every position of the k-best hypotheses
  const int* viterbi;      // [n_sent*beam]
  int* vit_rows;           // [n_sent][beam][Lmax]
  int* vit_tmp;            // same size, swapped with vit_rows like the rows above
  int* best_align;         // [n_sent][k_best][Lmax]
};
cudaError_t launch_beam_init(const BeamArgs& a, cudaStream_t st);
cudaError_t launch_beam_step(const BeamArgs& a, cudaStream_t st);

// ---- operand preparation for the tensor-core GEMMs (K-major rows; see tc_gemm.cuh)
// op_mode: 0 = bf16, 1 = fp32 as is, 2 = fp32 split into hi (tf32-representable) + lo (residual),
// 3 = fp16 split: hi = fp16(v), lo = fp16((v - hi) * 2^11) (dst_lo then points to fp16 storage)
// Packs G column-major (H x K, leading dimension lda) matrices into K-major rows: packed row
// r = tile*(G*TH) + g*TH + j holds row hid = tile*TH + j of matrix g (zero when hid >= H), written at
// dst[r*ld_dst + koff + k].  n_tiles = ceil(H / TH).
struct PackArgs {
  const float* src[4];
  int G, H, K, lda, TH, n_tiles;
  void* dst_hi;
  float* dst_lo;
  int op_mode, ld_dst, koff;
  // tile-contiguous destination (tiled_kbtot > 0): element (packed row r, K index kk = koff + k) goes to
  // (((r / rows_per_tile) * tiled_kbtot + kk / epk) * rows_per_tile + r % rows_per_tile) * epk + kk % epk,
  // i.e. every (row tile, 128-byte k-block) box of the GEMM is one contiguous chunk of memory; ld_dst is unused.
  int tiled_kbtot, tiled_epk;
};
cudaError_t launch_pack_weights(const PackArgs& a, cudaStream_t st);
// Converts `rows` K-major rows (fp32, stride ld_src) into operand form at dst[r*ld_dst + k].
cudaError_t launch_convert_rows(const float* src, long long rows, int K, long long ld_src, int op_mode, void* dst_hi,
                                float* dst_lo, long long ld_dst, cudaStream_t st);

// misc
cudaError_t launch_fill_int(int* p, int v, size_t n, cudaStream_t st);
// len[b] = number of unmasked steps of column b in mask[T x B]; offset[b] = T - len[b]
// (the reference's batch_info, src/fileHelper.h:480-496)
cudaError_t launch_src_len(const int* mask01, int T, int B, int* len, int* offset, cudaStream_t st);
// map[c] = c / div
cudaError_t launch_div_map(int* map, int n, int div, cudaStream_t st);
long long launch_count_value();
void launch_count_reset();

}  // namespace zrnn
