/*
 * zrnn.h - C ABI of the B200-native inference forward path for Zoph_RNN models
 * (embedding column gather -> stacked LSTM step -> attention -> vocabulary softmax, for
 * teacher-forced scoring and beam decoding).
 *
 * The reference exposes this path only as C++ template classes inside one translation unit;
 * each entry point below names the reference member it stands in for (paths are relative to
 * the reference project).  Conventions:
 *   - every function returns a zrnn_status; nothing exits the process; zrnn_last_error() gives
 *     the message of the last failure on the calling thread;
 *   - matrices are column-major exactly as in the reference (IDX2C(i,j,ld)=j*ld+i,
 *     src/BZ_CUDA_UTIL.h:26): activations H x B (one column per sentence), embeddings H x V,
 *     softmax weights V x H; token ids are int32, time-major idx[b + t*B], -1 = padding;
 *   - pointers named d_* are device pointers on the current CUDA device, pointers named h_* (or
 *     unprefixed in the model-level calls) are host pointers; `stream` is a cudaStream_t passed
 *     as void* (NULL = the legacy default stream);
 *   - handles own their device memory and free it in *_destroy; a handle is not thread-safe,
 *     distinct handles may be used from distinct host threads;
 *   - there is no CPU fallback: without a CUDA device every compute entry point fails with
 *     ZRNN_E_CUDA.
 */
#ifndef ZRNN_H
#define ZRNN_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  ZRNN_OK = 0,
  ZRNN_E_ARG = 1,     /* bad shape, null pointer, unsupported combination */
  ZRNN_E_CUDA = 2,    /* CUDA runtime error or no device */
  ZRNN_E_NCCL = 3,    /* NCCL could not be loaded, or one of its calls failed (zrnn_last_error() has the text) */
  ZRNN_E_TIMEOUT = 4, /* a bounded device-side wait gave up */
  ZRNN_E_IO = 5,      /* weight file missing, truncated or malformed */
  ZRNN_E_STATE = 6    /* call order violated (e.g. forward before load) */
} zrnn_status;

/* Arithmetic of the GEMM-shaped work (state, biases, activations functions and softmax reductions are fp32 in
 * every mode):
 *   ZRNN_F32        fp32-accurate: tcgen05 split-operand tensor-core kernels when H >= 64 and H % 4 == 0 (fp16
 *                   split, see ZRNN_F32_F16X2), else the exact fp32 FMA kernels.  Environment ZRNN_FP32_ENGINE =
 *                   simt forces the FMA kernels, = x3 the 3xTF32 kernels.
 *   ZRNN_BF16       tcgen05 tensor cores on bf16-rounded weights and activations (H % 8 == 0)
 *   ZRNN_TF32       tcgen05 tensor cores, single-pass tf32 (H % 4 == 0)
 *   ZRNN_F32_SIMT   always the exact fp32 FMA kernels
 *   ZRNN_F32_3XTF32 always the 3xTF32 tensor-core kernels (H % 4 == 0): operands as tf32 hi + fp32 residual
 *   ZRNN_F32_F16X2  always the fp16-split tensor-core kernels (H % 4 == 0): operands as fp16 hi + fp16 residual
 *                   scaled by 2^11 (11 + 11 significant bits like 3xTF32, half the bytes and tensor time); weights
 *                   must lie inside the fp16 range, which the load functions check (ZRNN_E_ARG otherwise) */
typedef enum {
  ZRNN_F32 = 0, ZRNN_BF16 = 1, ZRNN_TF32 = 2, ZRNN_F32_SIMT = 3, ZRNN_F32_3XTF32 = 4, ZRNN_F32_F16X2 = 5
} zrnn_dtype;
typedef enum { ZRNN_ATT_NONE = 0, ZRNN_ATT_LOCAL_P = 1, ZRNN_ATT_GLOBAL_DOT = 2 } zrnn_attention_type;

const char* zrnn_status_string(int status);
const char* zrnn_last_error(void);
/* library version, and the compute capability the kernels were built for (100 = sm_100a) */
int zrnn_version(void);
int zrnn_built_for_sm(void);
/* Device selection for the calling thread.  The reference binds a model to devices with --multi-gpu and
 * cudaSetDevice before every allocation (src/main.cu:28-30 of the option list, src/model.hpp:3-60); here one
 * device holds a whole model, so the caller selects it once before creating the model. */
int zrnn_device_count(int* n);
int zrnn_set_device(int device);
/* number of kernels this library has launched on the calling thread since the last reset */
long long zrnn_launch_count(void);
void zrnn_reset_launch_count(void);
/* Optional per-class kernel timing for the benchmark's roofline report (no reference counterpart; the
 * reference only has wall-clock Timer blocks, src/memory_util.h:83-124).  While on, the library records a CUDA
 * event pair around every launch group of each class on the launching stream (at most 16384 pairs per thread).
 * Classes: 0 embedding gather, 1 LSTM cell, 2 attention, 3 softmax GEMM, 4 softmax reduce / top-k, 5 beam step,
 * 6 state reorder.  zrnn_kernel_timing_read waits for the recorded events. */
int zrnn_kernel_timing(int on);
int zrnn_kernel_timing_read(int kernel_class, long long* launches, double* total_ms);

/* The GEMM building block: C[n_rows x m_cols] = W[n_rows x K] * X[K x m_cols], all column-major fp32, as the
 * reference's cublas_gemm_wrapper (src/BZ_CUDA_UTIL.h:691-696) called with CUBLAS_OP_N, CUBLAS_OP_N.
 * mode 0 = exact fp32 FMA kernel; 1 = tcgen05 tensor cores on bf16-rounded operands; 2 = tcgen05 tf32;
 * 3 = tcgen05 3xTF32 (operands split into tf32 hi + lo parts, fp32-level accuracy); 4 = tcgen05 fp16 split (fp16 hi
 * + scaled fp16 lo parts, fp32-level accuracy for operands inside the fp16 range).  Synchronous; allocates
 * scratch for the packed operands.  Returns ZRNN_E_TIMEOUT if a bounded device-side wait gave up. */
int zrnn_gemm(int mode, int n_rows, int m_cols, int K, const float* d_W, int ldw, const float* d_X, int ldx,
              float* d_C, int ldc, void* stream);
/* Reads and clears the device-side error word of the tensor-core kernels (0 = none). */
int zrnn_tc_error(void);
/* ------------------------------------------------------------------------------------------
 * Input preparation.  Replaces vocab_to_01 / vocab_to_nonM1 (src/custom_kernels.h:9-32), called
 * from Input_To_Hidden_Layer::prep_GPU_vocab_indices (src/Input_To_Hidden_Layer.hpp:1178-1225):
 * ids with -1 padding -> (id or 0, mask 0/1).
 * ---------------------------------------------------------------------------------------- */
int zrnn_prep_vocab_indices(const int* d_ids_raw, int n, int* d_ids_nonm1, int* d_mask01, void* stream);

/* ------------------------------------------------------------------------------------------
 * LSTM layers.  zrnn_lstm_layer stands for both Input_To_Hidden_Layer (layer 0: embedding
 * gather + LSTM, src/Input_To_Hidden_Layer.h:146-203) and Hidden_To_Hidden_Layer (layers >= 1,
 * src/Hidden_To_Hidden_Layer.h:138-177).
 * ---------------------------------------------------------------------------------------- */
typedef struct zrnn_lstm_layer zrnn_lstm_layer;

/* Input_To_Hidden_Layer::init_Input_To_Hidden_Layer (src/Input_To_Hidden_Layer.hpp:171) and
 * init_feed_input (:235).  V = input vocabulary size. */
int zrnn_ih_create(int H, int V, int feed_input, int dtype, zrnn_lstm_layer** out);
/* Hidden_To_Hidden_Layer::init_Hidden_To_Hidden_Layer (src/Hidden_To_Hidden_Layer.hpp:125). */
int zrnn_hh_create(int H, int dtype, zrnn_lstm_layer** out);
/* load_weights (src/Input_To_Hidden_Layer.hpp:1104-1171, src/Hidden_To_Hidden_Layer.hpp:704-742).
 * h_tensors: host pointers to column-major fp32 matrices in the reference's file order:
 *   W_hi b_i W_hf b_f W_hc b_c W_ho b_o [W (H x V), ih only] M_i M_f M_o M_c [Q_i Q_f Q_o Q_c, feed-input only]
 * n_tensors must equal 12 (+1 for ih) (+4 with feed-input). */
int zrnn_lstm_load(zrnn_lstm_layer* layer, const float* const* h_tensors, int n_tensors);
/* sparse_lookup_kernel (src/custom_kernels.h:340-348): d_x[:,n] = W[:,ids[n]], n_cols columns. */
int zrnn_ih_gather(zrnn_lstm_layer* layer, const int* d_ids_nonm1, int n_cols, float* d_x, void* stream);
/* LSTM_IH_Node::forward_prop_GPU (src/LSTM.hpp:76-421): gather + one LSTM step for B columns.
 * d_htild_prev non-NULL adds the feed-input term Q*htild (the reference skips it at node index 0,
 * src/LSTM.hpp:154,175).  h/c buffers are H x B; outputs may not alias inputs. */
int zrnn_ih_forward(zrnn_lstm_layer* layer, const int* d_ids_nonm1, const int* d_mask01, const float* d_h_prev,
                    const float* d_c_prev, const float* d_htild_prev, int B, float* d_h_out, float* d_c_out,
                    void* stream);
/* LSTM_HH_Node::forward_prop_GPU (src/LSTM_HH.hpp:103-333): one LSTM step on the h of the layer below. */
int zrnn_hh_forward(zrnn_lstm_layer* layer, const float* d_h_below, const int* d_mask01, const float* d_h_prev,
                    const float* d_c_prev, int B, float* d_h_out, float* d_c_out, void* stream);
int zrnn_lstm_destroy(zrnn_lstm_layer* layer);

/* ------------------------------------------------------------------------------------------
 * Attention (src/attention_layer.h:28-33, ctor src/attention_layer.hpp:3-173, decoder init
 * :176-259).  ZRNN_ATT_LOCAL_P is the reference's local-p model with the "general" score;
 * ZRNN_ATT_GLOBAL_DOT is an extension (dot score over every valid source position) that shares
 * the reference's tanh combiner and feed-input wiring.
 * ---------------------------------------------------------------------------------------- */
typedef struct zrnn_attention zrnn_attention;
int zrnn_att_create(int H, int D, int att_type, int dtype, zrnn_attention** out);
/* attention_layer::load_weights (src/attention_layer.hpp:485-491): W_a W_p v_p(1xH) output_bias W_c_p1 W_c_p2 */
int zrnn_att_load(zrnn_attention* att, const float* const* h_tensors, int n_tensors);
/* prep_minibatch_info (src/attention_layer.hpp:580-583) plus the d_total_hs_mat pointer table:
 * d_hs = S_max slots of H x B_src (slot t = top-layer source state at encoder step t); d_len/d_offset =
 * the reference's batch_info halves [S_b...][S_max-S_b...] (src/fileHelper.h:480-496).  Each source
 * column serves cols_per_sentence consecutive target columns (1 for scoring, beam for decoding, which
 * replaces the per-beam replication of src/model.hpp:2434-2445). */
int zrnn_att_set_source(zrnn_attention* att, const float* d_hs, int S_max, int B_src, const int* d_len,
                        const int* d_offset, int cols_per_sentence);
/* attention_node::forward_prop (src/attention_node.hpp:73-394).  d_align_out (optional): local-p
 * (2D+1) x B weights stored [j*B+b]; global S_max x B stored [s*B+b] in source-position order. */
int zrnn_att_forward(zrnn_attention* att, const float* d_h_t, const int* d_mask01, int B, float* d_htild_out,
                     float* d_align_out, void* stream);
/* The same step with the viterbi alignment of every column: get_viterbi_alignment_kernel
 * (src/custom_kernels.h:1621-1635, called from src/attention_node.hpp:225-234 when UNK replacement is on).
 * d_viterbi_out[b] = source position (un-reversed sentence) of the largest weight, -1 for a masked column. */
int zrnn_att_forward_viterbi(zrnn_attention* att, const float* d_h_t, const int* d_mask01, int B, float* d_htild_out,
                             int* d_viterbi_out, void* stream);
int zrnn_att_destroy(zrnn_attention* att);

/* ------------------------------------------------------------------------------------------
 * Softmax loss layer (base_loss_layer virtuals src/base_loss.h:17-63, softmax_layer
 * src/softmax.hpp).  A layer may hold only rows [shard_lo, shard_hi) of D for vocabulary sharding.
 * ---------------------------------------------------------------------------------------- */
typedef struct zrnn_softmax zrnn_softmax;
int zrnn_softmax_create(int V, int H, int dtype, int shard_lo, int shard_hi, zrnn_softmax** out);
/* softmax_layer::load_weights (src/softmax.hpp:337-355): D (V x H), b_d (V x 1), full matrices. */
int zrnn_softmax_load(zrnn_softmax* sm, const float* h_D, const float* h_b_d);
/* get_perplexity_GPU + compute_loss_GPU (src/softmax.hpp:636-692,867-900): natural-log probability of
 * d_targets[n] for each of N columns of d_h (H x N); 0 where d_mask01[n]==0.  The V x N logits are never
 * materialised.  Unsharded layers only. */
int zrnn_softmax_score(zrnn_softmax* sm, const float* d_h, const int* d_targets, const int* d_mask01, int N,
                       float* d_logp_out, void* stream);
/* Allocation-free variant of zrnn_softmax_score.  No counterpart in the reference: it exists for hosts that
 * cannot allocate device memory once they are running - a server whose own arena already owns the whole GPU,
 * or a latency-bound loop that cannot afford the device-wide stall of cudaMalloc/cudaFree.  Same arguments as
 * zrnn_softmax_score.  Arithmetic: always the exact fp32 FMA kernel on the layer's fp32 copy of D, whatever the
 * layer's zrnn_dtype - for a ZRNN_F32 / ZRNN_F32_SIMT layer the results equal zrnn_softmax_score's to fp32 rounding,
 * for a ZRNN_BF16 / ZRNN_TF32 layer they are the fp32 results (closer to the reference than that layer's own
 * tensor-core path, and slower at large V).  The per-tile scratch lives in a fixed 16 MiB array inside the library
 * (zrnn_softmax_score_noalloc_max_floats() floats, present on every GPU that loads the library until the process
 * exits) and the call performs no cudaMalloc, cudaFree or other allocating call.
 * Limit: (2*ceil(V/rows)+1)*N floats must fit, rows = 128 when N >= 96 and V >= 512, else 64; beyond it the call
 * returns ZRNN_E_ARG with the numbers in zrnn_last_error().  The first call on each device looks up the array's
 * device address (that device must be current); make that first call before starting any stream capture.
 * All calls on a device share the one array and it keeps the previous call's contents (the call clears what it
 * needs cleared); two calls that overlap on the GPU - different streams, or different threads - race. */
int zrnn_softmax_score_noalloc(zrnn_softmax* sm, const float* d_h, const int* d_targets, const int* d_mask01, int N,
                               float* d_logp_out, void* stream);
int zrnn_softmax_score_noalloc_max_floats(void);
/* Sharded scoring, step 1: per-column (max, sum exp(z-max), target logit or 0) over this shard's rows. */
int zrnn_softmax_partials(zrnn_softmax* sm, const float* d_h, const int* d_targets, int N, float* d_max,
                          float* d_sum, float* d_tgt, void* stream);
/* Sharded scoring, step 2: combine G shards' partials (each array G x N, shard-major) into log-probs. */
int zrnn_softmax_combine(const float* d_max, const float* d_sum, const float* d_tgt, int G, int N,
                         const int* d_mask01, float* d_logp_out, void* stream);
/* get_distribution_GPU (src/softmax.hpp:514-632) fused with the per-column pre-selection of
 * decoder::expand_hypothesis_without_fsa (src/decoder.h:1197-1219): the k largest log-probabilities of
 * each of N columns, sorted descending (k <= 33), their word ids, and the log-probability of <EOF> (id 1). */
int zrnn_softmax_topk(zrnn_softmax* sm, const float* d_h, int N, int k, float* d_logp_out, int* d_idx_out,
                      float* d_logp_eos, void* stream);
int zrnn_softmax_destroy(zrnn_softmax* sm);

/* ------------------------------------------------------------------------------------------
 * Collective layer: the output vocabulary sharded over the GPUs of one node.
 * The reference spreads a model over GPUs layer by layer (-M, src/global_params.h gpu_indicies,
 * src/model.hpp:80-140) and keeps the whole softmax on the last one (src/softmax.hpp:7-60); at the
 * sizes where one GPU no longer holds D, or where its V x H read bounds the step, the rows of D are
 * split here instead: rank r of `world` holds rows [V r / world, V (r + 1) / world)
 * (zrnn_shard_range).  One process per GPU; the collectives are NCCL's, loaded at first use
 * (libnccl.so.2), on the caller's stream.  At most 8 ranks.
 * ---------------------------------------------------------------------------------------- */
typedef struct zrnn_comm zrnn_comm;
#define ZRNN_COMM_ID_BYTES 128
/* Rank 0 makes the id and hands it to the other ranks by any host channel (a file, a socket, MPI,
 * torch.distributed's store); then every rank calls zrnn_comm_create with the same id. */
int zrnn_comm_unique_id(char* id128);
/* Collective call: blocks until all `world` ranks have joined.  The calling thread's current device is the
 * rank's GPU.  world == 1 needs no id (NULL) and no NCCL: its collectives are local copies. */
int zrnn_comm_create(const char* id128, int rank, int world, zrnn_comm** out);
/* The same around a communicator the host already owns (an ncclComm_t passed as void*; it must come from the NCCL
 * library this process has loaded as libnccl.so.2).  zrnn_comm_destroy leaves that communicator alone. */
int zrnn_comm_from_nccl(void* nccl_comm, int rank, int world, zrnn_comm** out);
int zrnn_comm_rank(const zrnn_comm* c, int* rank, int* world);
/* d_recv receives world * bytes_per_rank bytes, rank-major. */
int zrnn_comm_all_gather(zrnn_comm* c, const void* d_send, void* d_recv, size_t bytes_per_rank, void* stream);
/* Device time of the five stages of this rank's last zrnn_score_batch_sharded call, in milliseconds: [0] id upload +
 * recurrent stack and attention on the rank's columns, [1] all-gather of the top hidden states (+ operand conversion),
 * [2] this rank's vocabulary rows against all columns (GEMM with max/sum epilogue, reduce), [3] all-gather of
 * (max, sum, target logit) + combine, [4] copy of the log-probabilities to the host. */
int zrnn_comm_last_stage_ms(const zrnn_comm* c, float* ms5);
int zrnn_comm_destroy(zrnn_comm* c);
int zrnn_shard_range(int V, int world, int rank, int* lo, int* hi);

/* Sharded decoding, step 1 (a layer created with a vocabulary range): the k best rows of THIS layer's rows per
 * column, as log-probabilities under the layer's own normaliser, sorted descending; d_idx_out are row numbers
 * inside the shard (-1 beyond the shard's size); d_lse_out[n] = log of that normaliser; d_logp_eos (optional) is
 * the <EOF> row's value under it, or -inf when the shard does not hold word 1. */
int zrnn_softmax_topk_shard(zrnn_softmax* sm, const float* d_h, int N, int k, float* d_logp_out, int* d_idx_out,
                            float* d_lse_out, float* d_logp_eos, void* stream);
/* Sharded decoding, step 2: the k best of G shards' lists (d_val / d_idx [G][N][k], d_lse / d_eos [G][N],
 * d_shard_lo[G] = first word id of every shard) under the global normaliser log sum_g exp(lse_g); word ids are
 * global, ties go to the lower id, as in zrnn_softmax_topk.  G <= 8, k <= 33. */
int zrnn_topk_merge(const float* d_val, const int* d_idx, const float* d_lse, const float* d_eos, const int* d_shard_lo,
                    int G, int N, int k, float* d_val_out, int* d_idx_out, float* d_eos_out, void* stream);
/* Both steps with the all-gather between them (k (value, id) pairs and two floats per column and rank): what
 * zrnn_softmax_topk returns for the whole vocabulary, on every rank.  The layer must hold this rank's range. */
int zrnn_softmax_topk_sharded(zrnn_softmax* sm, zrnn_comm* c, const float* d_h, int N, int k, float* d_logp_out,
                              int* d_idx_out, float* d_logp_eos, void* stream);

/* ------------------------------------------------------------------------------------------
 * Whole model (neuralMT_model, src/model.h / src/model.hpp).
 * ---------------------------------------------------------------------------------------- */
typedef struct zrnn_model zrnn_model;
typedef struct {
  int num_layers;   /* -N */
  int H;            /* -H, LSTM_size */
  int V_src;        /* -v (ignored for language models) */
  int V_tgt;        /* -V */
  int lm;           /* 1 = sequence model (-s): no source side */
  int attention;    /* zrnn_attention_type; the reference's --attention-model means ZRNN_ATT_LOCAL_P */
  int feed_input;   /* --feed-input */
  int D;            /* --attention-width */
  int dtype;        /* zrnn_dtype of the arithmetic */
} zrnn_model_config;

/* neuralMT_model::initModel / initModel_decoding (src/model.hpp:3-435, 476-698). */
int zrnn_model_create(const zrnn_model_config* cfg, zrnn_model** out);
/* The same model with only rows [shard_lo, shard_hi) of the softmax's D and b_d on this GPU (the tensor list and
 * zrnn_model_set_tensor still take the full matrices; the rows outside the range are dropped at finalize).  Such a
 * model scores and decodes through the *_sharded calls below, with a zrnn_comm whose rank owns exactly that range. */
int zrnn_model_create_sharded(const zrnn_model_config* cfg, int shard_lo, int shard_hi, zrnn_model** out);
/* Tensor list in weight-file order (src/model.hpp:2172-2241). name buffer >= 32 bytes. */
int zrnn_model_num_tensors(zrnn_model* m);
int zrnn_model_tensor_info(zrnn_model* m, int i, char* name, int* rows, int* cols);
/* Copy one fp32 column-major host tensor into the model; zrnn_model_finalize after the last one. */
int zrnn_model_set_tensor(zrnn_model* m, int i, const float* h_data);
int zrnn_model_finalize(zrnn_model* m);
/* neuralMT_model::load_weights (src/model.hpp:2172-2241) with read_matrix_GPU (src/Eigen_Util.h:83-112):
 * parse a text model.nn.  The architecture comes from the file's 9-int header
 * (src/add_model_info.h:7-9); att_type_override picks local-p or global-dot when the header says the model
 * has attention (the reference has no flag for the type), D is --attention-width. */
int zrnn_model_load_file(const char* path, int att_type_override, int D, int dtype, zrnn_model** out);
/* The same for rank `rank` of `world` of a vocabulary-sharded group: only rows [V rank / world, V (rank+1) / world) of
 * D and b_d stay on this GPU (every rank parses the whole file). */
int zrnn_model_load_file_sharded(const char* path, int att_type_override, int D, int dtype, int world, int rank,
                                 zrnn_model** out);
int zrnn_model_get_config(zrnn_model* m, zrnn_model_config* cfg);
/* Host-only pieces of the same loader (no device is touched).  zrnn_model_file_header reads line 1 of a model.nn
 * (header[9], zero-filled beyond the *n_header_ints integers the file carries; src/add_model_info.h:7-9) and counts
 * the vocabulary lines.  zrnn_model_file_read parses the first n_matrices matrices (rows[i] x cols[i], in file
 * order) into the caller's column-major host buffers: read_matrix_GPU without the upload
 * (src/Eigen_Util.h:83-112). */
int zrnn_model_file_header(const char* path, int* header, int* n_header_ints, int* n_source_words,
                           int* n_target_words);
int zrnn_model_file_read(const char* path, int n_matrices, const int* rows, const int* cols, float* const* h_out);

/* neuralMT_model::getError / get_perplexity (src/model.hpp:1463-1802, 2281-2355) for one minibatch.
 * Host buffers: src_ids [S_max*B] reversed + left-padded with -1 (NULL for a language model),
 * tgt_in / tgt_out [T*B] right-padded with -1.  logp_out [T*B] receives the natural-log probability of
 * every target token (0 under padding); *total_logp their sum (what the reference prints per minibatch). */
int zrnn_score_batch(zrnn_model* m, const int* src_ids, int S_max, const int* tgt_in, const int* tgt_out, int T,
                     int B, float* logp_out, double* total_logp);
/* Same, with ids already on the device and results left on the device; asynchronous on `stream`. */
int zrnn_score_batch_device(zrnn_model* m, const int* d_src_ids, int S_max, const int* d_tgt_in,
                            const int* d_tgt_out, int T, int B, float* d_logp_out, void* stream);
/* The recurrent part of getError only (encoder, decoder stack, attention): writes the H x (T*B) vectors that the
 * reference hands to softmax_layer::backprop_prep_GPU (src/model.hpp:1752,1785) into d_top_out and skips the
 * softmax.  Used when the softmax is vocabulary-sharded over several GPUs. */
int zrnn_forward_states_device(zrnn_model* m, const int* d_src_ids, int S_max, const int* d_tgt_in, int T, int B,
                               float* d_top_out, void* stream);
/* Copies the top-layer vectors the last scoring call handed to the softmax (H x (T*B)) into d_out, which holds
 * capacity_cols columns; *n_cols receives the number of columns available.  For layer-level checks. */
int zrnn_model_copy_top_states(zrnn_model* m, float* d_out, int capacity_cols, int* n_cols, void* stream);
/* The model's softmax layer (owned by the model). */
zrnn_softmax* zrnn_model_softmax(zrnn_model* m);

/* Beam decoding of n_sent sentences at once: ensemble_factory::decode_file_batch
 * (src/ensemble_factory.hpp:583-765) with forward_prop_source / forward_prop_target /
 * swap_decoding_states (src/model.hpp:2367-2452, 2573-2726) and decoder::expand_hypothesis_without_fsa,
 * finish_current_hypotheses, output_k_best_hypotheses (src/decoder.h:1157-1315, 672-688, 1386-1463).
 * The reference decodes one sentence at a time; results equal n_sent independent decodes.
 * src_ids: concatenated reversed source ids; src_len[n_sent]; beam (-b) is capped at floor(sqrt(V_tgt)) as in the
 * reference and must then be at most 32 (ZRNN_E_ARG beyond);
 * k_best (-k n-best count); min_ratio/max_ratio (--dec-ratio); penalty (--penalty); longest_sent (-L).
 * Outputs (host): out_ids [n_sent*k_best*(longest_sent+4)] padded with -1, out_len [n_sent*k_best]
 * (0 = fewer than k hypotheses passed the length filter), out_score [n_sent*k_best]. */
int zrnn_beam_decode_batch(zrnn_model* m, const int* src_ids, const int* src_len, int n_sent, int beam, int k_best,
                           float min_ratio, float max_ratio, float penalty, int longest_sent, int* out_ids,
                           int* out_len, float* out_score);
/* Same with the source ids already resident on the device (padded [S_max*n_sent], reversed, left-padded
 * with -1) and results left in device buffers; asynchronous on `stream`. */
int zrnn_beam_decode_batch_device(zrnn_model* m, const int* d_src_ids_padded, const int* h_src_len, int S_max,
                                  int n_sent, int beam, int k_best, float min_ratio, float max_ratio, float penalty,
                                  int longest_sent, int* d_out_ids, int* d_out_len, float* d_out_score, void* stream);
/* The same two calls with viterbi-alignment tracking for UNK replacement (BZ_CUDA::unk_replacement,
 * src/attention_node.hpp:225-234; src/decoder.h:1266-1267, 1281-1282, 683-684): out_align has the shape of out_ids
 * and holds, for every position of every hypothesis, the source position (in the un-reversed sentence) that had the
 * largest attention weight at the step that produced the word; -20 at position 0, -1 without attention and under
 * the padding.  The reference writes align[j+1] for every hypothesis position j that holds <UNK> (id 2) to the
 * --UNK-decode file (src/decoder.h:1452-1459). */
int zrnn_beam_decode_batch_align(zrnn_model* m, const int* src_ids, const int* src_len, int n_sent, int beam,
                                 int k_best, float min_ratio, float max_ratio, float penalty, int longest_sent,
                                 int* out_ids, int* out_len, float* out_score, int* out_align);
int zrnn_beam_decode_batch_align_device(zrnn_model* m, const int* d_src_ids_padded, const int* h_src_len, int S_max,
                                        int n_sent, int beam, int k_best, float min_ratio, float max_ratio,
                                        float penalty, int longest_sent, int* d_out_ids, int* d_out_len,
                                        float* d_out_score, int* d_out_align, void* stream);
/* Ensemble decoding: ensemble_factory with several decoder_model_wrappers (src/ensemble_factory.hpp:13-118,
 * 583-765) and ensembles_models (:768-795).  Every model runs the same beam in lock step on its own source
 * sentences (src_ids[k], src_len[k]: the k-th model's reversed ids, --decode-main-data-files gives one file per
 * model); at every step the models' output distributions are averaged, renormalised and expanded once.  The models
 * must share the target vocabulary; length limits follow model 0's source lengths (:623, :637).  The reference puts
 * one model on each GPU; here all models of an ensemble sit on the current device (its memory holds them) and
 * sentences shard across devices as in the single-model path. */
int zrnn_beam_decode_ensemble(zrnn_model* const* models, int n_models, const int* const* src_ids,
                              const int* const* src_len, int n_sent, int beam, int k_best, float min_ratio,
                              float max_ratio, float penalty, int longest_sent, int* out_ids, int* out_len,
                              float* out_score);
/* The same with alignment tracking: the viterbi alignment of a step is the source position with the largest sum
 * over the models of the attention weight at that position (ensembles_models, src/ensemble_factory.hpp:798-834);
 * models without attention cast no vote.  out_align as in zrnn_beam_decode_batch_align. */
int zrnn_beam_decode_ensemble_align(zrnn_model* const* models, int n_models, const int* const* src_ids,
                                    const int* const* src_len, int n_sent, int beam, int k_best, float min_ratio,
                                    float max_ratio, float penalty, int longest_sent, int* out_ids, int* out_len,
                                    float* out_score, int* out_align);
/* Teacher-forced scoring over the ranks of a communicator.  Every rank passes the SAME host batch and receives the
 * whole result.  The recurrent stack and the attention run data-parallel over the batch columns (rank r takes
 * columns [B r / world, B (r + 1) / world)); the top hidden states are all-gathered; every rank scores all columns
 * against its rows of D; a second all-gather of (max, sum, target logit) per column and the combine follow.
 * Results equal zrnn_score_batch's of the unsharded model to fp32 rounding of the normaliser. */
int zrnn_score_batch_sharded(zrnn_model* m, zrnn_comm* c, const int* src_ids, int S_max, const int* tgt_in,
                             const int* tgt_out, int T, int B, float* logp_out, double* total_logp);
/* zrnn_beam_decode_batch over the ranks of a communicator: every rank runs the (replicated) recurrent stack and the
 * attention on the same hypotheses, the softmax's pre-selection is vocabulary-sharded (zrnn_softmax_topk_sharded),
 * and every rank returns the same hypotheses. */
int zrnn_beam_decode_batch_sharded(zrnn_model* m, zrnn_comm* c, const int* src_ids, const int* src_len, int n_sent,
                                   int beam, int k_best, float min_ratio, float max_ratio, float penalty,
                                   int longest_sent, int* out_ids, int* out_len, float* out_score);
int zrnn_model_destroy(zrnn_model* m);

#ifdef __cplusplus
}
#endif
#endif /* ZRNN_H */
