// CPU oracle for the Zoph_RNN inference forward path.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
// against (tests, the smoke check and the CPU-baseline leg of the benchmark).  It is
// never linked into, imported by or executed from the product library.
//
// Parity status: the reference project ships no golden vectors, known-answer tests or
// CPU implementation for this path and its CUDA 7.5 / cuDNN v4 / Eigen / Boost build
// cannot be compiled for this machine, so this oracle is "parity unpinned" by the
// reference's own tests.  It is instead cross-checked against a second, independent
// float64 NumPy restatement (oracle/ref_numpy.py) and against committed golden files.
//
// Everything here is a plain-loop restatement of the arithmetic of the reference's
// kernels and drivers.  Matrices are column-major as in the reference
// (IDX2C(i,j,ld) = j*ld+i, src/BZ_CUDA_UTIL.h:26): activations are H x B, embeddings
// H x V, softmax weights V x H.  Token ids are int32, time-major idx[b + t*B].
//
// Build: see oracle/Makefile (g++ -O3 -march=x86-64-v3 -fopenmp -shared).
#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <queue>
#include <type_traits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---------------------------------------------------------------------------------
// GEMM helpers.  The reference calls cublasSgemm (src/BZ_CUDA_UTIL.h:691-696), a plain
// fp32 product whose summation order is unspecified; the oracle accumulates in double
// (default) and rounds once to float, or in float when g_acc_float is set (used when the
// oracle is timed as the CPU baseline).
// ---------------------------------------------------------------------------------
bool g_acc_float = false;
// Summation order of the float accumulation (cublasSgemm leaves it unspecified): 0 = k ascending, 1 = k descending,
// 2 = blocks of 32 k summed separately and then added (how a tiled / split-K kernel sums).  The spread of the results
// over these orders is the fp32 noise floor of an input.
int g_acc_order = 0;
// Test aid: when on, every local-p attention call appends its columns' window positions p_t (NaN for a masked column).
// The window is cut at (int)p_t, a discontinuity: two correct fp32 implementations may land on different sides of an
// integer when p_t is within rounding of it, so parity checks need to know how close each decision was.
bool g_pt_log_on = false;
std::vector<float> g_pt_log;

template <class Acc>
void gemm_nn_t(int M, int N, int K, const float* A, int lda, const float* B, int ldb, float* C, int ldc) {
  const int MB = 128, NB = 8;
  const int nmb = (M + MB - 1) / MB, nnb = (N + NB - 1) / NB;
#pragma omp parallel for collapse(2) schedule(static)
  for (int nb = 0; nb < nnb; ++nb) {
    for (int mb = 0; mb < nmb; ++mb) {
      const int n0 = nb * NB, m0 = mb * MB;
      const int nn = std::min(NB, N - n0), mm = std::min(MB, M - m0);
      Acc acc[NB][MB];
      for (int j = 0; j < nn; ++j)
        for (int i = 0; i < mm; ++i) acc[j][i] = 0;
      const int order = std::is_same<Acc, float>::value ? g_acc_order : 0;
      Acc tot[NB][MB];
      if (order == 2)
        for (int j = 0; j < nn; ++j)
          for (int i = 0; i < mm; ++i) tot[j][i] = 0;
      for (int kk = 0; kk < K; ++kk) {
        const int k = order == 1 ? K - 1 - kk : kk;
        const float* a = A + (size_t)k * lda + m0;
        for (int j = 0; j < nn; ++j) {
          const Acc b = B[(size_t)(n0 + j) * ldb + k];
          Acc* ac = acc[j];
          for (int i = 0; i < mm; ++i) ac[i] += (Acc)a[i] * b;
        }
        if (order == 2 && ((kk & 31) == 31 || kk == K - 1))
          for (int j = 0; j < nn; ++j)
            for (int i = 0; i < mm; ++i) { tot[j][i] += acc[j][i]; acc[j][i] = 0; }
      }
      for (int j = 0; j < nn; ++j)
        for (int i = 0; i < mm; ++i) C[(size_t)(n0 + j) * ldc + m0 + i] = (float)(order == 2 ? tot[j][i] : acc[j][i]);
    }
  }
}

// C[M x N] = A[M x K] * B[K x N]
void gemm_nn(int M, int N, int K, const float* A, int lda, const float* B, int ldb, float* C, int ldc) {
  if (g_acc_float) gemm_nn_t<float>(M, N, K, A, lda, B, ldb, C, ldc);
  else gemm_nn_t<double>(M, N, K, A, lda, B, ldb, C, ldc);
}

// C[M x N] = A^T * B with A stored K x M (column-major, lda = K)
void gemm_tn(int M, int N, int K, const float* A, int lda, const float* B, int ldb, float* C, int ldc) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < N; ++n)
    for (int m = 0; m < M; ++m) {
      const float* a = A + (size_t)m * lda;
      const float* b = B + (size_t)n * ldb;
      if (g_acc_float) {
        float s = 0;
        if (g_acc_order == 1) {
          for (int k = K - 1; k >= 0; --k) s += a[k] * b[k];
        } else if (g_acc_order == 2) {
          float blk = 0;
          for (int k = 0; k < K; ++k) {
            blk += a[k] * b[k];
            if ((k & 31) == 31 || k == K - 1) { s += blk; blk = 0; }
          }
        } else {
          for (int k = 0; k < K; ++k) s += a[k] * b[k];
        }
        C[(size_t)n * ldc + m] = s;
      } else {
        double s = 0;
        for (int k = 0; k < K; ++k) s += (double)a[k] * (double)b[k];
        C[(size_t)n * ldc + m] = (float)s;
      }
    }
}

// ---------------------------------------------------------------------------------
// Model description
// ---------------------------------------------------------------------------------
enum { ATT_NONE = 0, ATT_LOCAL_P = 1, ATT_GLOBAL_DOT = 2 };

struct Cfg {
  int num_layers, H, V_src, V_tgt, lm, attention, feed_input, D;
};

// One LSTM layer in the order the reference writes/reads it
// (src/Input_To_Hidden_Layer.hpp:1104-1143, src/Hidden_To_Hidden_Layer.hpp:704-729).
struct LstmW {
  const float *W_hi = 0, *b_i = 0, *W_hf = 0, *b_f = 0, *W_hc = 0, *b_c = 0, *W_ho = 0, *b_o = 0;
  const float* W = 0;  // embedding H x V (layer 0 only)
  const float *M_i = 0, *M_f = 0, *M_o = 0, *M_c = 0;
  const float *Q_i = 0, *Q_f = 0, *Q_o = 0, *Q_c = 0;  // feed-input (target layer 0 only)
};
// src/attention_layer.hpp:485-491
struct AttW {
  const float *W_a = 0, *W_p = 0, *v_p = 0, *output_bias = 0, *W_c_p1 = 0, *W_c_p2 = 0;
};

struct TensorSlot {
  int rows, cols;
  const float** dst;
};

struct Model {
  Cfg cfg;
  std::vector<LstmW> src, tgt;
  AttW att;
  const float *D = 0, *b_d = 0;
  std::vector<TensorSlot> slots;
  std::vector<std::vector<float>> storage;
};

void add_lstm_slots(Model& m, LstmW& w, int H, int V_emb, bool feed) {
  auto add = [&](int r, int c, const float** p) { m.slots.push_back({r, c, p}); };
  add(H, H, &w.W_hi); add(H, 1, &w.b_i);
  add(H, H, &w.W_hf); add(H, 1, &w.b_f);
  add(H, H, &w.W_hc); add(H, 1, &w.b_c);
  add(H, H, &w.W_ho); add(H, 1, &w.b_o);
  if (V_emb > 0) add(H, V_emb, &w.W);
  add(H, H, &w.M_i); add(H, H, &w.M_f); add(H, H, &w.M_o); add(H, H, &w.M_c);
  if (feed) { add(H, H, &w.Q_i); add(H, H, &w.Q_f); add(H, H, &w.Q_o); add(H, H, &w.Q_c); }
}

void add_att_slots(Model& m, int H) {
  auto add = [&](int r, int c, const float** p) { m.slots.push_back({r, c, p}); };
  add(H, H, &m.att.W_a); add(H, H, &m.att.W_p); add(1, H, &m.att.v_p);
  add(H, 1, &m.att.output_bias); add(H, H, &m.att.W_c_p1); add(H, H, &m.att.W_c_p2);
}

// Tensor order of the weight file (src/model.hpp:2172-2241).
void build_slots(Model& m) {
  const Cfg& c = m.cfg;
  m.src.resize(c.lm ? 0 : c.num_layers);
  m.tgt.resize(c.num_layers);
  if (!c.lm)
    for (int l = 0; l < c.num_layers; ++l) add_lstm_slots(m, m.src[l], c.H, l == 0 ? c.V_src : 0, false);
  for (int l = 0; l < c.num_layers; ++l) {
    add_lstm_slots(m, m.tgt[l], c.H, l == 0 ? c.V_tgt : 0, l == 0 && c.feed_input && c.attention);
    if (c.attention && l == c.num_layers - 1) add_att_slots(m, c.H);
  }
  m.slots.push_back({c.V_tgt, c.H, &m.D});
  m.slots.push_back({c.V_tgt, 1, &m.b_d});
}

// ---------------------------------------------------------------------------------
// Kernel-level restatements
// ---------------------------------------------------------------------------------

// vocab_to_01 / vocab_to_nonM1 (src/custom_kernels.h:9-32)
inline int id_mask(int id) { return id == -1 ? 0 : 1; }
inline int id_nonm1(int id) { return id == -1 ? 0 : id; }

// sparse_lookup_kernel (src/custom_kernels.h:340-348): x[:,b] = W[:,id_b], a bit copy.
void gather(const float* W, int H, const int* ids, int n, float* x) {
  for (int b = 0; b < n; ++b) std::memcpy(x + (size_t)b * H, W + (size_t)ids[b] * H, sizeof(float) * H);
}

// One LSTM cell: src/LSTM.hpp:133-399 / src/LSTM_HH.hpp:130-317 with the element-wise
// kernels of src/custom_kernels.h:57-192.  `htild` non-null means the feed-input term
// Q_g*htild is added (the reference skips it when the node index is 0, LSTM.hpp:154,175).
// Non-feed gates use float expf/tanhf (ck:57-65,105-113); feed gates evaluate exp in
// double (ck:90-99) and tanhf (ck:126-135).
void lstm_cell(int H, int B, const LstmW& w, const float* x, const float* h_prev, const float* c_prev,
               const float* htild, const int* mask, float* h_out, float* c_out, std::vector<float>& scratch) {
  const size_t HB = (size_t)H * B;
  scratch.resize(HB * 12);
  float* t = scratch.data();
  const float* Ms[4] = {w.M_i, w.M_f, w.M_c, w.M_o};
  const float* Ws[4] = {w.W_hi, w.W_hf, w.W_hc, w.W_ho};
  const float* Qs[4] = {w.Q_i, w.Q_f, w.Q_c, w.Q_o};
  const float* bs[4] = {w.b_i, w.b_f, w.b_c, w.b_o};
  for (int g = 0; g < 4; ++g) {
    gemm_nn(H, B, H, Ms[g], H, x, H, t + HB * (3 * g + 0), H);
    gemm_nn(H, B, H, Ws[g], H, h_prev, H, t + HB * (3 * g + 1), H);
    if (htild) gemm_nn(H, B, H, Qs[g], H, htild, H, t + HB * (3 * g + 2), H);
  }
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b) {
    for (int i = 0; i < H; ++i) {
      const size_t idx = (size_t)b * H + i;
      float gate[4];
      for (int g = 0; g < 4; ++g) {
        float v;
        if (htild) v = t[HB * (3 * g) + idx] + t[HB * (3 * g + 1) + idx] + t[HB * (3 * g + 2) + idx] + bs[g][i];
        else v = t[HB * (3 * g) + idx] + t[HB * (3 * g + 1) + idx] + bs[g][i];
        if (g == 2) gate[g] = tanhf(v);
        else if (htild) gate[g] = (float)(1.0 / (1.0 + std::exp(-1.0 * (double)v)));
        else gate[g] = 1.0f / (1.0f + expf(-1.0f * v));
      }
      float c = gate[1] * c_prev[idx] + gate[0] * gate[2];  // forward_c_t_kernel ck:139-147
      float h = gate[3] * tanhf(c);                          // forward_h_t_kernel ck:160-168
      h = h * mask[b];                                       // zero_c_t_and_h_t ck:182-192
      c = c * mask[b];
      h_out[idx] = h;
      c_out[idx] = c;
    }
  }
}

// Attention forward for one target step.
//  type ATT_LOCAL_P  : src/attention_node.hpp:73-394 with src/custom_kernels.h:1566-1613,
//                      1649-1713, 1750-1813, 1842-1848, 1890-1925, 2210-2217.
//  type ATT_GLOBAL_DOT: extension (not in the reference): e_s = hs_s . h over every valid
//                      source position, standard softmax, same tanh combiner.
// hs_all: S_max slots of H x B (slot = source time step as the encoder ran it, i.e. reversed
// and left-padded).  Source position idx of sentence b lives in slot len_b-1-idx+offset_b
// (ck:1704).  align_out (optional): for local-p (2D+1) x B weights stored [j*B+b] plus the
// index table idx_out[j*B+b]; for global S_max x B stored [s*B+b] (position order).
void attention(int type, int H, int B, int D, const AttW& w, const float* h_t, const int* mask,
               const float* hs_all, int S_max, const int* len, const int* offset, float* htild_out,
               float* align_out, int* idx_out, int* viterbi_out = nullptr, float viterbi_init = -1.f) {
  const size_t HB = (size_t)H * B;
  std::vector<float> c_t(HB, 0.f), tmp1(HB), tmp2(HB);
  if (type == ATT_LOCAL_P) {
    const int Wn = 2 * D + 1;
    std::vector<float> tanh1(HB), sig(B), p_t(B), q(HB), align((size_t)Wn * B), hs((size_t)Wn * HB);
    std::vector<int> ind((size_t)Wn * B);
    gemm_nn(H, B, H, w.W_p, H, h_t, H, tanh1.data(), H);
    for (size_t i = 0; i < HB; ++i) tanh1[i] = tanhf(tanh1[i]);  // tanh_kernel ck:1566-1571
    gemm_nn(1, B, H, w.v_p, 1, tanh1.data(), H, sig.data(), 1);
    for (int b = 0; b < B; ++b) {
      sig[b] = (float)(1.0 / (1.0 + std::exp(-1.0 * (double)sig[b])));  // sigmoid_kernel ck:1581-1587
      p_t[b] = len[b] * sig[b];                                           // alignment_pos_kernel ck:1596-1603
      const int ip = (int)p_t[b];                                         // lower_upper_kernel ck:1606-1613
      if (g_pt_log_on) g_pt_log.push_back(mask[b] == 1 ? p_t[b] : NAN);
      const int lo = (0 > ip - D) ? 0 : (ip - D);
      const int hi = ((len[b] - 1) < ip + D) ? (len[b] - 1) : (ip + D);
      int cur = lo;  // create_indicies_kernel ck:1649-1673
      for (int j = 0; j < Wn; ++j) {
        if (mask[b] == 1) ind[(size_t)j * B + b] = (cur > hi) ? -1 : cur;
        else ind[(size_t)j * B + b] = -1;
        cur++;
      }
    }
    // load_in_hs_kernel ck:1692-1713
    for (int j = 0; j < Wn; ++j)
      for (int b = 0; b < B; ++b) {
        float* dst = hs.data() + (size_t)j * HB + (size_t)b * H;
        const int si = ind[(size_t)j * B + b];
        if (si != -1) {
          const int slot = len[b] - 1 - si + offset[b];
          std::memcpy(dst, hs_all + (size_t)slot * HB + (size_t)b * H, sizeof(float) * H);
        } else {
          std::memset(dst, 0, sizeof(float) * H);
        }
      }
    gemm_tn(H, B, H, w.W_a, H, h_t, H, q.data(), H);  // attention_node.hpp:195
    // elem_reduce_kernel_large ck:1890-1925
    for (int j = 0; j < Wn; ++j)
      for (int b = 0; b < B; ++b) {
        const float* a = hs.data() + (size_t)j * HB + (size_t)b * H;
        const float* qq = q.data() + (size_t)b * H;
        double s = 0;
        for (int i = 0; i < H; ++i) s += (double)a[i] * (double)qq[i];
        align[(size_t)j * B + b] = (float)s;
      }
    // alignment_reduction_kernel ck:1750-1794 (max starts at 0, Gaussian not renormalised)
    const float sigma_sq = (float)((D * D) / 4.0);
    for (int b = 0; b < B; ++b) {
      float sum = 0, max_val = 0;
      for (int j = 0; j < Wn; ++j)
        if (ind[(size_t)j * B + b] != -1 && align[(size_t)j * B + b] > max_val) max_val = align[(size_t)j * B + b];
      for (int j = 0; j < Wn; ++j) {
        float& a = align[(size_t)j * B + b];
        if (ind[(size_t)j * B + b] != -1) { a = expf(a - max_val); sum += a; }
        else a = 0;
      }
      for (int j = 0; j < Wn; ++j) {
        float& a = align[(size_t)j * B + b];
        if (ind[(size_t)j * B + b] != -1) {
          const float d = p_t[b] - ind[(size_t)j * B + b];
          const float temp = expf((-1 * powf(d, 2.0f)) / (2 * sigma_sq));
          if (sum != 0) a = (a / sum) * temp;
        } else a = 0;
      }
    }
    // get_viterbi_alignment_kernel ck:1621-1635 (attention_node.hpp:225-234): the window index of the largest
    // weight; the running maximum starts at -1 and only a strictly larger weight replaces it.  The decoder then
    // re-derives the index from the weights per source position with a maximum that starts at 0
    // (ensembles_models, ensemble_factory.hpp:812-834): viterbi_init = 0 gives that result.
    if (viterbi_out)
      for (int b = 0; b < B; ++b) {
        float max_val = viterbi_init;
        int max_index = -1;
        for (int j = 0; j < Wn; ++j)
          if (max_val < align[(size_t)j * B + b]) { max_val = align[(size_t)j * B + b]; max_index = ind[(size_t)j * B + b]; }
        viterbi_out[b] = max_index;
      }
    // create_c_t_kernel ck:1802-1813
    for (int b = 0; b < B; ++b)
      for (int i = 0; i < H; ++i) {
        float acc = 0;
        for (int j = 0; j < Wn; ++j) acc += align[(size_t)j * B + b] * hs[(size_t)j * HB + (size_t)b * H + i];
        c_t[(size_t)b * H + i] = acc;
      }
    if (align_out) std::memcpy(align_out, align.data(), sizeof(float) * align.size());
    if (idx_out) std::memcpy(idx_out, ind.data(), sizeof(int) * ind.size());
  } else {
    for (int b = 0; b < B; ++b) {
      if (align_out) for (int s = 0; s < S_max; ++s) align_out[(size_t)s * B + b] = 0;
      if (viterbi_out) viterbi_out[b] = -1;
      if (mask[b] != 1) continue;
      const int L = len[b];
      std::vector<double> e(L);
      double mx = -DBL_MAX;
      for (int s = 0; s < L; ++s) {
        const float* hsv = hs_all + (size_t)(L - 1 - s + offset[b]) * HB + (size_t)b * H;
        double acc = 0;
        for (int i = 0; i < H; ++i) acc += (double)hsv[i] * (double)h_t[(size_t)b * H + i];
        e[s] = (float)acc;
        mx = std::max(mx, e[s]);
      }
      double sum = 0;
      for (int s = 0; s < L; ++s) { e[s] = std::exp(e[s] - mx); sum += e[s]; }
      std::vector<double> ctx(H, 0.0);
      float best = viterbi_init;
      for (int s = 0; s < L; ++s) {
        const float a = (float)(e[s] / sum);
        if (viterbi_out && best < a) { best = a; viterbi_out[b] = s; }  // same rule over every source position
        if (align_out) align_out[(size_t)s * B + b] = a;
        const float* hsv = hs_all + (size_t)(L - 1 - s + offset[b]) * HB + (size_t)b * H;
        for (int i = 0; i < H; ++i) ctx[i] += (double)a * (double)hsv[i];
      }
      for (int i = 0; i < H; ++i) c_t[(size_t)b * H + i] = (float)ctx[i];
    }
  }
  // combiner: attention_node.hpp:352-379, tanh_att_forward_kernel ck:1842-1848, zero_h_t ck:2210-2217
  gemm_nn(H, B, H, w.W_c_p1, H, c_t.data(), H, tmp1.data(), H);
  gemm_nn(H, B, H, w.W_c_p2, H, h_t, H, tmp2.data(), H);
  for (int b = 0; b < B; ++b)
    for (int i = 0; i < H; ++i) {
      const size_t idx = (size_t)b * H + i;
      htild_out[idx] = tanhf(tmp1[idx] + tmp2[idx] + w.output_bias[i]) * mask[b];
    }
}

// Scoring log-softmax: src/softmax.hpp:636-692, outputdist_perplexity_kernel ck:581-660,
// matrix_bias_kernel ck:785-794.  z = D*h + b_d in float, then double log-softmax.
// Returns only what the caller needs: logp of `target` per column (and optionally the
// whole V x N double matrix).
void softmax_logp(int V, int H, int N, const float* D, const float* b_d, const float* h, const int* target,
                  double* logp_target, double* logp_all) {
  const int NB = 64;
  std::vector<float> z((size_t)V * NB);
  for (int n0 = 0; n0 < N; n0 += NB) {
    const int nn = std::min(NB, N - n0);
    gemm_nn(V, nn, H, D, V, h + (size_t)n0 * H, H, z.data(), V);
#pragma omp parallel for schedule(static)
    for (int j = 0; j < nn; ++j) {
      float* zc = z.data() + (size_t)j * V;
      double mx = -DBL_MAX;
      for (int v = 0; v < V; ++v) { zc[v] = zc[v] + b_d[v]; if (mx < (double)zc[v]) mx = zc[v]; }
      double sum = 0;
      for (int v = 0; v < V; ++v) sum += std::exp((double)zc[v] - mx);
      const double lsum = std::log(sum);
      if (logp_all)
        for (int v = 0; v < V; ++v) logp_all[(size_t)(n0 + j) * V + v] = std::log(std::exp((double)zc[v] - mx)) - lsum;
      if (logp_target) {
        const int y = target[n0 + j];
        logp_target[n0 + j] = std::log(std::exp((double)zc[y] - mx)) - lsum;
      }
    }
  }
}

// Decode-time distribution: src/softmax.hpp:514-632, outputdist_overflow_prevention_kernel
// ck:501-577.  Float probabilities p = expf(z-max)/sum.
void softmax_dist(int V, int H, int N, const float* D, const float* b_d, const float* h, float* p) {
  gemm_nn(V, N, H, D, V, h, H, p, V);
#pragma omp parallel for schedule(static)
  for (int j = 0; j < N; ++j) {
    float* zc = p + (size_t)j * V;
    float mx = -FLT_MAX;
    for (int v = 0; v < V; ++v) { zc[v] = zc[v] + b_d[v]; if (mx < zc[v]) mx = zc[v]; }
    double sum = 0;  // the kernel tree-sums 256 float partials; double keeps the oracle order-free
    for (int v = 0; v < V; ++v) { zc[v] = expf(zc[v] - mx); sum += zc[v]; }
    const float fs = (float)sum;
    for (int v = 0; v < V; ++v) zc[v] = zc[v] / fs;
  }
}

// ---------------------------------------------------------------------------------
// Drivers
// ---------------------------------------------------------------------------------

// Teacher-forced scoring: neuralMT_model::getError, src/model.hpp:1463-1802, with
// softmax_layer::compute_loss_GPU src/softmax.hpp:867-900.
// src_ids: [S_max*B] reversed + left-padded with -1 (ignored for LM); tgt_in/tgt_out: [T*B]
// right-padded with -1.  logp_out[T*B]: per-token natural-log prob (0 where masked).
// hs_top_out (optional, [T*H*B]): the vectors handed to the softmax, for layer tests.
double score_batch(const Model& m, const int* src_ids, int S_max, const int* tgt_in, const int* tgt_out, int T,
                   int B, double* logp_out, float* hs_top_out) {
  const Cfg& c = m.cfg;
  const int H = c.H, L = c.num_layers;
  const size_t HB = (size_t)H * B;
  std::vector<float> scratch;
  std::vector<std::vector<float>> h(L, std::vector<float>(HB, 0.f)), cc(L, std::vector<float>(HB, 0.f));
  std::vector<float> x(HB), hn(HB), cn(HB);
  std::vector<int> ids(B), mask(B);
  std::vector<float> hs_all;  // top-layer source states per source time step
  std::vector<int> len(B, 0), off(B, 0);
  if (!c.lm) {
    hs_all.resize((size_t)S_max * HB);
    for (int b = 0; b < B; ++b) {
      int n = 0;
      for (int t = 0; t < S_max; ++t) n += id_mask(src_ids[b + (size_t)t * B]);
      len[b] = n;
      off[b] = S_max - n;  // src/fileHelper.h:480-496
    }
    for (int t = 0; t < S_max; ++t) {
      for (int b = 0; b < B; ++b) { ids[b] = id_nonm1(src_ids[b + (size_t)t * B]); mask[b] = id_mask(src_ids[b + (size_t)t * B]); }
      gather(m.src[0].W, H, ids.data(), B, x.data());
      for (int l = 0; l < L; ++l) {
        lstm_cell(H, B, m.src[l], l == 0 ? x.data() : h[l - 1].data(), h[l].data(), cc[l].data(), nullptr, mask.data(),
                  hn.data(), cn.data(), scratch);
        h[l] = hn; cc[l] = cn;
      }
      std::memcpy(hs_all.data() + (size_t)t * HB, h[L - 1].data(), sizeof(float) * HB);
    }
  }
  // target side starts from the source's final (h,c) per layer (model.hpp:1714-1724), zeros for LM
  std::vector<float> htild(HB, 0.f), top(HB);
  std::vector<int> tgt(B), omask(B);
  std::vector<double> lp(B);
  double total = 0;
  for (int t = 0; t < T; ++t) {
    for (int b = 0; b < B; ++b) { ids[b] = id_nonm1(tgt_in[b + (size_t)t * B]); mask[b] = id_mask(tgt_in[b + (size_t)t * B]); }
    gather(m.tgt[0].W, H, ids.data(), B, x.data());
    for (int l = 0; l < L; ++l) {
      const bool feed = (l == 0 && c.feed_input && c.attention && t != 0);
      lstm_cell(H, B, m.tgt[l], l == 0 ? x.data() : h[l - 1].data(), h[l].data(), cc[l].data(),
                feed ? htild.data() : nullptr, mask.data(), hn.data(), cn.data(), scratch);
      h[l] = hn; cc[l] = cn;
    }
    if (c.attention) {
      attention(c.attention, H, B, c.D, m.att, h[L - 1].data(), mask.data(), hs_all.data(), S_max, len.data(),
                off.data(), htild.data(), nullptr, nullptr);
      top = htild;
    } else top = h[L - 1];
    if (hs_top_out) std::memcpy(hs_top_out + (size_t)t * HB, top.data(), sizeof(float) * HB);
    for (int b = 0; b < B; ++b) { tgt[b] = id_nonm1(tgt_out[b + (size_t)t * B]); omask[b] = id_mask(tgt_out[b + (size_t)t * B]); }
    softmax_logp(c.V_tgt, H, B, m.D, m.b_d, top.data(), tgt.data(), lp.data(), nullptr);
    for (int b = 0; b < B; ++b) {
      const double v = omask[b] == 1 ? lp[b] : 0.0;
      if (logp_out) logp_out[b + (size_t)t * B] = v;
      total += v;
    }
  }
  return total;
}

// Beam search for ONE source sentence exactly as the reference runs it (source minibatch 1,
// target minibatch = beam): ensemble_factory::decode_file_batch src/ensemble_factory.hpp:583-765,
// forward_prop_source / forward_prop_target / swap_decoding_states src/model.hpp:2367-2452,
// 2573-2726, decoder::expand_hypothesis_without_fsa src/decoder.h:1157-1315,
// finish_current_hypotheses :672-688, output_k_best_hypotheses :1386-1463.
struct Hyp { std::vector<int> ids; std::vector<int> align; float score; };

// Per-model decoder state: encoder outputs for one sentence and the recurrent state of `beam` columns.
struct DecModel {
  const Model* m;
  int S, beam;
  std::vector<std::vector<float>> hs, cs, h, cc, hp, cp;
  std::vector<float> hs_all, x, htild, htild_feed, P;
  std::vector<int> ones, ids, lenv, offv, vit;
  std::vector<float> scratch;
  // attention weight per source position and beam column of the last forward step, [pos * beam + j]
  // (BZ_CUDA::alignment_scores, attention_node.hpp:236-262); all zero without attention
  std::vector<float> pos_score;

  void encode(const int* src) {
    const Cfg& c = m->cfg;
    const int H = c.H, L = c.num_layers;
    const size_t HB = (size_t)H * beam;
    hs.assign(L, std::vector<float>(H, 0.f)); cs.assign(L, std::vector<float>(H, 0.f));
    std::vector<float> x1(H), hn1(H), cn1(H);
    hs_all.resize((size_t)S * HB);  // top source state replicated per beam column (model.hpp:2434-2445)
    const int one = 1;
    for (int t = 0; t < S; ++t) {
      const int id = id_nonm1(src[t]);
      gather(m->src[0].W, H, &id, 1, x1.data());
      for (int l = 0; l < L; ++l) {
        lstm_cell(H, 1, m->src[l], l == 0 ? x1.data() : hs[l - 1].data(), hs[l].data(), cs[l].data(), nullptr, &one,
                  hn1.data(), cn1.data(), scratch);
        hs[l] = hn1; cs[l] = cn1;
      }
      for (int j = 0; j < beam; ++j) std::memcpy(hs_all.data() + (size_t)t * HB + (size_t)j * H, hs[L - 1].data(), sizeof(float) * H);
    }
    h.assign(L, std::vector<float>(HB)); cc.assign(L, std::vector<float>(HB));
    hp.assign(L, std::vector<float>(HB)); cp.assign(L, std::vector<float>(HB));
    x.resize(HB); htild.assign(HB, 0.f); htild_feed.assign(HB, 0.f); P.resize((size_t)c.V_tgt * beam);
    ones.assign(beam, 1); ids.resize(beam); lenv.assign(beam, S); offv.assign(beam, 0);
    // viterbi alignment per beam column of the last forward step (BZ_CUDA::viterbi_alignments; -1 without attention,
    // decoder.h:1174-1178)
    vit.assign(beam, -1);
    pos_score.assign((size_t)S * beam, 0.f);
  }
  void forward(int idx, const std::vector<int>& cur) {
    const Cfg& c = m->cfg;
    const int H = c.H, L = c.num_layers, V = c.V_tgt;
    if (idx == 0)  // transfer_decoding_states_GPU: replicate the source's last (h,c) over the beam
      for (int l = 0; l < L; ++l)
        for (int j = 0; j < beam; ++j) {
          std::memcpy(hp[l].data() + (size_t)j * H, hs[l].data(), sizeof(float) * H);
          std::memcpy(cp[l].data() + (size_t)j * H, cs[l].data(), sizeof(float) * H);
        }
    for (int j = 0; j < beam; ++j) ids[j] = cur[j] < 0 ? 0 : cur[j];
    gather(m->tgt[0].W, H, ids.data(), beam, x.data());
    for (int l = 0; l < L; ++l) {
      const bool feed = (l == 0 && c.feed_input && c.attention && idx != 0);
      lstm_cell(H, beam, m->tgt[l], l == 0 ? x.data() : h[l - 1].data(), hp[l].data(), cp[l].data(),
                feed ? htild_feed.data() : nullptr, ones.data(), h[l].data(), cc[l].data(), scratch);
    }
    const float* top = h[L - 1].data();
    if (c.attention) {
      const int Wn = 2 * c.D + 1;
      std::vector<float> al((size_t)std::max(Wn, S) * beam, 0.f);
      std::vector<int> ix((size_t)Wn * beam, -1);
      attention(c.attention, H, beam, c.D, m->att, h[L - 1].data(), ones.data(), hs_all.data(), S, lenv.data(),
                offv.data(), htild.data(), al.data(), ix.data(), vit.data(), 0.f);
      std::fill(pos_score.begin(), pos_score.end(), 0.f);
      if (c.attention == ATT_LOCAL_P) {
        for (int j = 0; j < Wn; ++j)
          for (int b = 0; b < beam; ++b) {
            const int pos = ix[(size_t)j * beam + b];
            if (pos >= 0) pos_score[(size_t)pos * beam + b] = al[(size_t)j * beam + b];
          }
      } else {
        for (int p2 = 0; p2 < S; ++p2)
          for (int b = 0; b < beam; ++b) pos_score[(size_t)p2 * beam + b] = al[(size_t)p2 * beam + b];
      }
      top = htild.data();
    }
    softmax_dist(V, H, beam, m->D, m->b_d, top, P.data());
  }
  // swap_decoding_states + target_copy_prev_states (model.hpp:2691-2726)
  void reorder(const std::vector<int>& changes) {
    const Cfg& c = m->cfg;
    const int H = c.H, L = c.num_layers;
    for (int l = 0; l < L; ++l)
      for (int j = 0; j < beam; ++j) {
        std::memcpy(hp[l].data() + (size_t)j * H, h[l].data() + (size_t)changes[j] * H, sizeof(float) * H);
        std::memcpy(cp[l].data() + (size_t)j * H, cc[l].data() + (size_t)changes[j] * H, sizeof(float) * H);
      }
    if (c.feed_input && c.attention)
      for (int j = 0; j < beam; ++j)
        std::memcpy(htild_feed.data() + (size_t)j * H, htild.data() + (size_t)changes[j] * H, sizeof(float) * H);
  }
};

// models.size() > 1: ensemble decoding, ensemble_factory::ensembles_models src/ensemble_factory.hpp:768-795 (the
// distributions are averaged in double, stored as float, then every column is divided by its sum); each model reads
// its own source sentence, the length limits follow model 0's (:623, :637).
void beam_decode_one(const std::vector<const Model*>& models, const std::vector<const int*>& srcs,
                     const std::vector<int>& Ss, int beam, int k_best, float min_ratio, float max_ratio,
                     float penalty, int longest_sent_internal, std::vector<Hyp>& out, float* margin_out = nullptr) {
  // margin_out (test aid, no counterpart in the reference): the smallest score difference that decided anything in
  // this search - at every step between the last candidate that entered the beam (or finished) and the best one that
  // did not, and at the end between the best and the second-best hypothesis.  A search whose margin is below the
  // arithmetic noise of another implementation may legitimately come out differently there.
  float margin = 3.0e38f;
  const int K = (int)models.size();
  const int V = models[0]->cfg.V_tgt, S = Ss[0];
  const int START = 0, END = 1, INVALID = -1;
  if (beam > (int)std::sqrt((double)V)) beam = (int)std::sqrt((double)V);  // ensemble_factory.hpp:19-21
  std::vector<DecModel> dm(K);
  for (int k = 0; k < K; ++k) { dm[k].m = models[k]; dm[k].S = Ss[k]; dm[k].beam = beam; dm[k].encode(srcs[k]); }
  // ---- decoder state (decoder.h:1317-1337)
  const int Lmax = longest_sent_internal;
  std::vector<int> top_sent((size_t)beam * Lmax, START), top_tmp((size_t)beam * Lmax, START);
  std::vector<float> scores(beam, 0.f), scores_tmp(beam, 0.f);
  std::vector<int> cur(beam, START), changes(beam, 0);
  std::vector<Hyp> hyps;
  int current_index = 0;
  std::vector<float> Pens;
  // alignment per position of every beam entry (top_sentences_viterbi, initialised to -20, :1335)
  std::vector<int> top_vit((size_t)beam * Lmax, -20), top_vit_tmp((size_t)beam * Lmax, -20);
  const float* Pp = nullptr;
  const int* vitp = nullptr;
  std::vector<int> ens_vit;

  auto forward_target = [&](int idx) {
    for (int k = 0; k < K; ++k) dm[k].forward(idx, cur);
    vitp = dm[0].vit.data();
    if (K == 1) { Pp = dm[0].P.data(); return; }
    // alignment voting (ensemble_factory.hpp:798-834): sum the models' weights per source position, take the largest
    // (the running maximum starts at 0: -1 when every sum is zero)
    ens_vit.assign(beam, -1);
    int smax = 0;
    for (int k = 0; k < K; ++k) smax = std::max(smax, dm[k].S);
    for (int j = 0; j < beam; ++j) {
      float best = 0.f;
      for (int p2 = 0; p2 < smax; ++p2) {
        float sum = 0.f;
        for (int k = 0; k < K; ++k)
          if (p2 < dm[k].S) sum += dm[k].pos_score[(size_t)p2 * beam + j];
        if (sum > best) { best = sum; ens_vit[j] = p2; }
      }
    }
    vitp = ens_vit.data();
    Pens.resize((size_t)V * beam);
    for (int j = 0; j < beam; ++j) {
      float norm = 0.f;
      for (int i = 0; i < V; ++i) {
        double t = 0;
        for (int k = 0; k < K; ++k) t += dm[k].P[(size_t)j * V + i];
        Pens[(size_t)j * V + i] = (float)(t / K);
        norm += Pens[(size_t)j * V + i];
      }
      for (int i = 0; i < V; ++i) Pens[(size_t)j * V + i] = Pens[(size_t)j * V + i] / norm;
    }
    Pp = Pens.data();
  };

  struct Cand { float val; int beam_idx; int vocab; };
  auto cand_less = [](const Cand& a, const Cand& b) { return a.val < b.val; };

  const int max_steps = std::min((int)(max_ratio * S), Lmax - 2);
  int last_index = 0;
  for (int step = 0; step < max_steps; ++step) {
    forward_target(step);
    // ---- expand_hypothesis_without_fsa
    const int cols = (step == 0) ? 1 : beam;
    std::priority_queue<Cand, std::vector<Cand>, decltype(cand_less)> global(cand_less);
    for (int i = 0; i < cols; ++i) {
      if (cur[i] == INVALID) break;
      // keep the beam+1 largest probabilities of column i
      auto greater_p = [](const std::pair<float, int>& a, const std::pair<float, int>& b) { return a.first > b.first; };
      std::priority_queue<std::pair<float, int>, std::vector<std::pair<float, int>>, decltype(greater_p)> pq(greater_p);
      const float* col = Pp + (size_t)i * V;
      for (int j = 0; j < V; ++j) {
        if ((int)pq.size() < beam + 1) pq.push({col[j], j});
        else if (col[j] > pq.top().first) { pq.pop(); pq.push({col[j], j}); }
      }
      while (!pq.empty()) {
        global.push({std::log(pq.top().first) + scores[i], i, pq.top().second});
        pq.pop();
      }
    }
    int i = 0;
    while (i < beam) {
      if (global.empty()) {
        std::memcpy(&top_tmp[(size_t)i * Lmax], &top_sent[0], sizeof(int) * Lmax);
        std::memcpy(&top_vit_tmp[(size_t)i * Lmax], &top_vit[0], sizeof(int) * Lmax);  // decoder.h:1237
        top_tmp[(size_t)i * Lmax + current_index + 1] = START;
        cur[i] = INVALID; changes[i] = 0; scores_tmp[i] = 0;
        ++i;
        continue;
      }
      Cand t = global.top();
      global.pop();
      if (t.vocab == START) continue;
      if (t.vocab == END) {
        Hyp hy;
        hy.ids.assign(&top_sent[(size_t)t.beam_idx * Lmax], &top_sent[(size_t)t.beam_idx * Lmax] + current_index + 2);
        hy.ids[current_index + 1] = END;
        hy.align.assign(&top_vit[(size_t)t.beam_idx * Lmax], &top_vit[(size_t)t.beam_idx * Lmax] + current_index + 2);
        hy.align[current_index + 1] = vitp[t.beam_idx];  // decoder.h:1266-1267
        hy.score = t.val + penalty;
        hyps.push_back(hy);
      } else {
        std::memcpy(&top_tmp[(size_t)i * Lmax], &top_sent[(size_t)t.beam_idx * Lmax], sizeof(int) * Lmax);
        top_tmp[(size_t)i * Lmax + current_index + 1] = t.vocab;
        std::memcpy(&top_vit_tmp[(size_t)i * Lmax], &top_vit[(size_t)t.beam_idx * Lmax], sizeof(int) * Lmax);
        top_vit_tmp[(size_t)i * Lmax + current_index + 1] = vitp[t.beam_idx];  // decoder.h:1281-1282
        cur[i] = t.vocab; changes[i] = t.beam_idx; scores_tmp[i] = t.val + penalty;
        ++i;
        if (i == beam) {  // the beam is full: the best candidate left behind (never <START>) is the runner-up
          while (!global.empty() && global.top().vocab == START) global.pop();
          if (!global.empty()) margin = std::min(margin, t.val - global.top().val);
        }
      }
    }
    top_sent = top_tmp; top_vit = top_vit_tmp; scores = scores_tmp; current_index += 1;
    for (int k = 0; k < K; ++k) dm[k].reorder(changes);
    last_index = step;
  }
  forward_target(last_index + 1);
  // ---- finish_current_hypotheses (decoder.h:672-688)
  for (int i = 0; i < beam; ++i) {
    if (cur[i] == INVALID) continue;
    top_sent[(size_t)i * Lmax + current_index + 1] = END;
    scores[i] += std::log(Pp[(size_t)i * V + 1]) + penalty;
    Hyp hy;
    hy.ids.assign(&top_sent[(size_t)i * Lmax], &top_sent[(size_t)i * Lmax] + current_index + 2);
    hy.align.assign(&top_vit[(size_t)i * Lmax], &top_vit[(size_t)i * Lmax] + current_index + 2);
    hy.align[current_index + 1] = vitp[i];  // decoder.h:683-684
    hy.score = scores[i];
    hyps.push_back(hy);
  }
  // ---- output_k_best_hypotheses (decoder.h:1386-1463)
  std::vector<int> order;
  for (size_t i = 0; i < hyps.size(); ++i) {
    const float ratio = ((float)hyps[i].ids.size()) / S;
    if (ratio > min_ratio) order.push_back((int)i);
  }
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return hyps[a].score > hyps[b].score; });
  out.clear();
  for (int i = 0; i < (int)order.size() && i < k_best; ++i) out.push_back(hyps[order[i]]);
  if (order.size() >= 2) margin = std::min(margin, hyps[order[0]].score - hyps[order[1]].score);
  if (margin_out) *margin_out = margin;
}

}  // namespace

// ---------------------------------------------------------------------------------
// C API (ctypes)
// ---------------------------------------------------------------------------------
extern "C" {

// on: 0 = double accumulation, 1 / 2 / 3 = float accumulation with k ascending / descending / in blocks of 32
void orc_set_acc_float(int on) { g_acc_float = on != 0; g_acc_order = on > 1 ? on - 1 : 0; }
// window-position log of the local-p attention: start (clears), then read up to cap values; returns the count logged
void orc_pt_log_start(int on) { g_pt_log_on = on != 0; g_pt_log.clear(); }
int orc_pt_log_read(float* out, int cap) {
  const int n = (int)g_pt_log.size();
  for (int i = 0; i < n && i < cap; ++i) out[i] = g_pt_log[i];
  return n;
}
// n <= 0: leave the OpenMP default (OMP_NUM_THREADS or the core count)
void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
int orc_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// cfg = {num_layers, H, V_src, V_tgt, lm, attention, feed_input, D}
void* orc_model_create(const int* cfg) {
  Model* m = new Model();
  m->cfg = {cfg[0], cfg[1], cfg[2], cfg[3], cfg[4], cfg[5], cfg[6], cfg[7]};
  build_slots(*m);
  m->storage.resize(m->slots.size());
  return m;
}
void orc_model_destroy(void* p) { delete (Model*)p; }
int orc_model_num_tensors(void* p) { return (int)((Model*)p)->slots.size(); }
void orc_model_tensor_shape(void* p, int i, int* rows, int* cols) {
  Model* m = (Model*)p;
  *rows = m->slots[i].rows;
  *cols = m->slots[i].cols;
}
// copy=0 keeps the caller's pointer (must outlive the model)
void orc_model_set_tensor(void* p, int i, const float* data, int copy) {
  Model* m = (Model*)p;
  const size_t n = (size_t)m->slots[i].rows * m->slots[i].cols;
  if (copy) {
    m->storage[i].assign(data, data + n);
    *m->slots[i].dst = m->storage[i].data();
  } else {
    *m->slots[i].dst = data;
  }
}

double orc_score_batch(void* p, const int* src_ids, int S_max, const int* tgt_in, const int* tgt_out, int T, int B,
                       double* logp_out, float* hs_top_out) {
  return score_batch(*(Model*)p, src_ids, S_max, tgt_in, tgt_out, T, B, logp_out, hs_top_out);
}

// src_ids: concatenated reversed source ids; src_len[n_sent]; longest_sent is the user-level
// -L value (the reference adds 4 internally, src/main.cu:408).
// out_ids[n_sent*k_best*Lmax] (-1 padded), out_len[n_sent*k_best] (0 = no hypothesis), out_score.
// out_align (optional, same shape as out_ids): the viterbi alignment stored with every position of the hypothesis.
void orc_beam_decode_align(void* p, const int* src_ids, const int* src_len, int n_sent, int beam, int k_best,
                           float min_ratio, float max_ratio, float penalty, int longest_sent, int Lmax_out, int* out_ids,
                           int* out_len, float* out_score, int* out_align) {
  const Model& m = *(Model*)p;
  size_t pos = 0;
  for (int s = 0; s < n_sent; ++s) {
    std::vector<Hyp> res;
    beam_decode_one({&m}, {src_ids + pos}, {src_len[s]}, beam, k_best, min_ratio, max_ratio, penalty, longest_sent + 4, res);
    pos += src_len[s];
    for (int k = 0; k < k_best; ++k) {
      int* dst = out_ids + ((size_t)s * k_best + k) * Lmax_out;
      int* adst = out_align ? out_align + ((size_t)s * k_best + k) * Lmax_out : nullptr;
      for (int i = 0; i < Lmax_out; ++i) dst[i] = -1;
      if (adst) for (int i = 0; i < Lmax_out; ++i) adst[i] = -1;
      if (k < (int)res.size()) {
        const int n = std::min((int)res[k].ids.size(), Lmax_out);
        for (int i = 0; i < n; ++i) dst[i] = res[k].ids[i];
        if (adst) for (int i = 0; i < n; ++i) adst[i] = res[k].align[i];
        out_len[(size_t)s * k_best + k] = (int)res[k].ids.size();
        out_score[(size_t)s * k_best + k] = res[k].score;
      } else {
        out_len[(size_t)s * k_best + k] = 0;
        out_score[(size_t)s * k_best + k] = 0;
      }
    }
  }
}

// Test aid: the decision margin of each sentence's search (see beam_decode_one), 1-best only.
void orc_beam_decode_margins(void* p, const int* src_ids, const int* src_len, int n_sent, int beam, float min_ratio,
                             float max_ratio, float penalty, int longest_sent, float* out_margin) {
  const Model& m = *(Model*)p;
  size_t pos = 0;
  for (int s = 0; s < n_sent; ++s) {
    std::vector<Hyp> res;
    beam_decode_one({&m}, {src_ids + pos}, {src_len[s]}, beam, 1, min_ratio, max_ratio, penalty, longest_sent + 4, res,
                    out_margin + s);
    pos += src_len[s];
  }
}

void orc_beam_decode(void* p, const int* src_ids, const int* src_len, int n_sent, int beam, int k_best, float min_ratio,
                     float max_ratio, float penalty, int longest_sent, int Lmax_out, int* out_ids, int* out_len,
                     float* out_score) {
  orc_beam_decode_align(p, src_ids, src_len, n_sent, beam, k_best, min_ratio, max_ratio, penalty, longest_sent, Lmax_out,
                        out_ids, out_len, out_score, nullptr);
}

// Ensemble decoding: n_models models, model k reads src_ids[k] / src_len[k] (concatenated reversed ids per sentence).
void orc_beam_decode_ensemble(void* const* models, int n_models, const int* const* src_ids, const int* const* src_len,
                              int n_sent, int beam, int k_best, float min_ratio, float max_ratio, float penalty,
                              int longest_sent, int Lmax_out, int* out_ids, int* out_len, float* out_score,
                              int* out_align) {
  std::vector<size_t> pos(n_models, 0);
  for (int s = 0; s < n_sent; ++s) {
    std::vector<const Model*> ms;
    std::vector<const int*> srcs;
    std::vector<int> Ss;
    for (int k = 0; k < n_models; ++k) {
      ms.push_back((const Model*)models[k]);
      srcs.push_back(src_ids[k] + pos[k]);
      Ss.push_back(src_len[k][s]);
      pos[k] += src_len[k][s];
    }
    std::vector<Hyp> res;
    beam_decode_one(ms, srcs, Ss, beam, k_best, min_ratio, max_ratio, penalty, longest_sent + 4, res);
    for (int k = 0; k < k_best; ++k) {
      int* dst = out_ids + ((size_t)s * k_best + k) * Lmax_out;
      int* adst = out_align ? out_align + ((size_t)s * k_best + k) * Lmax_out : nullptr;
      for (int i = 0; i < Lmax_out; ++i) dst[i] = -1;
      if (adst) for (int i = 0; i < Lmax_out; ++i) adst[i] = -1;
      out_len[(size_t)s * k_best + k] = 0;
      out_score[(size_t)s * k_best + k] = 0;
      if (k < (int)res.size()) {
        const int n = std::min((int)res[k].ids.size(), Lmax_out);
        for (int i = 0; i < n; ++i) dst[i] = res[k].ids[i];
        if (adst) for (int i = 0; i < n; ++i) adst[i] = res[k].align[i];
        out_len[(size_t)s * k_best + k] = (int)res[k].ids.size();
        out_score[(size_t)s * k_best + k] = res[k].score;
      }
    }
  }
}

// ---- layer-level entry points for per-kernel parity tests
void orc_gather(const float* W, int H, const int* ids, int n, float* x) {
  std::vector<int> t(n);
  for (int i = 0; i < n; ++i) t[i] = id_nonm1(ids[i]);
  gather(W, H, t.data(), n, x);
}

// w[17] in file order: W_hi b_i W_hf b_f W_hc b_c W_ho b_o W(unused) M_i M_f M_o M_c Q_i Q_f Q_o Q_c
void orc_lstm_cell(int H, int B, const float* const* w, const float* x, const float* h_prev, const float* c_prev,
                   const float* htild, const int* mask, float* h_out, float* c_out) {
  LstmW lw;
  lw.W_hi = w[0]; lw.b_i = w[1]; lw.W_hf = w[2]; lw.b_f = w[3]; lw.W_hc = w[4]; lw.b_c = w[5]; lw.W_ho = w[6];
  lw.b_o = w[7]; lw.W = w[8]; lw.M_i = w[9]; lw.M_f = w[10]; lw.M_o = w[11]; lw.M_c = w[12];
  lw.Q_i = w[13]; lw.Q_f = w[14]; lw.Q_o = w[15]; lw.Q_c = w[16];
  std::vector<float> scratch;
  lstm_cell(H, B, lw, x, h_prev, c_prev, htild, mask, h_out, c_out, scratch);
}

// w[6]: W_a W_p v_p output_bias W_c_p1 W_c_p2
void orc_attention(int type, int H, int B, int D, const float* const* w, const float* h_t, const int* mask,
                   const float* hs_all, int S_max, const int* len, const int* offset, float* htild_out,
                   float* align_out, int* idx_out) {
  AttW aw;
  aw.W_a = w[0]; aw.W_p = w[1]; aw.v_p = w[2]; aw.output_bias = w[3]; aw.W_c_p1 = w[4]; aw.W_c_p2 = w[5];
  attention(type, H, B, D, aw, h_t, mask, hs_all, S_max, len, offset, htild_out, align_out, idx_out);
}
// the same step, also returning the viterbi alignment per column
void orc_attention_viterbi(int type, int H, int B, int D, const float* const* w, const float* h_t, const int* mask,
                           const float* hs_all, int S_max, const int* len, const int* offset, float* htild_out,
                           int* viterbi_out) {
  AttW aw;
  aw.W_a = w[0]; aw.W_p = w[1]; aw.v_p = w[2]; aw.output_bias = w[3]; aw.W_c_p1 = w[4]; aw.W_c_p2 = w[5];
  attention(type, H, B, D, aw, h_t, mask, hs_all, S_max, len, offset, htild_out, nullptr, nullptr, viterbi_out);
}

void orc_softmax_logp(int V, int H, int N, const float* D, const float* b_d, const float* h, const int* target,
                      double* logp_target, double* logp_all) {
  softmax_logp(V, H, N, D, b_d, h, target, logp_target, logp_all);
}
void orc_softmax_dist(int V, int H, int N, const float* D, const float* b_d, const float* h, float* p) {
  softmax_dist(V, H, N, D, b_d, h, p);
}

}  // extern "C"
