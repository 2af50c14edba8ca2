// C ABI (include/zrnn.h) and the C++ host side above it: layer objects mirroring the reference's
// Input_To_Hidden_Layer / Hidden_To_Hidden_Layer / attention_layer / softmax_layer, and the
// neuralMT_model drivers for teacher-forced scoring and batched beam decoding.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <set>
#include <string>
#include <vector>

#include "../../include/zrnn.h"
#include "../../include/zrnn_debug.h"
#include "kernels.cuh"
#include "model_file.hpp"
#include "tc_decoder.cuh"
#include "tc_gemm.cuh"

namespace {

thread_local std::string g_err;
int fail(int code, const std::string& msg) {
  g_err = msg;
  return code;
}
#define ZR_CUDA(expr)                                                                 \
  do {                                                                                \
    cudaError_t _e = (expr);                                                          \
    if (_e != cudaSuccess)                                                            \
      return fail(ZRNN_E_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e));   \
  } while (0)
#define ZR_CHECK(cond, msg)                    \
  do {                                         \
    if (!(cond)) return fail(ZRNN_E_ARG, msg); \
  } while (0)
#define ZR_TRY(expr)                \
  do {                              \
    int _s = (expr);                \
    if (_s != ZRNN_OK) return _s;   \
  } while (0)

// bumped whenever any scratch buffer is reallocated; captured graphs that may reference the old memory are dropped
unsigned long long g_buf_generation = 0;

// device buffer that only grows
struct DevBuf {
  void* p = nullptr;
  size_t cap = 0;
  cudaError_t reserve(size_t bytes) {
    if (bytes <= cap) return cudaSuccess;
    ++g_buf_generation;
    if (p) cudaFree(p);
    p = nullptr;
    cap = 0;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaSuccess) cap = bytes;
    return e;
  }
  void release() {
    if (p) cudaFree(p);
    p = nullptr;
    cap = 0;
  }
  template <class T> T* as() const { return reinterpret_cast<T*>(p); }
};

// carve 256-byte aligned pieces out of one DevBuf
struct Carver {
  char* base;
  size_t off = 0;
  explicit Carver(void* b) : base((char*)b) {}
  template <class T> T* take(size_t n) {
    T* r = reinterpret_cast<T*>(base + off);
    off += (n * sizeof(T) + 255) / 256 * 256;
    return r;
  }
};
size_t aligned(size_t bytes) { return (bytes + 255) / 256 * 256; }
// near-equal contiguous ranges of n items over `world` ranks: [n*r/world, n*(r+1)/world)
void shard_range(long long n, int world, int r, int* lo, int* hi) {
  *lo = (int)(n * r / world);
  *hi = (int)(n * (r + 1) / world);
}

cudaError_t upload(float** dst, const float* src, size_t n) {
  cudaError_t e = cudaMalloc((void**)dst, n * sizeof(float));
  if (e != cudaSuccess) return e;
  return cudaMemcpy(*dst, src, n * sizeof(float), cudaMemcpyHostToDevice);
}

// Optional CUDA-event timing of kernel classes (used by the benchmark's roofline report).
enum { KC_GATHER = 0, KC_LSTM = 1, KC_ATT = 2, KC_SOFTMAX_GEMM = 3, KC_SOFTMAX_REDUCE = 4, KC_BEAM = 5, KC_REORDER = 6, KC_COUNT = 7 };
struct KTiming {
  bool on = false;
  std::vector<cudaEvent_t> ev;  // pairs
  std::vector<int> cls;
  std::vector<int> cnt;  // launches covered by the pair
  size_t used = 0;       // pairs in use
  int group_cls = -1;    // a group scope of this class is open: its inner scopes do not record
  // launches of the persistent decoder kernel: it stamps %globaltimer at every phase boundary into a buffer of its
  // own, from which the per-class times are taken when the report is read
  struct DecRun { long long* d_stamps; int T, P, L; };
  std::vector<DecRun> dec_runs;
  void drop_dec_runs() {
    for (auto& r : dec_runs) cudaFree(r.d_stamps);
    dec_runs.clear();
  }
};
thread_local KTiming g_kt;
const size_t KT_CAP = 16384;
// One event pair around a launch, or (group = true) around `launches` back-to-back launches of one class, so that
// the per-launch average includes the overlap between consecutive launches and not one event pair's cost each.
struct KScope {
  long idx = -1;
  cudaStream_t s;
  bool group;
  KScope(int c, cudaStream_t st, int launches = 1, bool grp = false) : s(st), group(grp) {
    if (!g_kt.on || g_kt.used >= KT_CAP) return;
    if (!grp && g_kt.group_cls == c) return;
    if (g_kt.ev.size() < 2 * (g_kt.used + 1)) {
      cudaEvent_t a, b;
      if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
      g_kt.ev.push_back(a);
      g_kt.ev.push_back(b);
      g_kt.cls.push_back(c);
      g_kt.cnt.push_back(1);
    }
    idx = (long)g_kt.used++;
    g_kt.cls[idx] = c;
    g_kt.cnt[idx] = launches;
    if (grp) g_kt.group_cls = c;
    cudaEventRecord(g_kt.ev[2 * idx], s);
  }
  ~KScope() {
    if (idx < 0) return;
    cudaEventRecord(g_kt.ev[2 * idx + 1], s);
    if (group) g_kt.group_cls = -1;
  }
};

int check_device() {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return fail(ZRNN_E_CUDA, std::string("no CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "count 0"));
  return ZRNN_OK;
}

}  // namespace

// ------------------------------------------------------------------------------------------
// arithmetic engines
// ------------------------------------------------------------------------------------------
// ENG_SIMT : exact fp32 FMA kernels (kernels.cu)            - any shape
// ENG_X3   : tcgen05 3xTF32 (operands split into hi + lo)   - fp32-level accuracy, H % 4 == 0
// ENG_BF16 : tcgen05 on bf16-rounded weights / activations  - H % 8 == 0
// ENG_TF32 : tcgen05 single-pass tf32                       - H % 4 == 0
// ENG_H2   : tcgen05 fp16 split (hi + scaled lo, both fp16)  - fp32-level accuracy for operands inside the fp16
//            range (|x| < 65504; LSTM activations are bounded by 1, weights are checked at load), H % 4 == 0;
//            half the bytes and half the tensor time of ENG_X3
enum { ENG_SIMT = 0, ENG_BF16 = 1, ENG_TF32 = 2, ENG_X3 = 3, ENG_H2 = 4 };

namespace {

int eng_eb(int e) { return (e == ENG_BF16 || e == ENG_H2) ? 2 : 4; }
int eng_opmode(int e) { return e == ENG_BF16 ? 0 : (e == ENG_TF32 ? 1 : (e == ENG_H2 ? 3 : 2)); }
int eng_tcmode(int e) {
  return e == ENG_BF16 ? zrnn::TC_BF16 : (e == ENG_TF32 ? zrnn::TC_TF32 : (e == ENG_H2 ? zrnn::TC_F16X2 : zrnn::TC_TF32X3));
}
bool eng_split(int e) { return e == ENG_X3 || e == ENG_H2; }  // operands carry a lo part (same element size as hi)
int round64(int x) { return (x + 63) / 64 * 64; }

int pick_engine(int dtype, int H, int* eng) {
  switch (dtype) {
    case ZRNN_F32: {
      const char* e = std::getenv("ZRNN_FP32_ENGINE");
      const bool want_simt = e && std::strcmp(e, "simt") == 0;
      const bool want_x3 = e && std::strcmp(e, "x3") == 0;
      // the tensor-core path also wins on small layers (H = 100: 0.31 against 0.72 ms per config-1 step)
      *eng = (!want_simt && H % 4 == 0 && H >= 64) ? (want_x3 ? ENG_X3 : ENG_H2) : ENG_SIMT;
      return ZRNN_OK;
    }
    case ZRNN_F32_F16X2:
      ZR_CHECK(H % 4 == 0, "fp16-split arithmetic needs H to be a multiple of 4");
      *eng = ENG_H2;
      return ZRNN_OK;
    case ZRNN_F32_SIMT: *eng = ENG_SIMT; return ZRNN_OK;
    case ZRNN_F32_3XTF32:
      ZR_CHECK(H % 4 == 0, "3xTF32 arithmetic needs H to be a multiple of 4");
      *eng = ENG_X3;
      return ZRNN_OK;
    case ZRNN_BF16:
      ZR_CHECK(H % 8 == 0, "bf16 arithmetic needs H to be a multiple of 8");
      *eng = ENG_BF16;
      return ZRNN_OK;
    case ZRNN_TF32:
      ZR_CHECK(H % 4 == 0, "tf32 arithmetic needs H to be a multiple of 4");
      *eng = ENG_TF32;
      return ZRNN_OK;
  }
  return fail(ZRNN_E_ARG, "unknown dtype");
}

// ENG_H2 stores operands as fp16 pairs: every weight must be finite and inside the fp16 range
int check_f16_range(int eng, const float* p, size_t n, const char* what) {
  if (eng != ENG_H2) return ZRNN_OK;
  for (size_t i = 0; i < n; ++i)
    if (!(std::fabs(p[i]) < 60000.0f))
      return fail(ZRNN_E_ARG, std::string(what) + ": a weight is not finite or exceeds the fp16 range; use dtype "
                                  "ZRNN_F32_3XTF32 (or ZRNN_FP32_ENGINE=x3) for this model");
  return ZRNN_OK;
}

// weights / tables in tensor-core operand form (K-major rows)
struct OpMem {
  void* hi = nullptr;
  float* lo = nullptr;
  int alloc(size_t elems, int eng) {
    release();
    ++g_buf_generation;  // a captured graph may still hold the old addresses
    ZR_CUDA(cudaMalloc(&hi, elems * eng_eb(eng)));
    ZR_CUDA(cudaMemset(hi, 0, elems * eng_eb(eng)));
    if (eng_split(eng)) {
      ZR_CUDA(cudaMalloc((void**)&lo, elems * eng_eb(eng)));
      ZR_CUDA(cudaMemset(lo, 0, elems * eng_eb(eng)));
    }
    return ZRNN_OK;
  }
  void release() {
    if (hi || lo) ++g_buf_generation;
    cudaFree(hi);
    cudaFree(lo);
    hi = nullptr;
    lo = nullptr;
  }
};

// An activation matrix: column-major fp32 (H x cols) and/or its operand-form copy (cols rows of Kpad elements)
struct Act {
  float* f32 = nullptr;
  void* hi = nullptr;
  float* lo = nullptr;
};
struct Geom {
  int H, Kpad, eng;
};
Act act_at(const Act& a, size_t col, const Geom& g) {
  Act r;
  r.f32 = a.f32 ? a.f32 + col * g.H : nullptr;
  r.hi = a.hi ? (char*)a.hi + col * g.Kpad * eng_eb(g.eng) : nullptr;
  r.lo = a.lo ? (float*)((char*)a.lo + col * g.Kpad * eng_eb(g.eng)) : nullptr;  // lo elements have hi's size
  return r;
}

}  // namespace

// ------------------------------------------------------------------------------------------
// layer objects
// ------------------------------------------------------------------------------------------
struct zrnn_lstm_layer {
  int H = 0, V = 0, feed = 0, dtype = 0, is_ih = 0, eng = ENG_SIMT;
  bool loaded = false;
  float* W = nullptr;   // embedding H x V
  float* Wh = nullptr;  // 4 x (H x H): gates i,f,g,o
  float* Mx = nullptr;  // 4 x (H x H)
  float* Q = nullptr;   // 4 x (H x H), feed-input only
  float* b = nullptr;   // 4 x H
  DevBuf x;             // gather scratch for zrnn_ih_forward
  // tensor-core form: packed [n_tiles*BN rows] x [nsrc*Kpad] with the K axis = (x | h | htild)
  int Kpad = 0, BN = 128, n_tiles = 0;
  int kbtot = 0;  // > 0: weights stored tile-contiguously with this many k-blocks per row tile
  OpMem Wcat, emb;
  CUtensorMap wmap, wmap_lo;
  DevBuf sc_x, sc_h, sc_q, sc_xl, sc_hl, sc_ql;  // operand scratch for the fp32 layer-level entry points
  ~zrnn_lstm_layer() {
    cudaFree(W); cudaFree(Wh); cudaFree(Mx); cudaFree(Q); cudaFree(b);
    x.release(); Wcat.release(); emb.release();
    sc_x.release(); sc_h.release(); sc_q.release(); sc_xl.release(); sc_hl.release(); sc_ql.release();
  }
};

struct zrnn_attention {
  int H = 0, D = 0, type = 0, dtype = 0, eng = ENG_SIMT;
  bool loaded = false;
  float* WpWaT = nullptr;  // stacked [W_p ; W_a^T], 2H x H column-major (local-p only)
  float* v_p = nullptr;
  float* bias = nullptr;
  float* Wc1 = nullptr;
  float* Wc2 = nullptr;
  const float* hs = nullptr;
  int S_max = 0, B_src = 0, cols_per_sent = 1;
  const int* len = nullptr;
  const int* off = nullptr;
  DevBuf tq, ctx;
  int Kpad = 0, BN = 128;
  OpMem WpWaT_op, Wc_op;  // [2H rows x Kpad], [H rows x 2*Kpad]
  CUtensorMap pmap, pmap_lo, cmap, cmap_lo;
  DevBuf ctx_hi, ctx_lo, sc_h, sc_hl;
  ~zrnn_attention() {
    cudaFree(WpWaT); cudaFree(v_p); cudaFree(bias); cudaFree(Wc1); cudaFree(Wc2);
    tq.release(); ctx.release(); WpWaT_op.release(); Wc_op.release();
    ctx_hi.release(); ctx_lo.release(); sc_h.release(); sc_hl.release();
  }
};

struct zrnn_softmax {
  int V = 0, H = 0, dtype = 0, lo = 0, hi = 0, eng = ENG_SIMT;
  bool loaded = false;
  float* D = nullptr;  // (hi-lo) x H
  float* b = nullptr;  // hi-lo
  DevBuf parts, tgt, logits;
  int Kpad = 0, BN = 128, n_tiles = 0;
  int kbtot = 0;  // > 0: weights stored tile-contiguously with this many k-blocks per row tile
  OpMem D_op;  // [n_tiles*BN rows x Kpad]
  CUtensorMap dmap, dmap_lo;
  DevBuf sc_h, sc_hl;
  ~zrnn_softmax() {
    cudaFree(D); cudaFree(b);
    parts.release(); tgt.release(); logits.release(); D_op.release(); sc_h.release(); sc_hl.release();
  }
};

namespace {

// Split the K axis over a cluster when that shortens the launch: with one CTA per SM a launch runs in
// ceil(CTAs / SMs) waves, a split by s multiplies the CTAs by s and divides the work of each by s at the price of the
// exchange.  Picks the s that minimises waves * (1/s + exchange), e.g. 32 CTAs -> 4 (one wave of quarter-size CTAs),
// 16 CTAs -> 4, 64 CTAs -> 2, 192 CTAs (768 decode columns) -> 1 (splitting them was measured slightly slower).
int pick_splitk(int m_cols, int n_rows, int BN, int max_split) {
  if (BN != 128) return 1;
  const int ctas = ((m_cols + 127) / 128) * ((n_rows + BN - 1) / BN);
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  int best = 1;
  double best_t = 1e30;
  for (int s = 1; s <= max_split && s <= 8; s *= 2) {
    // 8-CTA clusters of one CTA per SM: no more than 8 of them are resident at once on this part (measured: 16 such
    // clusters ran as two waves)
    if (s == 8 && ctas > 8) break;
    const int waves = (ctas * s + sms - 1) / sms;
    const double t = waves * (1.0 / s + (s > 1 ? 0.2 : 0.0));  // exchange ~ 20 % of an unsplit CTA's time (measured)
    if (t < best_t - 1e-9) { best_t = t; best = s; }
  }
  return best;
}

long long* g_dec_detail = nullptr;  // developer timeline of the persistent decoder kernel (zrnn_debug_decoder_timeline)
int g_dec_detail_cta = 0;
long long* g_tc_prof = nullptr;  // developer profiling buffer (see zrnn_debug_tc_profile)
int g_tc_prof_slot = -1;          // >= 0: timeline mode, one slot per tensor-core launch
int g_tc_prof_cap = 0;
void prof_attach(zrnn::TcParams& tp) {
  tp.prof = g_tc_prof;
  tp.prof_slot = -1;
  if (g_tc_prof && g_tc_prof_slot >= 0) {
    if (g_tc_prof_slot < g_tc_prof_cap) tp.prof_slot = g_tc_prof_slot++;
    else tp.prof = nullptr;
  }
}

int* tc_error_word() {  // one word per device
  static int* p[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (!p[dev]) {
    if (cudaMalloc((void**)&p[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p[dev], 0, sizeof(int));
  }
  return p[dev];
}

// tensor maps of an activation operand: `rows` rows of H valid elements, stride Kpad
int act_maps(const Act& a, int eng, int H, int Kpad, int rows, CUtensorMap* hi, CUtensorMap* lo, int box_rows = 128) {
  if (!a.hi) return fail(ZRNN_E_STATE, "internal: activation has no operand-form copy");
  if (!zrnn::make_kmajor_map(hi, a.hi, eng_eb(eng), H, rows, Kpad, box_rows))
    return fail(ZRNN_E_CUDA, "cannot encode a TMA tensor map for an activation operand");
  if (eng_split(eng) && !zrnn::make_kmajor_map(lo, a.lo, eng_eb(eng), H, rows, Kpad, box_rows))
    return fail(ZRNN_E_CUDA, "cannot encode a TMA tensor map for an activation operand (lo)");
  return ZRNN_OK;
}

// fp32 activation (H x cols, column-major) -> operand form in scratch buffers
int to_operand(const float* f32, int H, int Kpad, int cols, int eng, DevBuf& hi, DevBuf& lo, Act* out, cudaStream_t st) {
  ZR_CUDA(hi.reserve((size_t)cols * Kpad * eng_eb(eng)));
  if (eng_split(eng)) ZR_CUDA(lo.reserve((size_t)cols * Kpad * eng_eb(eng)));
  ZR_CUDA(zrnn::launch_convert_rows(f32, cols, H, H, eng_opmode(eng), hi.p, lo.as<float>(), Kpad, st));
  out->f32 = const_cast<float*>(f32);
  out->hi = hi.p;
  out->lo = eng_split(eng) ? lo.as<float>() : nullptr;
  return ZRNN_OK;
}

int lstm_cell_simt(zrnn_lstm_layer* L, const float* x, const int* mask, const float* h_prev, const float* c_prev,
                   const float* htild, int B, float* h_out, float* c_out, cudaStream_t st) {
  const int H = L->H;
  const size_t HH = (size_t)H * H;
  zrnn::GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  int n = 0;
  auto add = [&](const float* A, const float* Bm) {
    for (int k = 0; k < 4; ++k) g.src[n].A[k] = A + k * HH;
    g.src[n].lda = H; g.src[n].B = Bm; g.src[n].ldb = H; g.src[n].K = H;
    ++n;
  };
  add(L->Mx, x);
  add(L->Wh, h_prev);
  if (htild) add(L->Q, htild);
  g.nsrc = n;
  g.M = H; g.N = B;
  for (int k = 0; k < 4; ++k) g.bias[k] = L->b + (size_t)k * H;
  g.mask = mask;
  g.c_prev = c_prev; g.h_out = h_out; g.c_out = c_out;
  KScope ks(KC_LSTM, st);
  ZR_CUDA(zrnn::launch_fused_gemm(g, 4, zrnn::EPI_LSTM, 0, st));
  return ZRNN_OK;
}

// where the epilogue leaves the operand-form copy of its output for the next GEMM
void set_operand_outputs(zrnn::TcParams& tp, int eng, const Act& out, int Kpad) {
  tp.ld_op = Kpad;
  if (eng == ENG_BF16) {
    tp.op_b16 = (__nv_bfloat16*)out.hi;
  } else if (eng == ENG_H2) {
    tp.op_h_hi = (__half*)out.hi;
    tp.op_h_lo = (__half*)out.lo;
  } else {
    tp.op_hi = (float*)out.hi;
    tp.op_lo = eng == ENG_X3 ? out.lo : nullptr;
  }
}

// One LSTM cell.  x / h_prev / htild and the output are activations in the form the layer's engine needs.
// kernel parameters of one tensor-core LSTM layer-step
int cell_params(zrnn_lstm_layer* L, const Act& x, const Act& hp, const Act* q, const int* mask, const float* c_prev,
                int B, const Act& out, float* c_out, zrnn::TcParams& tp) {
  const int H = L->H, Kpad = L->Kpad, eng = L->eng;
  const int kb = (H + 128 / eng_eb(eng) - 1) / (128 / eng_eb(eng));
  std::memset(&tp, 0, sizeof(tp));
  ZR_TRY(act_maps(x, eng, H, Kpad, B, &tp.a[0], &tp.a_lo[0]));
  ZR_TRY(act_maps(hp, eng, H, Kpad, B, &tp.a[1], &tp.a_lo[1]));
  tp.nsrc = 2;
  if (q) {
    ZR_TRY(act_maps(*q, eng, H, Kpad, B, &tp.a[2], &tp.a_lo[2]));
    tp.nsrc = 3;
  }
  for (int s = 0; s < 3; ++s) { tp.kblocks[s] = kb; tp.b_koff[s] = s * Kpad; }
  tp.b = L->wmap; tp.b_lo = L->wmap_lo; tp.b_tiled_kbtot = L->kbtot;
  tp.M = B; tp.N = H; tp.bias = L->b; tp.mask = mask;
  tp.C = out.f32; tp.ldc = H;
  set_operand_outputs(tp, eng, out, Kpad);
  tp.c_prev = c_prev; tp.c_out = c_out; tp.err = tc_error_word(); prof_attach(tp);
  return ZRNN_OK;
}
int cell_forward(zrnn_lstm_layer* L, const Act& x, const Act& hp, const Act* q, const int* mask, const float* c_prev,
                 int B, const Act& out, float* c_out, cudaStream_t st) {
  if (L->eng == ENG_SIMT)
    return lstm_cell_simt(L, x.f32, mask, hp.f32, c_prev, q ? q->f32 : nullptr, B, out.f32, c_out, st);
  const int H = L->H, eng = L->eng;
  zrnn::TcParams tp;
  ZR_TRY(cell_params(L, x, hp, q, mask, c_prev, B, out, c_out, tp));
  KScope ks(KC_LSTM, st);
  int bn = L->BN;
  const int splitk = pick_splitk(B, 4 * H, L->BN, 4);
  // many columns (beam decoding): 128-row tiles would need more than one wave of CTAs; 256-row tiles built from two
  // packed tiles halve the CTA count and the activation traffic per flop.  A 256-column tile leaves TMEM room for one
  // main accumulator only (measured per-token log-prob error at H = 1000: fp16 split 0.8e-6 -> 2.1e-6, 3xTF32
  // 1.6e-6 -> 3.9e-6), so the 3xTF32 engine, chosen for its accuracy margin, keeps the 128-row tiles.
  if (splitk == 1 && L->BN == 128 && eng != ENG_X3 && ((B + 127) / 128) * L->n_tiles > 148) {
    bn = 256;
    tp.b_pack_rows = 128;
  }
  ZR_CUDA(zrnn::launch_tc_gemm(tp, bn, eng_tcmode(eng), zrnn::TC_EPI_LSTM, st, splitk));
  return ZRNN_OK;
}

int att_forward(zrnn_attention* A, const Act& h_t, const int* mask, int B, const Act& out, float* align,
                cudaStream_t st, int* viterbi = nullptr, float viterbi_init = -1.f, bool align_by_pos = false) {
  const int H = A->H, eng = A->eng, Kpad = A->Kpad;
  ZR_CUDA(A->ctx.reserve(sizeof(float) * (size_t)H * B));
  KScope ks(KC_ATT, st);
  zrnn::AttArgs a;
  std::memset(&a, 0, sizeof(a));
  a.H = H; a.B = B; a.D = A->D; a.S_max = A->S_max; a.B_src = A->B_src; a.cols_per_sent = A->cols_per_sent;
  a.hs = A->hs; a.len = A->len; a.offset = A->off; a.mask = mask; a.h_t = h_t.f32;
  a.c_t = A->ctx.as<float>(); a.align_out = align; a.viterbi_out = viterbi; a.viterbi_init = viterbi_init;
  a.align_by_pos = align_by_pos ? 1 : 0;
  Act ctx;
  ctx.f32 = A->ctx.as<float>();
  if (eng != ENG_SIMT) {
    ZR_CUDA(A->ctx_hi.reserve((size_t)B * Kpad * eng_eb(eng)));
    if (eng_split(eng)) ZR_CUDA(A->ctx_lo.reserve((size_t)B * Kpad * eng_eb(eng)));
    ctx.hi = A->ctx_hi.p;
    ctx.lo = eng_split(eng) ? A->ctx_lo.as<float>() : nullptr;
    a.ld_op = Kpad;
    if (eng == ENG_BF16) a.op_b16 = ctx.hi;
    else if (eng == ENG_H2) { a.op_h_hi = ctx.hi; a.op_h_lo = ctx.lo; }
    else { a.op_hi = (float*)ctx.hi; a.op_lo = ctx.lo; }
  }
  if (A->type == ZRNN_ATT_LOCAL_P) {
    ZR_CUDA(A->tq.reserve(sizeof(float) * (size_t)2 * H * B));
    if (eng == ENG_SIMT) {
      zrnn::GemmArgs g;
      std::memset(&g, 0, sizeof(g));
      g.nsrc = 1;
      g.src[0].A[0] = A->WpWaT; g.src[0].lda = 2 * H; g.src[0].B = h_t.f32; g.src[0].ldb = H; g.src[0].K = H;
      g.M = 2 * H; g.N = B; g.C = A->tq.as<float>(); g.ldc = 2 * H; g.act = 1; g.act_rows = H;
      ZR_CUDA(zrnn::launch_fused_gemm(g, 1, zrnn::EPI_STORE, 0, st));
    } else {
      zrnn::TcParams tp;
      std::memset(&tp, 0, sizeof(tp));
      ZR_TRY(act_maps(h_t, eng, H, Kpad, B, &tp.a[0], &tp.a_lo[0]));
      tp.nsrc = 1; tp.kblocks[0] = (H + 128 / eng_eb(eng) - 1) / (128 / eng_eb(eng)); tp.b_koff[0] = 0;
      tp.b = A->pmap; tp.b_lo = A->pmap_lo;
      tp.M = B; tp.N = 2 * H; tp.C = A->tq.as<float>(); tp.ldc = 2 * H; tp.act = 1; tp.act_rows = H;
      tp.err = tc_error_word();
      if (g_tc_prof_slot >= 0) prof_attach(tp);
      ZR_CUDA(zrnn::launch_tc_gemm(tp, A->BN, eng_tcmode(eng), zrnn::TC_EPI_STORE, st, pick_splitk(B, 2 * H, A->BN, 8)));
    }
    a.tanh1 = A->tq.as<float>(); a.q = A->tq.as<float>() + H; a.ld_tq = 2 * H; a.v_p = A->v_p;
    ZR_CUDA(zrnn::launch_att_local(a, st));
  } else {
    ZR_CUDA(zrnn::launch_att_global(a, st));
  }
  if (eng == ENG_SIMT) {
    zrnn::GemmArgs g;
    std::memset(&g, 0, sizeof(g));
    g.nsrc = 2;
    g.src[0].A[0] = A->Wc1; g.src[0].lda = H; g.src[0].B = ctx.f32; g.src[0].ldb = H; g.src[0].K = H;
    g.src[1].A[0] = A->Wc2; g.src[1].lda = H; g.src[1].B = h_t.f32; g.src[1].ldb = H; g.src[1].K = H;
    g.M = H; g.N = B; g.C = out.f32; g.ldc = H; g.bias[0] = A->bias; g.mask = mask; g.act = 1;
    ZR_CUDA(zrnn::launch_fused_gemm(g, 1, zrnn::EPI_STORE, 0, st));
  } else {
    zrnn::TcParams tp;
    std::memset(&tp, 0, sizeof(tp));
    const int kb = (H + 128 / eng_eb(eng) - 1) / (128 / eng_eb(eng));
    ZR_TRY(act_maps(ctx, eng, H, Kpad, B, &tp.a[0], &tp.a_lo[0]));
    ZR_TRY(act_maps(h_t, eng, H, Kpad, B, &tp.a[1], &tp.a_lo[1]));
    tp.nsrc = 2; tp.kblocks[0] = tp.kblocks[1] = kb; tp.b_koff[0] = 0; tp.b_koff[1] = Kpad;
    tp.b = A->cmap; tp.b_lo = A->cmap_lo;
    tp.M = B; tp.N = H; tp.bias = A->bias; tp.mask = mask; tp.act = 1;
    tp.C = out.f32; tp.ldc = H;
    set_operand_outputs(tp, eng, out, Kpad);
    tp.err = tc_error_word();
    if (g_tc_prof_slot >= 0) prof_attach(tp);
    ZR_CUDA(zrnn::launch_tc_gemm(tp, A->BN, eng_tcmode(eng), zrnn::TC_EPI_STORE, st, pick_splitk(B, H, A->BN, 8)));
  }
  return ZRNN_OK;
}

// per-column (max, sum exp) partials over this layer's rows + target logit into S->parts / tgt
int softmax_partials_launch(zrnn_softmax* S, const Act& h, const int* targets, int N, int* n_parts, float** pm,
                            float** ps, float* tgt, cudaStream_t st) {
  const int Vs = S->hi - S->lo, H = S->H;
  ZR_CUDA(cudaMemsetAsync(tgt, 0, sizeof(float) * (size_t)N, st));
  if (S->eng == ENG_SIMT) {
    const int tile = (N >= 96 && Vs >= 512) ? 1 : 0;
    const int rows = zrnn::gemm_rows_per_tile(1, tile);
    const int np = (Vs + rows - 1) / rows;
    ZR_CUDA(S->parts.reserve(sizeof(float) * 2 * (size_t)np * N));
    zrnn::GemmArgs g;
    std::memset(&g, 0, sizeof(g));
    g.nsrc = 1;
    g.src[0].A[0] = S->D; g.src[0].lda = Vs; g.src[0].B = h.f32; g.src[0].ldb = H; g.src[0].K = H;
    g.M = Vs; g.N = N; g.bias[0] = S->b;
    g.target = targets; g.target_offset = S->lo;
    g.part_max = S->parts.as<float>(); g.part_sum = S->parts.as<float>() + (size_t)np * N;
    g.tgt_logit = tgt;
    *n_parts = np; *pm = g.part_max; *ps = g.part_sum;
    KScope ks(KC_SOFTMAX_GEMM, st);
    ZR_CUDA(zrnn::launch_fused_gemm(g, 1, zrnn::EPI_LSE, tile, st));
    return ZRNN_OK;
  }
  const int eng = S->eng, np = S->n_tiles * zrnn::kPersistentParts;
  ZR_CUDA(S->parts.reserve(sizeof(float) * 2 * (size_t)np * N));
  zrnn::TcParams tp;
  std::memset(&tp, 0, sizeof(tp));
  ZR_TRY(act_maps(h, eng, H, S->Kpad, N, &tp.a[0], &tp.a_lo[0]));
  tp.nsrc = 1; tp.kblocks[0] = (H + 128 / eng_eb(eng) - 1) / (128 / eng_eb(eng)); tp.b_koff[0] = 0;
  tp.b = S->dmap; tp.b_lo = S->dmap_lo;
  tp.M = N; tp.N = Vs; tp.bias = S->b;
  tp.target = targets; tp.target_offset = S->lo;
  tp.part_max = S->parts.as<float>(); tp.part_sum = S->parts.as<float>() + (size_t)np * N; tp.tgt_logit = tgt;
  tp.err = tc_error_word();
  if (g_tc_prof_slot >= 0) prof_attach(tp);
  *n_parts = np; *pm = tp.part_max; *ps = tp.part_sum;
  KScope ks(KC_SOFTMAX_GEMM, st);
  ZR_CUDA(zrnn::launch_tc_gemm_persistent(tp, eng_tcmode(eng), zrnn::TC_EPI_LSE, st));
  return ZRNN_OK;
}

int softmax_score_act(zrnn_softmax* S, const Act& h, const int* targets, const int* mask, int N, float* logp,
                      cudaStream_t st) {
  ZR_CUDA(S->tgt.reserve(sizeof(float) * (size_t)N));
  int np = 0;
  float *pm, *ps;
  ZR_TRY(softmax_partials_launch(S, h, targets, N, &np, &pm, &ps, S->tgt.as<float>(), st));
  KScope ks(KC_SOFTMAX_REDUCE, st);
  ZR_CUDA(zrnn::launch_lse_combine(pm, ps, S->tgt.as<float>(), np, N, mask, logp, st));
  return ZRNN_OK;
}

// logits = D h + b_d into S->logits (V x N); tensor-core engines also leave each tile's maximum (*pm, *np tiles) and,
// when ps_out is given, each tile's sum of exp(x - maximum)
int softmax_logits_act(zrnn_softmax* S, const Act& h, int N, cudaStream_t st, const float** pm_out, int* np_out,
                       const float** ps_out = nullptr) {
  const int Vs = S->hi - S->lo;  // rows this layer holds (the whole vocabulary unless it is a shard)
  ZR_CUDA(S->logits.reserve(sizeof(float) * (size_t)Vs * N));
  const float *pm = nullptr;
  int np = 0;
  if (S->eng == ENG_SIMT) {
    zrnn::GemmArgs g;
    std::memset(&g, 0, sizeof(g));
    g.nsrc = 1;
    g.src[0].A[0] = S->D; g.src[0].lda = Vs; g.src[0].B = h.f32; g.src[0].ldb = S->H; g.src[0].K = S->H;
    g.M = Vs; g.N = N; g.C = S->logits.as<float>(); g.ldc = Vs; g.bias[0] = S->b;
    KScope ks(KC_SOFTMAX_GEMM, st);
    ZR_CUDA(zrnn::launch_fused_gemm(g, 1, zrnn::EPI_STORE, (N >= 96 && Vs >= 512) ? 1 : 0, st));
  } else {
    const int eng = S->eng;
    np = S->n_tiles * zrnn::kPersistentParts;
    ZR_CUDA(S->parts.reserve(sizeof(float) * 2 * (size_t)np * N));
    zrnn::TcParams tp;
    std::memset(&tp, 0, sizeof(tp));
    ZR_TRY(act_maps(h, eng, S->H, S->Kpad, N, &tp.a[0], &tp.a_lo[0]));
    tp.nsrc = 1; tp.kblocks[0] = (S->H + 128 / eng_eb(eng) - 1) / (128 / eng_eb(eng)); tp.b_koff[0] = 0;
    tp.b = S->dmap; tp.b_lo = S->dmap_lo;
    tp.M = N; tp.N = Vs; tp.bias = S->b; tp.C = S->logits.as<float>(); tp.ldc = Vs;
    // the epilogue also leaves each tile's maximum and exp-sum: the top-k kernel derives the normaliser and its
    // selection bound from them and then reads only the few tiles that reach the bound
    tp.part_max = S->parts.as<float>(); tp.part_sum = ps_out ? tp.part_max + (size_t)np * N : nullptr;
    pm = tp.part_max;
    if (ps_out) *ps_out = tp.part_sum;
    tp.err = tc_error_word();
    KScope ks(KC_SOFTMAX_GEMM, st);
    ZR_CUDA(zrnn::launch_tc_gemm_persistent(tp, eng_tcmode(eng), zrnn::TC_EPI_STORE, st));
  }
  *pm_out = pm;
  *np_out = np;
  if (ps_out && !pm) *ps_out = nullptr;
  return ZRNN_OK;
}
// the k best rows of this layer's part of the vocabulary per column, as log-probabilities under the layer's own
// normaliser; row numbers are local to the layer; lse (optional) receives the log of that normaliser
int softmax_topk_act(zrnn_softmax* S, const Act& h, int N, int k, float* logp, int* idx, float* eos, cudaStream_t st,
                     float* lse = nullptr) {
  const float *pm = nullptr, *ps = nullptr;
  int np = 0;
  ZR_TRY(softmax_logits_act(S, h, N, st, &pm, &np, &ps));
  KScope ks(KC_SOFTMAX_REDUCE, st);
  const int Vs = S->hi - S->lo;
  const int eos_row = (1 >= S->lo && 1 < S->hi) ? 1 - S->lo : -1;  // <EOF> is word 1
  ZR_CUDA(zrnn::launch_topk_logp(S->logits.as<float>(), Vs, N, k, logp, idx, eos, st, pm, ps, np,
                                 S->BN / zrnn::kPersistentParts, eos_row, lse));
  return ZRNN_OK;
}

// pack G column-major (rows x K) matrices into operand form at K offset koff
int pack_into(OpMem& dst, int eng, const float* const* src, int G, int rows, int K, int lda, int TH, int n_tiles,
              int ld_dst, int koff, int tiled_kbtot = 0) {
  zrnn::PackArgs pk;
  std::memset(&pk, 0, sizeof(pk));
  for (int g = 0; g < G; ++g) pk.src[g] = src[g];
  pk.G = G; pk.H = rows; pk.K = K; pk.lda = lda; pk.TH = TH; pk.n_tiles = n_tiles;
  pk.dst_hi = dst.hi; pk.dst_lo = dst.lo; pk.op_mode = eng_opmode(eng); pk.ld_dst = ld_dst; pk.koff = koff;
  pk.tiled_kbtot = tiled_kbtot; pk.tiled_epk = 128 / eng_eb(eng);
  ZR_CUDA(zrnn::launch_pack_weights(pk, nullptr));
  return ZRNN_OK;
}
int weight_maps(const OpMem& w, int eng, long long K, long long rows, int box_rows, CUtensorMap* hi, CUtensorMap* lo) {
  if (!zrnn::make_kmajor_map(hi, w.hi, eng_eb(eng), K, rows, K, box_rows))
    return fail(ZRNN_E_CUDA, "cannot encode a TMA tensor map for a weight operand");
  if (eng_split(eng) && !zrnn::make_kmajor_map(lo, w.lo, eng_eb(eng), K, rows, K, box_rows))
    return fail(ZRNN_E_CUDA, "cannot encode a TMA tensor map for a weight operand (lo)");
  return ZRNN_OK;
}

}  // namespace

// ------------------------------------------------------------------------------------------
// model
// ------------------------------------------------------------------------------------------
struct TensorSlot {
  std::string name;
  int rows, cols;
  int owner;  // 0 = src layer, 1 = tgt layer, 2 = attention, 3 = softmax
  int layer;
  int index;  // position in the owner's load list
};

struct zrnn_model {
  zrnn_model_config cfg;
  int eng = ENG_SIMT;
  std::vector<zrnn_lstm_layer*> src, tgt;
  zrnn_attention* att = nullptr;
  zrnn_softmax* sm = nullptr;
  std::vector<TensorSlot> slots;
  std::vector<std::vector<float>> staged;
  std::vector<char> have_host;     // per slot: host data staged since the last upload
  std::set<size_t> group_loaded;   // first slot of every tensor group that is on the device
  bool finalized = false;
  cudaStream_t stream = nullptr;
  DevBuf ws, io;
  DevBuf dec_counter;       // phase counter of the persistent decoder kernel
  DevBuf seq_xp;            // input half of the pre-activations for the resident-weight sequence kernel
  int persist_state = 0;    // 0 untried, 1 works, -1 refused by the runtime (the per-launch path is used)
  zrnn::TcMulti enc_multi;  // parameter block of the encoder's multi-cell launches (host scratch)
  const float* last_top = nullptr;
  int last_top_cols = 0;
  Act last_top_act;  // the same vectors with their operand-form copies
  bool sharded = false;  // the softmax layer holds a slice of the vocabulary: scoring / decoding need a zrnn_comm
  std::vector<int> h_tmp;
  // CUDA graph of one scoring pass, replayed while the shapes, buffers and stream stay the same
  struct ScoreGraph {
    int S = -1, T = -1, B = -1;
    const void *src = nullptr, *tin = nullptr, *tout = nullptr, *out = nullptr;
    void* ws = nullptr;
    unsigned long long gen = 0;
    cudaStream_t stream = nullptr;
    int seen = 0;
    int persistent = 0;  // the pass was recorded with the persistent decoder kernel switched on
    cudaGraphExec_t exec = nullptr;
  } sg;
  void drop_graph() {
    if (sg.exec) cudaGraphExecDestroy(sg.exec);
    sg = ScoreGraph();
  }
  ~zrnn_model() {
    drop_graph();
    for (auto* l : src) delete l;
    for (auto* l : tgt) delete l;
    delete att;
    delete sm;
    ws.release(); io.release(); dec_counter.release(); seq_xp.release();
    if (stream) cudaStreamDestroy(stream);
  }
};


namespace {
// Host id arrays: -1 is padding, everything else must index the vocabulary.  An id from another vocabulary would make
// the embedding gather read past its table.
int check_ids(const int* ids, size_t n, int V, const char* what) {
  for (size_t i = 0; i < n; ++i)
    if (ids[i] < -1 || ids[i] >= V)
      return fail(ZRNN_E_ARG, std::string(what) + ": token id " + std::to_string(ids[i]) + " at position " +
                                  std::to_string(i) + " is outside the vocabulary of " + std::to_string(V) + " words");
  return ZRNN_OK;
}
// Reads and clears the device error word after a synchronised pass and turns it into a status.
int device_error_status(const char* what) {
  const int code = zrnn_tc_error();
  if (code == 0) return ZRNN_OK;
  if (code == zrnn::kErrBadTokenId)
    return fail(ZRNN_E_ARG, std::string(what) + ": a token id on the device is outside the vocabulary (column 0 was read instead)");
  return fail(ZRNN_E_TIMEOUT, std::string(what) + ": a bounded device wait gave up (role " + std::to_string(code) + ")");
}
}  // namespace

extern "C" {

const char* zrnn_status_string(int s) {
  switch (s) {
    case ZRNN_OK: return "ok";
    case ZRNN_E_ARG: return "invalid argument";
    case ZRNN_E_CUDA: return "CUDA error";
    case ZRNN_E_NCCL: return "NCCL error";
    case ZRNN_E_TIMEOUT: return "device wait timed out";
    case ZRNN_E_IO: return "weight file error";
    case ZRNN_E_STATE: return "invalid call order";
  }
  return "unknown status";
}
const char* zrnn_last_error(void) { return g_err.c_str(); }
int zrnn_version(void) { return 100; }
int zrnn_built_for_sm(void) { return 100; }
int zrnn_device_count(int* n) {
  ZR_CHECK(n, "device_count: null argument");
  *n = 0;
  ZR_CUDA(cudaGetDeviceCount(n));
  return ZRNN_OK;
}
int zrnn_set_device(int device) {
  ZR_CUDA(cudaSetDevice(device));
  return ZRNN_OK;
}
long long zrnn_launch_count(void) { return zrnn::launch_count_value(); }
void zrnn_reset_launch_count(void) { zrnn::launch_count_reset(); }

/* developer aid: LSTM tensor-core launches write 8 globaltimer stamps per CTA into buf */
int zrnn_debug_tc_profile(long long* d_buf) {
  g_tc_prof = d_buf;
  g_tc_prof_slot = -1;
  return ZRNN_OK;
}
/* timeline mode: every tensor-core launch gets the next of `slots` 8-stamp records (CTA 0 only) */
int zrnn_debug_tc_timeline(long long* d_buf, int slots) {
  g_tc_prof = d_buf;
  g_tc_prof_slot = d_buf ? 0 : -1;
  g_tc_prof_cap = slots;
  return ZRNN_OK;
}

/* developer aid: CTA `cta` of every persistent decoder launch writes 8 stamps per phase (phase entered, accumulators
 * complete, cluster ready, partial tile pushed, exchange complete, results stored, earlier phases complete, counted)
 * to d_buf[phase * 8 ..]; NULL switches it off */
int zrnn_debug_decoder_timeline(long long* d_buf, int cta) {
  g_dec_detail = d_buf;
  g_dec_detail_cta = cta;
  return ZRNN_OK;
}

int zrnn_debug_bounded_wait(long long limit_cycles, void* stream) {
  ZR_CHECK(limit_cycles > 0 && limit_cycles <= 2000000000LL, "debug_bounded_wait: limit must be in (0, 2e9] cycles");
  ZR_TRY(check_device());
  ZR_CUDA(zrnn::launch_wait_probe(tc_error_word(), limit_cycles, 77, (cudaStream_t)stream));
  return ZRNN_OK;
}

int zrnn_tc_error(void) {
  int* d = tc_error_word();
  int v = 0;
  if (!d) return -1;
  if (cudaMemcpy(&v, d, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(d, 0, sizeof(int));
  return v;
}

int zrnn_kernel_timing(int on) {
  g_kt.on = on != 0;
  if (on) {
    g_kt.used = 0;
    g_kt.drop_dec_runs();
  }
  return ZRNN_OK;
}
int zrnn_kernel_timing_read(int kernel_class, long long* launches, double* total_ms) {
  ZR_CHECK(kernel_class >= 0 && kernel_class < KC_COUNT && launches && total_ms, "kernel_timing_read: bad arguments");
  *launches = 0;
  *total_ms = 0.0;
  for (size_t i = 0; i < g_kt.used; ++i) {
    if (g_kt.cls[i] != kernel_class) continue;
    ZR_CUDA(cudaEventSynchronize(g_kt.ev[2 * i + 1]));
    float ms = 0.f;
    ZR_CUDA(cudaEventElapsedTime(&ms, g_kt.ev[2 * i], g_kt.ev[2 * i + 1]));
    *launches += g_kt.cnt[i];
    *total_ms += ms;
  }
  if (kernel_class == KC_LSTM || kernel_class == KC_ATT) {
    // phases of the persistent decoder launches: stamps[0] = kernel start, stamps[1 + ph] = end of phase ph; phases
    // 0 .. L-1 of a step are the cells, the rest (stacked local-p GEMM, attention, combiner) is the attention group
    ZR_CUDA(cudaDeviceSynchronize());
    std::vector<long long> st;
    for (const auto& r : g_kt.dec_runs) {
      const int NP = r.T * r.P;
      st.resize((size_t)NP + 1);
      ZR_CUDA(cudaMemcpy(st.data(), r.d_stamps, sizeof(long long) * st.size(), cudaMemcpyDeviceToHost));
      for (int ph = 0; ph < NP; ++ph) {
        const bool cell = (ph % r.P) < r.L;
        if (cell != (kernel_class == KC_LSTM) || st[ph + 1] == 0 || st[ph] == 0) continue;
        *total_ms += (double)(st[ph + 1] - st[ph]) * 1e-6;
        if (cell) *launches += 1;
        else if ((ph % r.P) == r.P - 1) *launches += 1;  // one attention group per step
      }
    }
  }
  return ZRNN_OK;
}

int zrnn_prep_vocab_indices(const int* d_ids_raw, int n, int* d_ids_nonm1, int* d_mask01, void* stream) {
  ZR_CHECK(d_ids_raw && n >= 0, "prep_vocab_indices: null ids or negative n");
  ZR_CUDA(zrnn::launch_prep_ids(d_ids_raw, n, d_ids_nonm1, d_mask01, (cudaStream_t)stream));
  return ZRNN_OK;
}

// ---------------------------------------------------------------- LSTM layers
static int lstm_create(int H, int V, int feed, int dtype, int is_ih, zrnn_lstm_layer** out) {
  ZR_CHECK(out, "lstm_create: null out");
  ZR_CHECK(H > 0, "lstm_create: H must be positive");
  ZR_CHECK(!is_ih || V > 0, "ih_create: V must be positive");
  int eng = ENG_SIMT;
  ZR_TRY(pick_engine(dtype, H, &eng));
  ZR_TRY(check_device());
  auto* L = new zrnn_lstm_layer();
  L->H = H; L->V = V; L->feed = feed ? 1 : 0; L->dtype = dtype; L->is_ih = is_ih; L->eng = eng;
  L->Kpad = round64(H);
  *out = L;
  return ZRNN_OK;
}
int zrnn_ih_create(int H, int V, int feed_input, int dtype, zrnn_lstm_layer** out) {
  return lstm_create(H, V, feed_input, dtype, 1, out);
}
int zrnn_hh_create(int H, int dtype, zrnn_lstm_layer** out) { return lstm_create(H, 0, 0, dtype, 0, out); }

int zrnn_lstm_load(zrnn_lstm_layer* L, const float* const* t, int n) {
  ZR_CHECK(L && t, "lstm_load: null argument");
  const int expect = 12 + (L->is_ih ? 1 : 0) + (L->feed ? 4 : 0);
  ZR_CHECK(n == expect, "lstm_load: expected " + std::to_string(expect) + " tensors, got " + std::to_string(n));
  for (int i = 0; i < n; ++i) ZR_CHECK(t[i], "lstm_load: null tensor " + std::to_string(i));
  const int H = L->H;
  const size_t HH = (size_t)H * H;
  {
    int q = 8;
    for (int g = 0; g < 4; ++g) ZR_TRY(check_f16_range(L->eng, t[2 * g], HH, "lstm_load"));
    if (L->is_ih) ZR_TRY(check_f16_range(L->eng, t[q++], (size_t)H * L->V, "lstm_load (embedding)"));
    for (int k = 0; k < (L->feed ? 8 : 4); ++k) ZR_TRY(check_f16_range(L->eng, t[q + k], HH, "lstm_load"));
  }
  ++g_buf_generation;  // every weight buffer moves: graphs captured over the old ones must not be replayed
  cudaFree(L->W); cudaFree(L->Wh); cudaFree(L->Mx); cudaFree(L->Q); cudaFree(L->b);
  L->W = L->Wh = L->Mx = L->Q = L->b = nullptr;
  L->loaded = false;
  // file order: W_hi b_i W_hf b_f W_hc b_c W_ho b_o [W] M_i M_f M_o M_c [Q_i Q_f Q_o Q_c]; device gate order i,f,g,o
  std::vector<float> pack(4 * HH);
  for (int g = 0; g < 4; ++g) std::memcpy(pack.data() + g * HH, t[2 * g], sizeof(float) * HH);
  ZR_CUDA(upload(&L->Wh, pack.data(), 4 * HH));
  std::vector<float> bias(4 * (size_t)H);
  for (int g = 0; g < 4; ++g) std::memcpy(bias.data() + (size_t)g * H, t[2 * g + 1], sizeof(float) * H);
  ZR_CUDA(upload(&L->b, bias.data(), 4 * (size_t)H));
  int p = 8;
  if (L->is_ih) { ZR_CUDA(upload(&L->W, t[p], (size_t)H * L->V)); ++p; }
  const int order[4] = {0, 1, 3, 2};  // file i,f,o,c -> gate slots i,f,o(3),g(2)
  for (int k = 0; k < 4; ++k) std::memcpy(pack.data() + order[k] * HH, t[p + k], sizeof(float) * HH);
  ZR_CUDA(upload(&L->Mx, pack.data(), 4 * HH));
  p += 4;
  if (L->feed) {
    for (int k = 0; k < 4; ++k) std::memcpy(pack.data() + order[k] * HH, t[p + k], sizeof(float) * HH);
    ZR_CUDA(upload(&L->Q, pack.data(), 4 * HH));
  }
  if (L->eng != ENG_SIMT) {
    // operand form: gate-interleaved rows (tile of TH hidden units x 4 gates), K axis = x | h | htild
    const int TH = L->BN / 4, Kpad = L->Kpad, nsrc = L->feed ? 3 : 2;
    L->n_tiles = (H + TH - 1) / TH;
    const long long rows = (long long)L->n_tiles * L->BN, Kcat = (long long)nsrc * Kpad;
    ZR_TRY(L->Wcat.alloc((size_t)rows * Kcat, L->eng));
    // Tile-contiguous storage: the 128 rows x 128 bytes a CTA fetches per k-block are one 16 KB chunk of memory
    // instead of 128 pieces that lie a whole row (8-12 KB) apart, so the weight stream reads whole DRAM pages.
    static const bool tiled = std::getenv("ZRNN_WEIGHT_ROWMAJOR") == nullptr;
    const int epk = 128 / eng_eb(L->eng);
    L->kbtot = tiled ? (int)(Kcat / epk) : 0;
    const float* srcs[3] = {L->Mx, L->Wh, L->Q};
    for (int s = 0; s < nsrc; ++s) {
      const float* g4[4] = {srcs[s], srcs[s] + HH, srcs[s] + 2 * HH, srcs[s] + 3 * HH};
      ZR_TRY(pack_into(L->Wcat, L->eng, g4, 4, H, H, H, TH, L->n_tiles, (int)Kcat, s * Kpad, L->kbtot));
    }
    if (tiled) ZR_TRY(weight_maps(L->Wcat, L->eng, epk, rows * L->kbtot, L->BN, &L->wmap, &L->wmap_lo));
    else ZR_TRY(weight_maps(L->Wcat, L->eng, Kcat, rows, L->BN, &L->wmap, &L->wmap_lo));
    if (L->is_ih) {
      ZR_TRY(L->emb.alloc((size_t)L->V * Kpad, L->eng));
      ZR_CUDA(zrnn::launch_convert_rows(L->W, L->V, H, H, eng_opmode(L->eng), L->emb.hi, L->emb.lo, Kpad, nullptr));
    }
    ZR_CUDA(cudaDeviceSynchronize());
  }
  L->loaded = true;
  return ZRNN_OK;
}

int zrnn_ih_gather(zrnn_lstm_layer* L, const int* d_ids, int n_cols, float* d_x, void* stream) {
  ZR_CHECK(L && L->is_ih, "ih_gather: not an input layer");
  if (!L->loaded) return fail(ZRNN_E_STATE, "ih_gather: weights not loaded");
  ZR_CHECK(d_ids && d_x && n_cols >= 0, "ih_gather: bad arguments");
  ZR_CUDA(zrnn::launch_gather_columns(L->W, L->H, L->V, d_ids, n_cols, d_x, tc_error_word(), (cudaStream_t)stream));
  return ZRNN_OK;
}

// gather layer-0 inputs in the form the engine consumes
static int gather_act(zrnn_lstm_layer* L, const int* ids, int n, const Act& x, cudaStream_t st) {
  KScope ks(KC_GATHER, st);
  if (L->eng == ENG_SIMT) {
    ZR_CUDA(zrnn::launch_gather_columns(L->W, L->H, L->V, ids, n, x.f32, tc_error_word(), st));
    return ZRNN_OK;
  }
  const size_t rb = (size_t)L->Kpad * eng_eb(L->eng);
  ZR_CUDA(zrnn::launch_gather_rows16(L->emb.hi, rb, L->V, ids, n, x.hi, tc_error_word(), st));
  if (eng_split(L->eng)) ZR_CUDA(zrnn::launch_gather_rows16(L->emb.lo, rb, L->V, ids, n, x.lo, tc_error_word(), st));
  return ZRNN_OK;
}

static int layer_forward_f32(zrnn_lstm_layer* L, const int* d_ids, const float* d_x, const int* d_mask,
                             const float* d_h_prev, const float* d_c_prev, const float* d_htild, int B, float* d_h_out,
                             float* d_c_out, cudaStream_t st) {
  const int H = L->H;
  Act x, hp, q, out;
  out.f32 = d_h_out;
  if (L->eng == ENG_SIMT) {
    if (d_ids) {
      ZR_CUDA(L->x.reserve(sizeof(float) * (size_t)H * B));
      x.f32 = L->x.as<float>();
      ZR_TRY(gather_act(L, d_ids, B, x, st));
    } else x.f32 = const_cast<float*>(d_x);
    hp.f32 = const_cast<float*>(d_h_prev);
    q.f32 = const_cast<float*>(d_htild);
  } else {
    if (d_ids) {
      ZR_CUDA(L->sc_x.reserve((size_t)B * L->Kpad * eng_eb(L->eng)));
      if (eng_split(L->eng)) ZR_CUDA(L->sc_xl.reserve((size_t)B * L->Kpad * eng_eb(L->eng)));
      x.hi = L->sc_x.p;
      x.lo = eng_split(L->eng) ? L->sc_xl.as<float>() : nullptr;
      ZR_TRY(gather_act(L, d_ids, B, x, st));
    } else {
      ZR_TRY(to_operand(d_x, H, L->Kpad, B, L->eng, L->sc_x, L->sc_xl, &x, st));
    }
    ZR_TRY(to_operand(d_h_prev, H, L->Kpad, B, L->eng, L->sc_h, L->sc_hl, &hp, st));
    if (d_htild) ZR_TRY(to_operand(d_htild, H, L->Kpad, B, L->eng, L->sc_q, L->sc_ql, &q, st));
  }
  return cell_forward(L, x, hp, d_htild ? &q : nullptr, d_mask, d_c_prev, B, out, d_c_out, st);
}

int zrnn_ih_forward(zrnn_lstm_layer* L, const int* d_ids, const int* d_mask, const float* d_h_prev,
                    const float* d_c_prev, const float* d_htild_prev, int B, float* d_h_out, float* d_c_out,
                    void* stream) {
  ZR_CHECK(L && L->is_ih, "ih_forward: not an input layer");
  if (!L->loaded) return fail(ZRNN_E_STATE, "ih_forward: weights not loaded");
  ZR_CHECK(d_ids && d_h_prev && d_c_prev && d_h_out && d_c_out && B >= 0, "ih_forward: bad arguments");
  ZR_CHECK(!d_htild_prev || L->feed, "ih_forward: htild given but the layer has no feed-input weights");
  ZR_CHECK(d_h_out != d_h_prev && d_c_out != d_c_prev, "ih_forward: outputs may not alias inputs");
  if (B == 0) return ZRNN_OK;
  return layer_forward_f32(L, d_ids, nullptr, d_mask, d_h_prev, d_c_prev, d_htild_prev, B, d_h_out, d_c_out,
                           (cudaStream_t)stream);
}

int zrnn_hh_forward(zrnn_lstm_layer* L, const float* d_h_below, const int* d_mask, const float* d_h_prev,
                    const float* d_c_prev, int B, float* d_h_out, float* d_c_out, void* stream) {
  ZR_CHECK(L, "hh_forward: null layer");
  if (!L->loaded) return fail(ZRNN_E_STATE, "hh_forward: weights not loaded");
  ZR_CHECK(d_h_below && d_h_prev && d_c_prev && d_h_out && d_c_out && B >= 0, "hh_forward: bad arguments");
  ZR_CHECK(d_h_out != d_h_prev && d_c_out != d_c_prev, "hh_forward: outputs may not alias inputs");
  if (B == 0) return ZRNN_OK;
  return layer_forward_f32(L, nullptr, d_h_below, d_mask, d_h_prev, d_c_prev, nullptr, B, d_h_out, d_c_out,
                           (cudaStream_t)stream);
}
int zrnn_lstm_destroy(zrnn_lstm_layer* L) {
  delete L;
  return ZRNN_OK;
}

// ---------------------------------------------------------------- attention
int zrnn_att_create(int H, int D, int att_type, int dtype, zrnn_attention** out) {
  ZR_CHECK(out, "att_create: null out");
  ZR_CHECK(H > 0, "att_create: H must be positive");
  ZR_CHECK(att_type == ZRNN_ATT_LOCAL_P || att_type == ZRNN_ATT_GLOBAL_DOT, "att_create: unknown attention type");
  ZR_CHECK(att_type != ZRNN_ATT_LOCAL_P || (D >= 1 && 2 * D + 1 <= 64), "att_create: D must be in [1,31]");
  int eng = ENG_SIMT;
  ZR_TRY(pick_engine(dtype, H, &eng));
  ZR_TRY(check_device());
  auto* A = new zrnn_attention();
  A->H = H; A->D = D; A->type = att_type; A->dtype = dtype; A->eng = eng; A->Kpad = round64(H);
  *out = A;
  return ZRNN_OK;
}
int zrnn_att_load(zrnn_attention* A, const float* const* t, int n) {
  ZR_CHECK(A && t, "att_load: null argument");
  ZR_CHECK(n == 6, "att_load: expected 6 tensors (W_a W_p v_p output_bias W_c_p1 W_c_p2)");
  for (int i = 0; i < n; ++i) ZR_CHECK(t[i], "att_load: null tensor");
  const int H = A->H;
  const size_t HH = (size_t)H * H;
  for (int i : {0, 1, 4, 5}) ZR_TRY(check_f16_range(A->eng, t[i], HH, "att_load"));
  ++g_buf_generation;
  cudaFree(A->WpWaT); cudaFree(A->v_p); cudaFree(A->bias); cudaFree(A->Wc1); cudaFree(A->Wc2);
  A->WpWaT = A->v_p = A->bias = A->Wc1 = A->Wc2 = nullptr;
  A->loaded = false;
  if (A->type == ZRNN_ATT_LOCAL_P) {
    // rows 0..H-1 = W_p, rows H..2H-1 = W_a^T, so one GEMM gives tanh(W_p h) and q = W_a^T h
    std::vector<float> st(2 * HH);
    const float* Wa = t[0];
    const float* Wp = t[1];
    for (int k = 0; k < H; ++k)
      for (int r = 0; r < H; ++r) {
        st[(size_t)k * 2 * H + r] = Wp[(size_t)k * H + r];
        st[(size_t)k * 2 * H + H + r] = Wa[(size_t)r * H + k];
      }
    ZR_CUDA(upload(&A->WpWaT, st.data(), 2 * HH));
    ZR_CUDA(upload(&A->v_p, t[2], H));
  }
  ZR_CUDA(upload(&A->bias, t[3], H));
  ZR_CUDA(upload(&A->Wc1, t[4], HH));
  ZR_CUDA(upload(&A->Wc2, t[5], HH));
  if (A->eng != ENG_SIMT) {
    const int Kpad = A->Kpad, BN = A->BN;
    if (A->type == ZRNN_ATT_LOCAL_P) {
      const int nt = (2 * H + BN - 1) / BN;
      ZR_TRY(A->WpWaT_op.alloc((size_t)nt * BN * Kpad, A->eng));
      const float* g1[1] = {A->WpWaT};
      ZR_TRY(pack_into(A->WpWaT_op, A->eng, g1, 1, 2 * H, H, 2 * H, BN, nt, Kpad, 0));
      ZR_TRY(weight_maps(A->WpWaT_op, A->eng, Kpad, (long long)nt * BN, BN, &A->pmap, &A->pmap_lo));
    }
    const int nt = (H + BN - 1) / BN;
    ZR_TRY(A->Wc_op.alloc((size_t)nt * BN * 2 * Kpad, A->eng));
    const float* c1[1] = {A->Wc1};
    const float* c2[1] = {A->Wc2};
    ZR_TRY(pack_into(A->Wc_op, A->eng, c1, 1, H, H, H, BN, nt, 2 * Kpad, 0));
    ZR_TRY(pack_into(A->Wc_op, A->eng, c2, 1, H, H, H, BN, nt, 2 * Kpad, Kpad));
    ZR_TRY(weight_maps(A->Wc_op, A->eng, 2 * Kpad, (long long)nt * BN, BN, &A->cmap, &A->cmap_lo));
    ZR_CUDA(cudaDeviceSynchronize());
  }
  A->loaded = true;
  return ZRNN_OK;
}
int zrnn_att_set_source(zrnn_attention* A, const float* d_hs, int S_max, int B_src, const int* d_len,
                        const int* d_offset, int cols_per_sentence) {
  ZR_CHECK(A && d_hs && d_len && d_offset, "att_set_source: null argument");
  ZR_CHECK(S_max > 0 && B_src > 0 && cols_per_sentence > 0, "att_set_source: sizes must be positive");
  ZR_CHECK(S_max <= 10000, "att_set_source: S_max too large");
  A->hs = d_hs; A->S_max = S_max; A->B_src = B_src; A->len = d_len; A->off = d_offset;
  A->cols_per_sent = cols_per_sentence;
  return ZRNN_OK;
}
static thread_local int* g_att_viterbi_out = nullptr;  // set only inside zrnn_att_forward_viterbi
int zrnn_att_forward(zrnn_attention* A, const float* d_h_t, const int* d_mask, int B, float* d_htild_out,
                     float* d_align_out, void* stream) {
  ZR_CHECK(A && d_h_t && d_htild_out && B >= 0, "att_forward: bad arguments");
  if (!A->loaded) return fail(ZRNN_E_STATE, "att_forward: weights not loaded");
  if (!A->hs) return fail(ZRNN_E_STATE, "att_forward: zrnn_att_set_source has not been called");
  ZR_CHECK(B <= A->B_src * A->cols_per_sent, "att_forward: more target columns than source columns provide");
  if (B == 0) return ZRNN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  Act h, out;
  h.f32 = const_cast<float*>(d_h_t);
  out.f32 = d_htild_out;
  if (A->eng != ENG_SIMT) ZR_TRY(to_operand(d_h_t, A->H, A->Kpad, B, A->eng, A->sc_h, A->sc_hl, &h, st));
  return att_forward(A, h, d_mask, B, out, d_align_out, st, g_att_viterbi_out);
}
int zrnn_att_forward_viterbi(zrnn_attention* A, const float* d_h_t, const int* d_mask, int B, float* d_htild_out,
                             int* d_viterbi_out, void* stream) {
  ZR_CHECK(d_viterbi_out, "att_forward_viterbi: null output");
  g_att_viterbi_out = d_viterbi_out;
  const int st = zrnn_att_forward(A, d_h_t, d_mask, B, d_htild_out, nullptr, stream);
  g_att_viterbi_out = nullptr;
  return st;
}
int zrnn_att_destroy(zrnn_attention* A) {
  delete A;
  return ZRNN_OK;
}

// ---------------------------------------------------------------- softmax
int zrnn_softmax_create(int V, int H, int dtype, int shard_lo, int shard_hi, zrnn_softmax** out) {
  ZR_CHECK(out, "softmax_create: null out");
  ZR_CHECK(V > 0 && H > 0, "softmax_create: V and H must be positive");
  ZR_CHECK(0 <= shard_lo && shard_lo < shard_hi && shard_hi <= V, "softmax_create: bad shard range");
  int eng = ENG_SIMT;
  ZR_TRY(pick_engine(dtype, H, &eng));
  ZR_TRY(check_device());
  auto* S = new zrnn_softmax();
  S->V = V; S->H = H; S->dtype = dtype; S->lo = shard_lo; S->hi = shard_hi; S->eng = eng; S->Kpad = round64(H);
  S->BN = eng_split(eng) ? 128 : 256;
  *out = S;
  return ZRNN_OK;
}
int zrnn_softmax_load(zrnn_softmax* S, const float* h_D, const float* h_b_d) {
  ZR_CHECK(S && h_D && h_b_d, "softmax_load: null argument");
  ZR_TRY(check_f16_range(S->eng, h_D, (size_t)S->V * S->H, "softmax_load"));
  ++g_buf_generation;
  cudaFree(S->D); cudaFree(S->b);
  S->D = S->b = nullptr;
  S->loaded = false;
  const int Vs = S->hi - S->lo;
  ZR_CUDA(cudaMalloc((void**)&S->D, sizeof(float) * (size_t)Vs * S->H));
  ZR_CUDA(cudaMemcpy2D(S->D, sizeof(float) * (size_t)Vs, h_D + S->lo, sizeof(float) * (size_t)S->V,
                       sizeof(float) * (size_t)Vs, S->H, cudaMemcpyHostToDevice));
  ZR_CUDA(upload(&S->b, h_b_d + S->lo, Vs));
  if (S->eng != ENG_SIMT) {
    S->n_tiles = (Vs + S->BN - 1) / S->BN;
    ZR_TRY(S->D_op.alloc((size_t)S->n_tiles * S->BN * S->Kpad, S->eng));
    const float* g1[1] = {S->D};
    ZR_TRY(pack_into(S->D_op, S->eng, g1, 1, Vs, S->H, Vs, S->BN, S->n_tiles, S->Kpad, 0));
    ZR_TRY(weight_maps(S->D_op, S->eng, S->Kpad, (long long)S->n_tiles * S->BN, S->BN, &S->dmap, &S->dmap_lo));
    ZR_CUDA(cudaDeviceSynchronize());
  }
  S->loaded = true;
  return ZRNN_OK;
}
static int softmax_input(zrnn_softmax* S, const float* d_h, int N, Act* h, cudaStream_t st) {
  h->f32 = const_cast<float*>(d_h);
  if (S->eng != ENG_SIMT) ZR_TRY(to_operand(d_h, S->H, S->Kpad, N, S->eng, S->sc_h, S->sc_hl, h, st));
  return ZRNN_OK;
}
int zrnn_softmax_partials(zrnn_softmax* S, const float* d_h, const int* d_targets, int N, float* d_max, float* d_sum,
                          float* d_tgt, void* stream) {
  ZR_CHECK(S && d_h && d_targets && d_max && d_sum && d_tgt && N >= 0, "softmax_partials: bad arguments");
  if (!S->loaded) return fail(ZRNN_E_STATE, "softmax_partials: weights not loaded");
  if (N == 0) return ZRNN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  Act h;
  ZR_TRY(softmax_input(S, d_h, N, &h, st));
  int np = 0;
  float *pm, *ps;
  ZR_TRY(softmax_partials_launch(S, h, d_targets, N, &np, &pm, &ps, d_tgt, st));
  // reduce this shard's row tiles to one (max, sum) per column
  KScope ks(KC_SOFTMAX_REDUCE, st);
  ZR_CUDA(zrnn::launch_lse_reduce(pm, ps, np, N, d_max, d_sum, st));
  return ZRNN_OK;
}
int zrnn_softmax_combine(const float* d_max, const float* d_sum, const float* d_tgt, int G, int N,
                         const int* d_mask, float* d_logp_out, void* stream) {
  ZR_CHECK(d_max && d_sum && d_tgt && d_logp_out && G >= 1 && N >= 0, "softmax_combine: bad arguments");
  if (N == 0) return ZRNN_OK;
  ZR_CUDA(zrnn::launch_lse_combine_shards(d_max, d_sum, d_tgt, G, N, d_mask, d_logp_out, (cudaStream_t)stream));
  return ZRNN_OK;
}
int zrnn_softmax_score(zrnn_softmax* S, const float* d_h, const int* d_targets, const int* d_mask, int N,
                       float* d_logp_out, void* stream) {
  ZR_CHECK(S && d_h && d_targets && d_logp_out && N >= 0, "softmax_score: bad arguments");
  if (!S->loaded) return fail(ZRNN_E_STATE, "softmax_score: weights not loaded");
  ZR_CHECK(S->lo == 0 && S->hi == S->V, "softmax_score: layer is vocabulary-sharded; use partials + combine");
  if (N == 0) return ZRNN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  Act h;
  ZR_TRY(softmax_input(S, d_h, N, &h, st));
  return softmax_score_act(S, h, d_targets, d_mask, N, d_logp_out, st);
}
int zrnn_softmax_topk(zrnn_softmax* S, const float* d_h, int N, int k, float* d_logp_out, int* d_idx_out,
                      float* d_logp_eos, void* stream) {
  ZR_CHECK(S && d_h && d_logp_out && d_idx_out && N >= 0, "softmax_topk: bad arguments");
  ZR_CHECK(k >= 1 && k <= ZR_BEAM_MAX + 1, "softmax_topk: k must be in [1,33]");
  if (!S->loaded) return fail(ZRNN_E_STATE, "softmax_topk: weights not loaded");
  ZR_CHECK(S->lo == 0 && S->hi == S->V, "softmax_topk: layer is vocabulary-sharded");
  if (N == 0) return ZRNN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  Act h;
  ZR_TRY(softmax_input(S, d_h, N, &h, st));
  return softmax_topk_act(S, h, N, k, d_logp_out, d_idx_out, d_logp_eos, st);
}
int zrnn_softmax_destroy(zrnn_softmax* S) {
  delete S;
  return ZRNN_OK;
}

// ---------------------------------------------------------------- model
static void add_lstm_slots(zrnn_model* m, const std::string& pre, int owner, int layer, int H, int V_emb, bool feed) {
  int idx = 0;
  auto add = [&](const std::string& n, int r, int c) { m->slots.push_back({pre + "." + n, r, c, owner, layer, idx++}); };
  const char* g1[4] = {"i", "f", "c", "o"};
  for (int g = 0; g < 4; ++g) { add(std::string("W_h") + g1[g], H, H); add(std::string("b_") + g1[g], H, 1); }
  if (V_emb > 0) add("W", H, V_emb);
  const char* g2[4] = {"i", "f", "o", "c"};
  for (int g = 0; g < 4; ++g) add(std::string("M_") + g2[g], H, H);
  if (feed) for (int g = 0; g < 4; ++g) add(std::string("Q_") + g2[g], H, H);
}

static int model_create_impl(const zrnn_model_config* c, int shard_lo, int shard_hi, zrnn_model** out);
int zrnn_model_create(const zrnn_model_config* c, zrnn_model** out) {
  ZR_CHECK(c && out, "model_create: null argument");
  return model_create_impl(c, 0, c->V_tgt, out);
}
int zrnn_model_create_sharded(const zrnn_model_config* c, int shard_lo, int shard_hi, zrnn_model** out) {
  ZR_CHECK(c && out, "model_create_sharded: null argument");
  ZR_CHECK(0 <= shard_lo && shard_lo < shard_hi && shard_hi <= c->V_tgt, "model_create_sharded: bad vocabulary range");
  return model_create_impl(c, shard_lo, shard_hi, out);
}
static int model_create_impl(const zrnn_model_config* c, int shard_lo, int shard_hi, zrnn_model** out) {
  ZR_CHECK(c && out, "model_create: null argument");
  ZR_CHECK(c->num_layers >= 1 && c->num_layers <= 8, "model_create: num_layers must be in [1,8]");
  ZR_CHECK(c->H > 0 && c->V_tgt > 1, "model_create: H and V_tgt must be positive");
  ZR_CHECK(c->lm || c->V_src > 0, "model_create: V_src must be positive for a sequence-to-sequence model");
  ZR_CHECK(c->attention >= 0 && c->attention <= 2, "model_create: unknown attention type");
  ZR_CHECK(!(c->lm && c->attention), "model_create: a language model has no source to attend to");
  ZR_CHECK(!c->feed_input || c->attention, "model_create: feed-input needs an attention model");
  int eng = ENG_SIMT;
  ZR_TRY(pick_engine(c->dtype, c->H, &eng));
  ZR_TRY(check_device());
  auto* m = new zrnn_model();
  m->cfg = *c;
  m->eng = eng;
  const int H = c->H, L = c->num_layers;
  int st = ZRNN_OK;
  if (!c->lm)
    for (int l = 0; l < L && st == ZRNN_OK; ++l) {
      zrnn_lstm_layer* ly = nullptr;
      st = l == 0 ? zrnn_ih_create(H, c->V_src, 0, c->dtype, &ly) : zrnn_hh_create(H, c->dtype, &ly);
      if (st == ZRNN_OK) {
        m->src.push_back(ly);
        add_lstm_slots(m, "src" + std::to_string(l), 0, l, H, l == 0 ? c->V_src : 0, false);
      }
    }
  for (int l = 0; l < L && st == ZRNN_OK; ++l) {
    zrnn_lstm_layer* ly = nullptr;
    st = l == 0 ? zrnn_ih_create(H, c->V_tgt, c->feed_input, c->dtype, &ly) : zrnn_hh_create(H, c->dtype, &ly);
    if (st != ZRNN_OK) break;
    m->tgt.push_back(ly);
    add_lstm_slots(m, "tgt" + std::to_string(l), 1, l, H, l == 0 ? c->V_tgt : 0, l == 0 && c->feed_input);
    if (c->attention && l == L - 1) {
      st = zrnn_att_create(H, c->D, c->attention, c->dtype, &m->att);
      const char* names[6] = {"att.W_a", "att.W_p", "att.v_p", "att.output_bias", "att.W_c_p1", "att.W_c_p2"};
      const int rows[6] = {H, H, 1, H, H, H}, cols[6] = {H, H, H, 1, H, H};
      for (int i = 0; i < 6; ++i) m->slots.push_back({names[i], rows[i], cols[i], 2, 0, i});
    }
  }
  if (st == ZRNN_OK) st = zrnn_softmax_create(c->V_tgt, H, c->dtype, shard_lo, shard_hi, &m->sm);
  m->sharded = !(shard_lo == 0 && shard_hi == c->V_tgt);
  if (st == ZRNN_OK) {
    m->slots.push_back({"softmax.D", c->V_tgt, H, 3, 0, 0});
    m->slots.push_back({"softmax.b_d", c->V_tgt, 1, 3, 0, 1});
    m->staged.resize(m->slots.size());
    m->have_host.assign(m->slots.size(), 0);
    if (cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) != cudaSuccess)
      st = fail(ZRNN_E_CUDA, "model_create: cannot create stream");
  }
  if (st != ZRNN_OK) {
    delete m;
    return st;
  }
  *out = m;
  return ZRNN_OK;
}

int zrnn_model_num_tensors(zrnn_model* m) { return m ? (int)m->slots.size() : 0; }
int zrnn_model_tensor_info(zrnn_model* m, int i, char* name, int* rows, int* cols) {
  ZR_CHECK(m && i >= 0 && i < (int)m->slots.size(), "tensor_info: bad index");
  if (name) { std::strncpy(name, m->slots[i].name.c_str(), 31); name[31] = 0; }
  if (rows) *rows = m->slots[i].rows;
  if (cols) *cols = m->slots[i].cols;
  return ZRNN_OK;
}
int zrnn_model_set_tensor(zrnn_model* m, int i, const float* h_data) {
  ZR_CHECK(m && h_data && i >= 0 && i < (int)m->slots.size(), "set_tensor: bad arguments");
  const size_t n = (size_t)m->slots[i].rows * m->slots[i].cols;
  m->staged[i].assign(h_data, h_data + n);
  m->have_host[i] = 1;
  m->finalized = false;
  m->drop_graph();  // a captured scoring pass must not outlive the weights it was captured over
  return ZRNN_OK;
}
// Uploads what zrnn_model_set_tensor staged.  Tensors belong to groups that are loaded as a whole (one LSTM layer, the
// attention layer, the softmax).  The first finalize needs every tensor; a later one re-loads exactly the groups whose
// tensors were all set again and keeps the others as they are on the device; a group of which only some tensors were
// set again is an error that names the missing tensor (the host copies of a loaded group are not kept).
int zrnn_model_finalize(zrnn_model* m) {
  ZR_CHECK(m, "finalize: null model");
  m->drop_graph();
  const size_t ns = m->slots.size();
  // groups = maximal runs of slots with the same (owner, layer)
  struct Group { size_t lo, hi; bool reload; };
  std::vector<Group> groups;
  for (size_t i = 0; i < ns;) {
    size_t j = i;
    while (j < ns && m->slots[j].owner == m->slots[i].owner && m->slots[j].layer == m->slots[i].layer) ++j;
    size_t present = 0, first_missing = ns;
    for (size_t k = i; k < j; ++k) {
      if (m->have_host[k]) ++present;
      else if (first_missing == ns) first_missing = k;
    }
    const bool was_loaded = m->group_loaded.count(i) != 0;
    if (present == j - i) groups.push_back({i, j, true});
    else if (present == 0 && was_loaded) groups.push_back({i, j, false});
    else if (present == 0)
      return fail(ZRNN_E_STATE, "finalize: tensor " + m->slots[i].name + " was never set");
    else
      return fail(ZRNN_E_STATE, "finalize: tensor " + m->slots[first_missing].name + " must be set again: its layer "
                                "was only partly updated and is loaded as a whole");
    i = j;
  }
  for (const Group& g : groups) {
    if (!g.reload) continue;
    std::vector<const float*> ptrs;
    for (size_t k = g.lo; k < g.hi; ++k) ptrs.push_back(m->staged[k].data());
    const TensorSlot& s0 = m->slots[g.lo];
    if (s0.owner == 0) ZR_TRY(zrnn_lstm_load(m->src[s0.layer], ptrs.data(), (int)ptrs.size()));
    else if (s0.owner == 1) ZR_TRY(zrnn_lstm_load(m->tgt[s0.layer], ptrs.data(), (int)ptrs.size()));
    else if (s0.owner == 2) ZR_TRY(zrnn_att_load(m->att, ptrs.data(), (int)ptrs.size()));
    else {
      ZR_CHECK(ptrs.size() == 2, "finalize: internal: softmax group");
      ZR_TRY(zrnn_softmax_load(m->sm, ptrs[0], ptrs[1]));
    }
    m->group_loaded.insert(g.lo);
    for (size_t k = g.lo; k < g.hi; ++k) {
      std::vector<float>().swap(m->staged[k]);  // the data now lives on the device
      m->have_host[k] = 0;
    }
  }
  m->finalized = true;
  return ZRNN_OK;
}

static int model_load_file_impl(const char* path, int att_type_override, int D, int dtype, int world, int rank,
                                zrnn_model** out);
int zrnn_model_load_file(const char* path, int att_type_override, int D, int dtype, zrnn_model** out) {
  return model_load_file_impl(path, att_type_override, D, dtype, 1, 0, out);
}
int zrnn_model_load_file_sharded(const char* path, int att_type_override, int D, int dtype, int world, int rank,
                                 zrnn_model** out) {
  ZR_CHECK(world >= 1 && world <= ZR_SHARD_MAX && rank >= 0 && rank < world, "load_file_sharded: bad rank / world");
  return model_load_file_impl(path, att_type_override, D, dtype, world, rank, out);
}
static int model_load_file_impl(const char* path, int att_type_override, int D, int dtype, int world, int rank,
                                zrnn_model** out) {
  ZR_CHECK(path && out, "load_file: null argument");
  zrnn::ModelFileReader rd;
  zrnn::ModelFileHeader h;
  std::string err;
  if (!rd.open(path, &h, &err)) return fail(ZRNN_E_IO, "load_file: " + err);
  if (h.multi_source || h.char_cnn) return fail(ZRNN_E_ARG, "load_file: multi-source / char-CNN models are not supported");
  zrnn_model_config c;
  std::memset(&c, 0, sizeof(c));
  c.num_layers = h.num_layers; c.H = h.H; c.V_src = h.lm ? 0 : h.V_src; c.V_tgt = h.V_tgt; c.lm = h.lm ? 1 : 0;
  c.attention = h.attention ? (att_type_override ? att_type_override : ZRNN_ATT_LOCAL_P) : ZRNN_ATT_NONE;
  c.feed_input = (h.attention && h.feed_input) ? 1 : 0;
  c.D = D > 0 ? D : 10;
  c.dtype = dtype;
  zrnn_model* m = nullptr;
  int lo = 0, hi = c.V_tgt;
  if (world > 1) shard_range(c.V_tgt, world, rank, &lo, &hi);
  ZR_TRY(model_create_impl(&c, lo, hi, &m));
  for (size_t i = 0; i < m->slots.size(); ++i) {
    m->staged[i].resize((size_t)m->slots[i].rows * m->slots[i].cols);
    m->have_host[i] = 1;
    if (!rd.read_matrix(m->slots[i].rows, m->slots[i].cols, m->staged[i].data(), &err)) {
      const std::string nm = m->slots[i].name;
      delete m;
      return fail(ZRNN_E_IO, "load_file: " + nm + ": " + err);
    }
  }
  const int st = zrnn_model_finalize(m);
  if (st != ZRNN_OK) { delete m; return st; }
  *out = m;
  return ZRNN_OK;
}

int zrnn_model_file_header(const char* path, int* header, int* n_header_ints, int* n_source_words,
                           int* n_target_words) {
  ZR_CHECK(path && header, "model_file_header: null argument");
  zrnn::ModelFileReader rd;
  zrnn::ModelFileHeader h;
  std::string err;
  if (!rd.open(path, &h, &err)) return fail(ZRNN_E_IO, "model_file_header: " + err);
  const int v[9] = {h.num_layers, h.H, h.V_tgt, h.V_src, h.attention, h.feed_input, h.multi_source, h.combine, h.char_cnn};
  for (int i = 0; i < 9; ++i) header[i] = v[i];
  if (n_header_ints) *n_header_ints = h.n_header_ints;
  if (n_source_words) *n_source_words = (int)rd.source_vocab().size();
  if (n_target_words) *n_target_words = (int)rd.target_vocab().size();
  return ZRNN_OK;
}
int zrnn_model_file_read(const char* path, int n_matrices, const int* rows, const int* cols, float* const* h_out) {
  ZR_CHECK(path && rows && cols && h_out && n_matrices >= 0, "model_file_read: bad arguments");
  zrnn::ModelFileReader rd;
  zrnn::ModelFileHeader h;
  std::string err;
  if (!rd.open(path, &h, &err)) return fail(ZRNN_E_IO, "model_file_read: " + err);
  for (int i = 0; i < n_matrices; ++i) {
    ZR_CHECK(rows[i] > 0 && cols[i] > 0 && h_out[i], "model_file_read: bad matrix shape or buffer");
    if (!rd.read_matrix(rows[i], cols[i], h_out[i], &err))
      return fail(ZRNN_E_IO, "model_file_read: matrix " + std::to_string(i) + ": " + err);
  }
  return ZRNN_OK;
}

int zrnn_model_get_config(zrnn_model* m, zrnn_model_config* cfg) {
  ZR_CHECK(m && cfg, "get_config: null argument");
  *cfg = m->cfg;
  return ZRNN_OK;
}
zrnn_softmax* zrnn_model_softmax(zrnn_model* m) { return m ? m->sm : nullptr; }
int zrnn_model_copy_top_states(zrnn_model* m, float* d_out, int capacity_cols, int* n_cols, void* stream) {
  ZR_CHECK(m && n_cols, "copy_top_states: null argument");
  *n_cols = m->last_top_cols;
  if (!d_out || !m->last_top) return ZRNN_OK;
  const int n = std::min(capacity_cols, m->last_top_cols);
  ZR_CUDA(cudaMemcpyAsync(d_out, m->last_top, sizeof(float) * (size_t)n * m->cfg.H, cudaMemcpyDeviceToDevice,
                          (cudaStream_t)stream));
  return ZRNN_OK;
}
int zrnn_model_destroy(zrnn_model* m) {
  delete m;
  return ZRNN_OK;
}

// ---------------------------------------------------------------- drivers
// A sequence of activations: `slots` consecutive H x B matrices (fp32) and/or operand-form copies.
static size_t act_bytes(const Geom& g, size_t cols, bool f32, bool op) {
  size_t b = 0;
  if (f32) b += aligned(sizeof(float) * cols * g.H);
  if (op && g.eng != ENG_SIMT) {
    b += aligned(cols * g.Kpad * eng_eb(g.eng));
    if (eng_split(g.eng)) b += aligned(cols * g.Kpad * eng_eb(g.eng));
  }
  return b;
}
static Act act_take(Carver& cv, const Geom& g, size_t cols, bool f32, bool op) {
  Act a;
  if (f32) a.f32 = cv.take<float>(cols * g.H);
  if (op && g.eng != ENG_SIMT) {
    a.hi = cv.take<char>(cols * g.Kpad * eng_eb(g.eng));
    if (eng_split(g.eng)) a.lo = (float*)cv.take<char>(cols * g.Kpad * eng_eb(g.eng));
  }
  return a;
}
static int act_zero(const Act& a, const Geom& g, size_t cols, cudaStream_t s) {
  if (a.f32) ZR_CUDA(cudaMemsetAsync(a.f32, 0, sizeof(float) * cols * g.H, s));
  if (a.hi) ZR_CUDA(cudaMemsetAsync(a.hi, 0, cols * g.Kpad * eng_eb(g.eng), s));
  if (a.lo) ZR_CUDA(cudaMemsetAsync(a.lo, 0, cols * g.Kpad * eng_eb(g.eng), s));
  return ZRNN_OK;
}

// Encoder over S steps of B columns.  seq[l] receives every step's h of layer l; c ping-pongs in cst.
// On return cur[l] indexes the final cell state of layer l.
// A stack of LSTM layers over S steps whose inputs X0 (one slot per step) are all known in advance: the source side
// always, the target side of language models and of models without feed-input.  h0[l] is layer l's state before
// step 0; its c comes from cst[cur[l]][l].
// Small layers take the resident-weight sequence kernel (see run_stack); it gathers its layer-0 inputs itself.
static bool stack_is_resident(const Geom& g, int B) {
  static const bool no_resident = std::getenv("ZRNN_NO_RESIDENT") != nullptr;
  return !no_resident && zrnn::lstm_seq_resident_supported(g.H, B);
}
static int run_stack(zrnn_model* m, const std::vector<zrnn_lstm_layer*>& layers, const Geom& g, const int* mask, int S,
                     int B, const Act& X0, const std::vector<Act>& h0, std::vector<Act>& seq, std::vector<float*> cst[2],
                     std::vector<int>& cur, cudaStream_t s, const int* ids0 = nullptr) {
  const int L = (int)layers.size();
  // Small layers: the recurrent weights fit the shared memory of one cluster, so a layer's S steps run as one launch
  // with the weights resident on chip (kernels.cu, lstm_seq_resident_kernel; exact fp32 arithmetic whatever the
  // engine).  ZRNN_NO_RESIDENT=1 keeps the per-step launches.
  if (ids0 && S >= 1 && stack_is_resident(g, B)) {
    ZR_CUDA(m->seq_xp.reserve(sizeof(float) * 4 * (size_t)S * B * g.H));
    KScope sweep(KC_LSTM, s, S * L, true);
    for (int l = 0; l < L; ++l) {
      zrnn_lstm_layer* Ly = layers[l];
      zrnn::SeqArgs a;
      std::memset(&a, 0, sizeof(a));
      a.H = g.H; a.B = B; a.S = S;
      a.Mx = Ly->Mx; a.Wh = Ly->Wh; a.bias = Ly->b;
      a.err = tc_error_word();
      if (l == 0) { a.emb = Ly->W; a.ids = ids0; a.V = Ly->V; }
      else a.x_seq = seq[l - 1].f32;
      a.mask = mask;
      a.h0 = h0[l].f32;
      const int cu = cur[l];
      a.c0 = cst[cu][l];
      a.c_out = cst[cu ^ 1][l];
      cur[l] = cu ^ 1;
      a.h_seq = seq[l].f32;
      a.xp = m->seq_xp.as<float>();
      a.ld_op = g.Kpad;
      if (g.eng == ENG_BF16) a.op_b16 = seq[l].hi;
      else if (g.eng == ENG_H2) { a.op_h_hi = seq[l].hi; a.op_h_lo = seq[l].lo; }
      else if (g.eng != ENG_SIMT) { a.op_hi = (float*)seq[l].hi; a.op_lo = g.eng == ENG_X3 ? seq[l].lo : nullptr; }
      ZR_CUDA(zrnn::launch_lstm_seq_resident(a, s));
    }
    return ZRNN_OK;
  }
  // Anti-diagonal order: the cells (layer l, step d - l) of diagonal d depend only on diagonal d - 1, so one launch
  // runs them side by side.  L cells fill the SMs with less (or no) K splitting than one cell alone: each CTA streams a
  // longer K slice, no partial tiles cross the cluster, and S + L - 1 launches replace S * L.  Needs one column tile
  // per cell, the tensor-core engine, and all L cells' row tiles resident at once.
  static const bool by_layers = [] {
    const char* e = std::getenv("ZRNN_ENCODER_ORDER");
    return e && std::string(e) == "layers";
  }();
  const zrnn_lstm_layer* L0 = layers[0];
  int dsplit = 0;
  // Not for 3xTF32: its tf32 MMAs cover 8 k-values each, so an unsplit K = 2H chain puts twice as many truncating
  // additions into one accumulator as the fp16 split does (measured at H = 1000, 4 layers: per-token log-prob error
  // 9e-6 against 4e-6), too close to the 1e-5 this engine promises.
  if (!by_layers && L >= 2 && L <= zrnn::TcMulti::MAX && L0->eng != ENG_SIMT && L0->eng != ENG_X3 && B <= 128 &&
      L0->BN == 128)
    for (int k = 4; k >= 1 && !dsplit; k >>= 1)
      if (L * L0->n_tiles * k <= 148) dsplit = k;
  if (dsplit && std::getenv("ZRNN_DIAG_SPLITK")) {  // developer knob: 1, 2 or 4 (more CTAs than SMs run in waves)
    const int k = std::atoi(std::getenv("ZRNN_DIAG_SPLITK"));
    if (k == 1 || k == 2 || k == 4) dsplit = k;
  }
  if (dsplit) {
    KScope sweep(KC_LSTM, s, S * L, true);
    zrnn::TcMulti* pm = &m->enc_multi;
    for (int d = 0; d < S + L - 1; ++d) {
      int n = 0;
      for (int l = std::max(0, d - S + 1); l <= std::min(L - 1, d); ++l) {
        const int t = d - l;
        const Act x = l == 0 ? act_at(X0, (size_t)t * B, g) : act_at(seq[l - 1], (size_t)t * B, g);
        const Act hp = t == 0 ? h0[l] : act_at(seq[l], (size_t)(t - 1) * B, g);
        const Act out = act_at(seq[l], (size_t)t * B, g);
        const int cu = cur[l];
        ZR_TRY(cell_params(layers[l], x, hp, nullptr, mask + (size_t)t * B, cst[cu][l], B, out, cst[cu ^ 1][l], pm->p[n]));
        cur[l] = cu ^ 1;
        ++n;
      }
      ZR_CUDA(zrnn::launch_tc_lstm_multi(*pm, n, eng_tcmode(L0->eng), s, dsplit));
    }
    return ZRNN_OK;
  }
  // Layer by layer, not step by step: layer l only needs layer l-1's finished sequence, and running all S steps
  // of one layer back to back keeps that layer's weights resident in the 126 MB L2 (all layers together do not fit).
  for (int l = 0; l < L; ++l) {
    KScope sweep(KC_LSTM, s, S, true);
    for (int t = 0; t < S; ++t) {
      const Act x = l == 0 ? act_at(X0, (size_t)t * B, g) : act_at(seq[l - 1], (size_t)t * B, g);
      const Act hp = t == 0 ? h0[l] : act_at(seq[l], (size_t)(t - 1) * B, g);
      const Act out = act_at(seq[l], (size_t)t * B, g);
      const int cu = cur[l];
      ZR_TRY(cell_forward(layers[l], x, hp, nullptr, mask + (size_t)t * B, cst[cu][l], B, out, cst[cu ^ 1][l], s));
      cur[l] = cu ^ 1;
    }
  }
  return ZRNN_OK;
}
static int run_encoder(zrnn_model* m, const Geom& g, const int* ids, const int* mask, int S, int B, const Act& X0,
                       const Act& zero, std::vector<Act>& seq, std::vector<float*> cst[2], std::vector<int>& cur,
                       cudaStream_t s) {
  if (!stack_is_resident(g, B)) ZR_TRY(gather_act(m->src[0], ids, S * B, X0, s));
  const std::vector<Act> h0(m->cfg.num_layers, zero);
  return run_stack(m, m->src, g, mask, S, B, X0, h0, seq, cst, cur, s, ids);
}

// The target side of a feed-input model as ONE launch of the persistent decoder kernel (tc_decoder.cu) instead of
// L + 2 (or 3) launches per time step.  Opt-in (environment ZRNN_PERSISTENT=1, read at every call): on the shapes
// measured so far the per-launch path, replayed as a CUDA graph with programmatic dependent launch, is as fast or
// faster - a phase of the persistent kernel pays for its grid-wide hand-over and keeps fewer bytes in flight per SM
// (its exchange slots cannot alias the operand ring) - so that path stays the default.  *done stays false when the
// kernel is off or the shape, the engine or the device cannot run it (the caller then takes the per-launch path).
static int run_decoder_persistent(zrnn_model* m, const Geom& g, int S, int T, int B, const Act& Xt,
                                  const std::vector<Act>& sseq, const std::vector<Act>& tseq, const Act& hts,
                                  const int* tin_mk, const int* len, const int* off, std::vector<float*> cst[2],
                                  std::vector<int>& cur, cudaStream_t s, bool* done) {
  *done = false;
  const char* want = std::getenv("ZRNN_PERSISTENT");
  const bool disabled = !(want && want[0] == '1');
  const zrnn_model_config& c = m->cfg;
  const int L = c.num_layers, H = c.H, eng = m->eng;
  zrnn_attention* A = m->att;
  if (disabled || m->persist_state < 0 || eng == ENG_SIMT || !A || c.lm || !c.feed_input) return ZRNN_OK;
  if (A->BN != 128 || A->eng != eng) return ZRNN_OK;
  for (int l = 0; l < L; ++l)
    if (m->tgt[l]->BN != 128 || m->tgt[l]->eng != eng) return ZRNN_OK;
  if (!zrnn::tc_decoder_supported(eng_tcmode(eng), H, B, L, c.attention)) return ZRNN_OK;
  const int eb = eng_eb(eng), epk = 128 / eb, Kpad = g.Kpad;
  const size_t nT = (size_t)T * B;
  zrnn::DecParams p;
  std::memset(&p, 0, sizeof(p));
  p.H = H; p.Kpad = Kpad; p.B = B; p.T = T; p.L = L; p.att_type = c.attention; p.D = A->D;
  p.kb = (H + epk - 1) / epk;
  p.kpb = Kpad / epk;
  p.groups = zrnn::tc_decoder_default_groups(B);
  const int ar = std::min(128, ((B + p.groups - 1) / p.groups + 7) / 8 * 8);
  p.a_rows = ar;
  ZR_TRY(act_maps(Xt, eng, H, Kpad, (int)nT, &p.x_hi, &p.x_lo, ar));
  for (int l = 0; l < L; ++l) {
    zrnn_lstm_layer* Ly = m->tgt[l];
    ZR_TRY(act_maps(tseq[l], eng, H, Kpad, (int)nT, &p.h_hi[l], &p.h_lo[l], ar));
    ZR_TRY(act_maps(sseq[l], eng, H, Kpad, S * B, &p.h0_hi[l], &p.h0_lo[l], ar));
    p.h0_row[l] = (S - 1) * B;
    p.w_hi[l] = Ly->wmap; p.w_lo[l] = Ly->wmap_lo; p.w_tiled[l] = Ly->kbtot;
    p.bias[l] = Ly->b;
    p.c_buf[l][0] = cst[cur[l]][l];
    p.c_buf[l][1] = cst[cur[l] ^ 1][l];
    p.h_f32[l] = tseq[l].f32; p.h_op_hi[l] = tseq[l].hi; p.h_op_lo[l] = tseq[l].lo;
  }
  ZR_TRY(act_maps(hts, eng, H, Kpad, (int)nT, &p.ht_hi, &p.ht_lo, ar));
  p.ht_f32 = hts.f32; p.ht_op_hi = hts.hi; p.ht_op_lo = hts.lo;
  // the step's context vectors and (local-p) the stacked projection live in the attention layer's own buffers
  ZR_CUDA(A->ctx.reserve(sizeof(float) * (size_t)H * B));
  ZR_CUDA(A->ctx_hi.reserve((size_t)B * Kpad * eb));
  if (eng_split(eng)) ZR_CUDA(A->ctx_lo.reserve((size_t)B * Kpad * eb));
  Act ctx;
  ctx.f32 = A->ctx.as<float>(); ctx.hi = A->ctx_hi.p; ctx.lo = eng_split(eng) ? A->ctx_lo.as<float>() : nullptr;
  ZR_TRY(act_maps(ctx, eng, H, Kpad, B, &p.ctx_hi, &p.ctx_lo, ar));
  p.ctx_f32 = ctx.f32; p.ctx_op_hi = ctx.hi; p.ctx_op_lo = ctx.lo;
  p.wc_hi = A->cmap; p.wc_lo = A->cmap_lo;
  if (c.attention == ZRNN_ATT_LOCAL_P) {
    ZR_CUDA(A->tq.reserve(sizeof(float) * (size_t)2 * H * B));
    p.tq = A->tq.as<float>();
    p.wp_hi = A->pmap; p.wp_lo = A->pmap_lo;
    p.v_p = A->v_p;
  }
  p.att_bias = A->bias;
  p.mask = tin_mk;
  p.hs = sseq[L - 1].f32; p.S_max = S; p.len = len; p.off = off;
  ZR_CUDA(m->dec_counter.reserve(1024));  // one counter per column group, 128 bytes apart
  p.counter = m->dec_counter.as<unsigned int>();
  p.err = tc_error_word();
  const int P = zrnn::dec_phases_per_step(p);
  if (g_kt.on) {
    long long* st = nullptr;
    ZR_CUDA(cudaMalloc((void**)&st, sizeof(long long) * ((size_t)T * P + 1)));
    ZR_CUDA(cudaMemsetAsync(st, 0, sizeof(long long) * ((size_t)T * P + 1), s));
    g_kt.dec_runs.push_back({st, T, P, L});
    p.stamps = st;
  }
  p.detail = g_dec_detail;
  p.hold_loads = std::getenv("ZRNN_DEC_NO_HOLD") == nullptr;
  p.w_evict_first = std::getenv("ZRNN_DEC_NO_EVICT") == nullptr;
  p.detail_cta = g_dec_detail_cta;
  ZR_CUDA(cudaMemsetAsync(p.counter, 0, 1024, s));
  const cudaError_t e = zrnn::launch_tc_decoder(p, eng_tcmode(eng), s);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    if (m->persist_state == 0) {  // first attempt refused (e.g. the CTAs cannot be co-resident): remember and fall back
      m->persist_state = -1;
      return ZRNN_OK;
    }
    return fail(ZRNN_E_CUDA, std::string("persistent decoder launch: ") + cudaGetErrorString(e));
  }
  m->persist_state = 1;
  for (int l = 0; l < L; ++l) cur[l] ^= (T & 1);
  *done = true;
  return ZRNN_OK;
}

// d_logp_out == nullptr: stop after the recurrent stack (the top-layer vectors stay in m->last_top)
static int score_batch_body(zrnn_model* m, const int* d_src_ids, int S_max, const int* d_tgt_in, const int* d_tgt_out,
                            int T, int B, float* d_logp_out, cudaStream_t s);

int zrnn_score_batch_device(zrnn_model* m, const int* d_src_ids, int S_max, const int* d_tgt_in,
                            const int* d_tgt_out, int T, int B, float* d_logp_out, void* stream) {
  ZR_CHECK(m && d_tgt_in && d_tgt_out && d_logp_out, "score_batch: null argument");
  if (!m->finalized) return fail(ZRNN_E_STATE, "score_batch: model weights not finalized");
  ZR_CHECK(!m->sharded, "score_batch: the model's softmax is vocabulary-sharded; use zrnn_score_batch_sharded");
  ZR_CHECK(T >= 0 && B >= 0, "score_batch: negative size");
  ZR_CHECK(m->cfg.lm || (d_src_ids && S_max > 0), "score_batch: a sequence-to-sequence model needs source ids");
  if (T == 0 || B == 0) return ZRNN_OK;
  cudaStream_t s = (cudaStream_t)stream;
  // The pass is a fixed sequence of ~10 launches per time step with no host decisions inside, so the second call
  // with the same shapes and buffers is captured into a CUDA graph and later calls replay it (launch cost and
  // tensor-map encoding disappear from the step).  The legacy default stream cannot be captured; kernel timing
  // needs eager launches; ZRNN_NO_GRAPH=1 turns the graph off.
  static const bool no_graph = std::getenv("ZRNN_NO_GRAPH") != nullptr;
  const bool can_graph = !no_graph && s != nullptr && !g_kt.on;
  auto& sg = m->sg;
  const char* pe = std::getenv("ZRNN_PERSISTENT");
  const int persistent = (pe && pe[0] == '1') ? 1 : 0;
  const bool same = sg.S == S_max && sg.T == T && sg.B == B && sg.src == d_src_ids && sg.tin == d_tgt_in &&
                    sg.tout == d_tgt_out && sg.out == d_logp_out && sg.stream == s && sg.ws == m->ws.p &&
                    sg.gen == g_buf_generation && sg.persistent == persistent;
  if (can_graph && same && sg.exec) {
    ZR_CUDA(cudaGraphLaunch(sg.exec, s));
    return ZRNN_OK;
  }
  if (!same) {
    m->drop_graph();
    sg.S = S_max; sg.T = T; sg.B = B; sg.src = d_src_ids; sg.tin = d_tgt_in; sg.tout = d_tgt_out; sg.out = d_logp_out;
    sg.stream = s;
    sg.persistent = persistent;
  }
  if (can_graph && same && sg.seen >= 1 && !sg.exec) {
    cudaGraph_t graph = nullptr;
    ZR_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    const int st = score_batch_body(m, d_src_ids, S_max, d_tgt_in, d_tgt_out, T, B, d_logp_out, s);
    const cudaError_t ce = cudaStreamEndCapture(s, &graph);
    if (st != ZRNN_OK) {
      if (graph) cudaGraphDestroy(graph);
      return st;
    }
    ZR_CUDA(ce);
    cudaError_t ie = cudaGraphInstantiate(&sg.exec, graph, 0);
    cudaGraphDestroy(graph);
    ZR_CUDA(ie);
    ZR_CUDA(cudaGraphLaunch(sg.exec, s));
    return ZRNN_OK;
  }
  const int st = score_batch_body(m, d_src_ids, S_max, d_tgt_in, d_tgt_out, T, B, d_logp_out, s);
  sg.ws = m->ws.p;  // the eager pass has grown every buffer the pass needs
  sg.gen = g_buf_generation;
  sg.seen += 1;
  return st;
}

static int score_batch_body(zrnn_model* m, const int* d_src_ids, int S_max, const int* d_tgt_in, const int* d_tgt_out,
                            int T, int B, float* d_logp_out, cudaStream_t s) {
  const zrnn_model_config& c = m->cfg;
  const int H = c.H, L = c.num_layers;
  const Geom g{H, round64(H), m->eng};
  const bool tc = m->eng != ENG_SIMT;
  const size_t HB = (size_t)H * B;
  const int S = c.lm ? 0 : S_max;
  const size_t nS = (size_t)S * B, nT = (size_t)T * B;
  // ---- workspace
  size_t bytes = 2 * aligned(sizeof(int) * (nS + 1)) + 4 * aligned(sizeof(int) * nT) + 2 * aligned(sizeof(int) * B);
  bytes += act_bytes(g, nS + 1, !tc, true) + act_bytes(g, nT, !tc, true);          // gathered inputs
  bytes += (size_t)L * (act_bytes(g, nS + 1, true, true) + act_bytes(g, nT, true, true));  // per-layer h sequences
  bytes += act_bytes(g, nT, true, true) + act_bytes(g, B, true, true);            // htild sequence, zero state
  bytes += 2 * (size_t)L * aligned(sizeof(float) * HB);
  ZR_CUDA(m->ws.reserve(bytes));
  Carver cv(m->ws.p);
  int* src_id = cv.take<int>(nS + 1);
  int* src_mk = cv.take<int>(nS + 1);
  int* tin_id = cv.take<int>(nT);
  int* tin_mk = cv.take<int>(nT);
  int* tout_id = cv.take<int>(nT);
  int* tout_mk = cv.take<int>(nT);
  int* len = cv.take<int>(B);
  int* off = cv.take<int>(B);
  const Act X0 = act_take(cv, g, nS + 1, !tc, true);
  const Act Xt = act_take(cv, g, nT, !tc, true);
  std::vector<Act> sseq(L), tseq(L);
  for (int l = 0; l < L; ++l) { sseq[l] = act_take(cv, g, nS + 1, true, true); tseq[l] = act_take(cv, g, nT, true, true); }
  const Act hts = act_take(cv, g, nT, true, true);
  const Act zero = act_take(cv, g, B, true, true);
  std::vector<float*> cst[2];
  for (int k = 0; k < 2; ++k) { cst[k].resize(L); for (int l = 0; l < L; ++l) cst[k][l] = cv.take<float>(HB); }
  std::vector<int> cur(L, 0);
  {
    // one launch: the three id preparations and the zero fills of the start states
    zrnn::PrologueArgs pa;
    std::memset(&pa, 0, sizeof(pa));
    pa.raw[0] = d_tgt_in; pa.n[0] = (int)nT; pa.ids[0] = tin_id; pa.mask[0] = tin_mk;
    pa.raw[1] = d_tgt_out; pa.n[1] = (int)nT; pa.ids[1] = tout_id; pa.mask[1] = tout_mk;
    if (!c.lm) { pa.raw[2] = d_src_ids; pa.n[2] = (int)nS; pa.ids[2] = src_id; pa.mask[2] = src_mk; }
    auto zero_fill = [&](void* p, size_t bytes) {
      if (p && bytes) { pa.zero_ptr[pa.n_zero] = p; pa.zero_bytes[pa.n_zero] = bytes; ++pa.n_zero; }
    };
    zero_fill(zero.f32, sizeof(float) * B * g.H);
    zero_fill(zero.hi, (size_t)B * g.Kpad * eng_eb(g.eng));
    zero_fill(zero.lo, (size_t)B * g.Kpad * eng_eb(g.eng));
    for (int l = 0; l < L; ++l) zero_fill(cst[0][l], sizeof(float) * HB);
    ZR_CUDA(zrnn::launch_score_prologue(pa, s));
  }
  if (!c.lm) {
    ZR_CUDA(zrnn::launch_src_len(src_mk, S, B, len, off, s));
    ZR_TRY(run_encoder(m, g, src_id, src_mk, S, B, X0, zero, sseq, cst, cur, s));
    if (c.attention) ZR_TRY(zrnn_att_set_source(m->att, sseq[L - 1].f32, S, B, len, off, 1));
  }
  // target side: layer l starts from the encoder's final (h,c) of layer l (src/model.hpp:1714-1724)
  if (c.feed_input || !stack_is_resident(g, B)) ZR_TRY(gather_act(m->tgt[0], tin_id, (int)nT, Xt, s));
  if (!c.feed_input) {
    // no cell waits for an attention output: the target side is a plain stack too (anti-diagonal order where it
    // fits), and attention follows per step on the finished top layer
    std::vector<Act> h0(L);
    for (int l = 0; l < L; ++l) h0[l] = c.lm ? zero : act_at(sseq[l], (size_t)(S - 1) * B, g);
    ZR_TRY(run_stack(m, m->tgt, g, tin_mk, T, B, Xt, h0, tseq, cst, cur, s, tin_id));
    if (c.attention)
      for (int t = 0; t < T; ++t)
        ZR_TRY(att_forward(m->att, act_at(tseq[L - 1], (size_t)t * B, g), tin_mk + (size_t)t * B, B,
                           act_at(hts, (size_t)t * B, g), nullptr, s));
  } else {
    // feed-input: layer 0 of step t reads the attention output of step t - 1, so the steps form one chain
    bool done = false;
    ZR_TRY(run_decoder_persistent(m, g, S, T, B, Xt, sseq, tseq, hts, tin_mk, len, off, cst, cur, s, &done));
    for (int t = 0; t < T && !done; ++t) {
      Act x = act_at(Xt, (size_t)t * B, g);
      const int* mk = tin_mk + (size_t)t * B;
      for (int l = 0; l < L; ++l) {
        Act hp = t > 0 ? act_at(tseq[l], (size_t)(t - 1) * B, g) : (c.lm ? zero : act_at(sseq[l], (size_t)(S - 1) * B, g));
        const Act out = act_at(tseq[l], (size_t)t * B, g);
        const Act feed = act_at(hts, (size_t)(t > 0 ? t - 1 : 0) * B, g);
        const bool use_feed = (l == 0 && t > 0);
        const int cu = cur[l];
        ZR_TRY(cell_forward(m->tgt[l], x, hp, use_feed ? &feed : nullptr, mk, cst[cu][l], B, out, cst[cu ^ 1][l], s));
        cur[l] = cu ^ 1;
        x = out;
      }
      if (c.attention) ZR_TRY(att_forward(m->att, x, mk, B, act_at(hts, (size_t)t * B, g), nullptr, s));
    }
  }
  const Act& top = c.attention ? hts : tseq[L - 1];
  m->last_top = top.f32;
  m->last_top_act = top;
  m->last_top_cols = (int)nT;
  if (!d_logp_out) return ZRNN_OK;
  return softmax_score_act(m->sm, top, tout_id, tout_mk, (int)nT, d_logp_out, s);
}

int zrnn_forward_states_device(zrnn_model* m, const int* d_src_ids, int S_max, const int* d_tgt_in, int T, int B,
                               float* d_top_out, void* stream) {
  ZR_CHECK(m && d_tgt_in && d_top_out, "forward_states: null argument");
  if (!m->finalized) return fail(ZRNN_E_STATE, "forward_states: model weights not finalized");
  ZR_CHECK(T >= 0 && B >= 0, "forward_states: negative size");
  ZR_CHECK(m->cfg.lm || (d_src_ids && S_max > 0), "forward_states: a sequence-to-sequence model needs source ids");
  if (T == 0 || B == 0) return ZRNN_OK;
  cudaStream_t s = (cudaStream_t)stream;
  m->drop_graph();
  // the target-output ids only feed the softmax, which is skipped: reuse the inputs as a placeholder
  ZR_TRY(score_batch_body(m, d_src_ids, S_max, d_tgt_in, d_tgt_in, T, B, nullptr, s));
  ZR_CUDA(cudaMemcpyAsync(d_top_out, m->last_top, sizeof(float) * (size_t)T * B * m->cfg.H, cudaMemcpyDeviceToDevice, s));
  return ZRNN_OK;
}

int zrnn_score_batch(zrnn_model* m, const int* src_ids, int S_max, const int* tgt_in, const int* tgt_out, int T,
                     int B, float* logp_out, double* total_logp) {
  ZR_CHECK(m && tgt_in && tgt_out && logp_out, "score_batch: null argument");
  ZR_CHECK(T >= 0 && B >= 0 && S_max >= 0, "score_batch: negative size");
  if (total_logp) *total_logp = 0.0;
  if (T == 0 || B == 0) return ZRNN_OK;
  const size_t nS = m->cfg.lm ? 0 : (size_t)S_max * B, nT = (size_t)T * B;
  ZR_CHECK(m->cfg.lm || src_ids, "score_batch: a sequence-to-sequence model needs source ids");
  if (nS) ZR_TRY(check_ids(src_ids, nS, m->cfg.V_src, "score_batch (source)"));
  ZR_TRY(check_ids(tgt_in, nT, m->cfg.V_tgt, "score_batch (target input)"));
  ZR_TRY(check_ids(tgt_out, nT, m->cfg.V_tgt, "score_batch (target output)"));
  ZR_CUDA(m->io.reserve(aligned(sizeof(int) * (nS + 1)) + 2 * aligned(sizeof(int) * nT) + aligned(sizeof(float) * nT)));
  Carver cv(m->io.p);
  int* d_src = cv.take<int>(nS + 1);
  int* d_tin = cv.take<int>(nT);
  int* d_tout = cv.take<int>(nT);
  float* d_lp = cv.take<float>(nT);
  cudaStream_t s = m->stream;
  if (nS) ZR_CUDA(cudaMemcpyAsync(d_src, src_ids, sizeof(int) * nS, cudaMemcpyHostToDevice, s));
  ZR_CUDA(cudaMemcpyAsync(d_tin, tgt_in, sizeof(int) * nT, cudaMemcpyHostToDevice, s));
  ZR_CUDA(cudaMemcpyAsync(d_tout, tgt_out, sizeof(int) * nT, cudaMemcpyHostToDevice, s));
  ZR_TRY(zrnn_score_batch_device(m, nS ? d_src : nullptr, S_max, d_tin, d_tout, T, B, d_lp, s));
  ZR_CUDA(cudaMemcpyAsync(logp_out, d_lp, sizeof(float) * nT, cudaMemcpyDeviceToHost, s));
  ZR_CUDA(cudaStreamSynchronize(s));
  ZR_TRY(device_error_status("score_batch"));
  if (total_logp) {
    double tot = 0;
    for (size_t i = 0; i < nT; ++i) tot += logp_out[i];
    *total_logp = tot;
  }
  return ZRNN_OK;
}

// ---------------------------------------------------------------- beam decoding driver
int zrnn_beam_decode_batch_device(zrnn_model* m, const int* d_src, const int* h_src_len, int S_max, int n_sent,
                                  int beam, int k_best, float min_ratio, float max_ratio, float penalty,
                                  int longest_sent, int* d_out_ids, int* d_out_len, float* d_out_score,
                                  void* stream) {
  return zrnn_beam_decode_batch_align_device(m, d_src, h_src_len, S_max, n_sent, beam, k_best, min_ratio, max_ratio,
                                             penalty, longest_sent, d_out_ids, d_out_len, d_out_score, nullptr, stream);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// collective layer: NCCL, loaded at first use (the library has no link-time dependency on it)
// ------------------------------------------------------------------------------------------
struct zrnn_comm {
  ncclComm_t comm = nullptr;
  bool owned = true;  // false: the communicator belongs to the host (zrnn_comm_from_nccl)
  int rank = 0, world = 1;
  DevBuf send, recv, aux, lo_buf;  // staging for the all-gathers; first vocabulary row of every rank
  int lo_V = -1;                   // vocabulary size lo_buf was computed for
  cudaEvent_t ev[6] = {};          // stage boundaries of the last sharded scoring call
  float stage_ms[5] = {};
  void* pin = nullptr;             // page-locked host staging for the ids going in and the log-probabilities coming out
  size_t pin_cap = 0;
  cudaError_t pin_reserve(size_t bytes) {
    if (bytes <= pin_cap) return cudaSuccess;
    if (pin) cudaFreeHost(pin);
    pin = nullptr;
    pin_cap = 0;
    cudaError_t e = cudaHostAlloc(&pin, bytes, cudaHostAllocDefault);
    if (e == cudaSuccess) pin_cap = bytes;
    return e;
  }
  ~zrnn_comm() {
    send.release(); recv.release(); aux.release(); lo_buf.release();
    for (auto& e : ev) if (e) cudaEventDestroy(e);
    if (pin) cudaFreeHost(pin);
  }
};

namespace {
struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};
NcclApi* nccl_api() {
  static NcclApi api;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (h) {
      api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
      api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
      api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
      api.AllGather = (decltype(api.AllGather))dlsym(h, "ncclAllGather");
      api.GroupStart = (decltype(api.GroupStart))dlsym(h, "ncclGroupStart");
      api.GroupEnd = (decltype(api.GroupEnd))dlsym(h, "ncclGroupEnd");
      api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
      api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.GroupStart && api.GroupEnd &&
               api.GetErrorString;
    }
  }
  return &api;
}
#define ZR_NCCL(expr)                                                                                    \
  do {                                                                                                   \
    ncclResult_t _r = (expr);                                                                            \
    if (_r != ncclSuccess) return fail(ZRNN_E_NCCL, std::string(#expr) + ": " + nccl_api()->GetErrorString(_r)); \
  } while (0)

// all-gather of `bytes` bytes per rank (device buffers; recv holds world * bytes, rank-major)
int comm_all_gather(zrnn_comm* c, const void* send, void* recv, size_t bytes, cudaStream_t s) {
  if (c->world == 1) {
    if (send != recv) ZR_CUDA(cudaMemcpyAsync(recv, send, bytes, cudaMemcpyDeviceToDevice, s));
    return ZRNN_OK;
  }
  ZR_NCCL(nccl_api()->AllGather(send, recv, bytes, ncclChar, c->comm, s));
  return ZRNN_OK;
}


// first vocabulary row of every rank's shard, on the device (cached per vocabulary size)
int comm_shard_lo(zrnn_comm* c, int V, const int** d_lo) {
  if (c->lo_V != V) {
    std::vector<int> lo(c->world);
    int hi_unused;
    for (int g = 0; g < c->world; ++g) shard_range(V, c->world, g, &lo[g], &hi_unused);
    ZR_CUDA(c->lo_buf.reserve(sizeof(int) * c->world));
    ZR_CUDA(cudaMemcpy(c->lo_buf.p, lo.data(), sizeof(int) * c->world, cudaMemcpyHostToDevice));
    c->lo_V = V;
  }
  *d_lo = c->lo_buf.as<int>();
  return ZRNN_OK;
}

// Vocabulary-sharded pre-selection: this rank's k best rows and normaliser, ONE all-gather of k (value, row) pairs and
// two floats per column, and the merge under the global normaliser, which reads the receive buffer in place.  Every
// rank ends up with the same k candidates.
int softmax_topk_sharded_act(zrnn_softmax* S, zrnn_comm* c, const Act& h, int N, int k, float* logp, int* idx, float* eos,
                             cudaStream_t st) {
  const int G = c->world;
  int lo, hi;
  shard_range(S->V, G, c->rank, &lo, &hi);
  ZR_CHECK(S->lo == lo && S->hi == hi, "softmax_topk_sharded: the layer's vocabulary range is not this rank's share");
  // per rank: [N*k val][N*k idx][N lse][N eos] as 4-byte words
  const size_t words = (size_t)N * (2 * k + 2);
  ZR_CUDA(c->send.reserve(words * 4));
  ZR_CUDA(c->recv.reserve(words * 4 * G));
  const int* d_lo = nullptr;
  ZR_TRY(comm_shard_lo(c, S->V, &d_lo));
  float* sv = c->send.as<float>();
  int* si = (int*)(sv + (size_t)N * k);
  float* sl = sv + 2 * (size_t)N * k;
  float* se = sl + N;
  ZR_TRY(softmax_topk_act(S, h, N, k, sv, si, se, st, sl));
  ZR_TRY(comm_all_gather(c, c->send.p, c->recv.p, words * 4, st));
  const float* rv = c->recv.as<float>();
  KScope ks(KC_SOFTMAX_REDUCE, st);
  ZR_CUDA(zrnn::launch_topk_merge(rv, (const int*)(rv + (size_t)N * k), rv + 2 * (size_t)N * k, rv + 2 * (size_t)N * k + N, d_lo,
                                  G, N, k, logp, idx, eos, st, words, words));
  return ZRNN_OK;
}
}  // namespace

namespace {
// Per-model state of a (possibly ensembled) beam search: encoder outputs and the decoder's recurrent state for
// n_sent * beam columns.  Everything lives in the model's own workspace.
struct BeamModel {
  zrnn_model* m = nullptr;
  Geom g{0, 0, 0};
  bool tc = false;
  int S_max = 0, n = 0, NB = 0, beam = 0;
  int *src_id = nullptr, *src_mk = nullptr, *len = nullptr, *off = nullptr, *rep_map = nullptr;
  Act X0, zero, x, htild_new, htild_feed;
  std::vector<Act> sseq, hp, hn;
  std::vector<float*> cst[2], cp, cn;
  std::vector<int> cur;
  int* vit = nullptr;  // viterbi alignment per column of the last forward step (tracking on)
  float* align_pos = nullptr;  // ensemble tracking: attention weights by source position, S_max x NB

  size_t bytes(bool track, bool vote = false) const {
    const zrnn_model_config& c = m->cfg;
    const int H = c.H, L = c.num_layers;
    const size_t HBs = (size_t)H * n, HB = (size_t)H * NB, nS = (size_t)S_max * n;
    size_t b = 2 * aligned(sizeof(int) * nS) + 2 * aligned(sizeof(int) * n) + aligned(sizeof(int) * NB);
    b += act_bytes(g, nS, !tc, true) + (size_t)L * act_bytes(g, nS, true, true) + act_bytes(g, n, true, true);
    b += 2 * (size_t)L * aligned(sizeof(float) * HBs);
    b += (2 * (size_t)L + 3) * act_bytes(g, NB, true, true) + 2 * (size_t)L * aligned(sizeof(float) * HB);
    if (track) b += aligned(sizeof(int) * NB);
    if (vote) b += aligned(sizeof(float) * (size_t)S_max * NB);
    return b;
  }
  void carve(Carver& cv, bool track, bool vote = false) {
    const zrnn_model_config& c = m->cfg;
    const int H = c.H, L = c.num_layers;
    const size_t HBs = (size_t)H * n, HB = (size_t)H * NB, nS = (size_t)S_max * n;
    src_id = cv.take<int>(nS);
    src_mk = cv.take<int>(nS);
    len = cv.take<int>(n);
    off = cv.take<int>(n);
    rep_map = cv.take<int>(NB);
    X0 = act_take(cv, g, nS, !tc, true);
    sseq.resize(L);
    for (int l = 0; l < L; ++l) sseq[l] = act_take(cv, g, nS, true, true);
    zero = act_take(cv, g, n, true, true);
    for (int k = 0; k < 2; ++k) { cst[k].resize(L); for (int l = 0; l < L; ++l) cst[k][l] = cv.take<float>(HBs); }
    hp.resize(L); hn.resize(L); cp.resize(L); cn.resize(L);
    for (int l = 0; l < L; ++l) {
      hp[l] = act_take(cv, g, NB, true, true);
      hn[l] = act_take(cv, g, NB, true, true);
      cp[l] = cv.take<float>(HB);
      cn[l] = cv.take<float>(HB);
    }
    x = act_take(cv, g, NB, true, true);
    htild_new = act_take(cv, g, NB, true, true);
    htild_feed = act_take(cv, g, NB, true, true);
    vit = track ? cv.take<int>(NB) : nullptr;
    align_pos = vote ? cv.take<float>((size_t)S_max * NB) : nullptr;
  }
  // column gathers move whole operand rows: every array is expressed as floats-per-column, and all arrays of a
  // reorder go into one launch
  void add_plain(zrnn::ColGatherArgs* ga, const float* src, float* dst, int floats_per_col) const {
    const int i = ga->n_arrays++;
    ga->src[i] = src; ga->dst[i] = dst; ga->h_arr[i] = floats_per_col;
  }
  void add_gather(zrnn::ColGatherArgs* ga, const Act& srcA, const Act& dstA) const {
    add_plain(ga, srcA.f32, dstA.f32, g.H);
    if (tc) {
      const int opf = g.Kpad * eng_eb(g.eng) / 4;
      add_plain(ga, (const float*)srcA.hi, (float*)dstA.hi, opf);
      if (eng_split(g.eng)) add_plain(ga, (const float*)srcA.lo, (float*)dstA.lo, opf);
    }
  }
  int run_gathers(zrnn::ColGatherArgs* ga, const int* map, cudaStream_t s) const {
    if (ga->n_arrays == 0) return ZRNN_OK;
    ga->H = g.H; ga->n_cols = NB; ga->map = map;
    KScope ks(KC_REORDER, s);
    ZR_CUDA(zrnn::launch_col_gather(*ga, s));
    return ZRNN_OK;
  }
  // forward_prop_source + transfer_decoding_states_GPU (src/model.hpp:2367-2452)
  int encode(const int* d_src, cudaStream_t s) {
    const zrnn_model_config& c = m->cfg;
    const int L = c.num_layers;
    const size_t HBs = (size_t)c.H * n, nS = (size_t)S_max * n;
    cur.assign(L, 0);
    ZR_TRY(act_zero(zero, g, n, s));
    for (int l = 0; l < L; ++l) ZR_CUDA(cudaMemsetAsync(cst[0][l], 0, sizeof(float) * HBs, s));
    ZR_CUDA(zrnn::launch_prep_ids(d_src, (int)nS, src_id, src_mk, s));
    ZR_CUDA(zrnn::launch_src_len(src_mk, S_max, n, len, off, s));
    ZR_TRY(run_encoder(m, g, src_id, src_mk, S_max, n, X0, zero, sseq, cst, cur, s));
    if (c.attention) ZR_TRY(zrnn_att_set_source(m->att, sseq[L - 1].f32, S_max, n, len, off, beam));
    if (vit) ZR_CUDA(cudaMemsetAsync(vit, 0xff, sizeof(int) * NB, s));  // -1 without attention (src/decoder.h:1174-1178)
    if (align_pos) ZR_CUDA(cudaMemsetAsync(align_pos, 0, sizeof(float) * (size_t)S_max * NB, s));  // no attention: no votes
    // replicate the encoder's final (h,c) over the beam
    ZR_CUDA(zrnn::launch_div_map(rep_map, NB, beam, s));
    zrnn::ColGatherArgs ga;
    std::memset(&ga, 0, sizeof(ga));
    for (int l = 0; l < L; ++l) {
      add_gather(&ga, act_at(sseq[l], (size_t)(S_max - 1) * n, g), hp[l]);
      add_plain(&ga, cst[cur[l]][l], cp[l], c.H);
    }
    return run_gathers(&ga, rep_map, s);
  }
  // forward_prop_target (src/model.hpp:2573-2689) up to the vector handed to the softmax
  int forward(int t, const int* cur_ids, Act* top, cudaStream_t s) {
    const zrnn_model_config& c = m->cfg;
    ZR_TRY(gather_act(m->tgt[0], cur_ids, NB, x, s));
    Act xin = x;
    for (int l = 0; l < c.num_layers; ++l) {
      const bool use_feed = (l == 0 && c.feed_input && t > 0);
      ZR_TRY(cell_forward(m->tgt[l], xin, hp[l], use_feed ? &htild_feed : nullptr, nullptr, cp[l], NB, hn[l], cn[l], s));
      xin = hn[l];
    }
    *top = xin;
    if (c.attention) {
      ZR_TRY(att_forward(m->att, xin, nullptr, NB, htild_new, align_pos, s, vit, 0.f, align_pos != nullptr));
      *top = htild_new;
    }
    return ZRNN_OK;
  }
  // swap_decoding_states + target_copy_prev_states (src/model.hpp:2691-2726)
  int reorder(const int* col_map, cudaStream_t s) {
    const zrnn_model_config& c = m->cfg;
    zrnn::ColGatherArgs ga;
    std::memset(&ga, 0, sizeof(ga));
    for (int l = 0; l < c.num_layers; ++l) {
      add_gather(&ga, hn[l], hp[l]);
      add_plain(&ga, cn[l], cp[l], c.H);
    }
    if (c.feed_input) add_gather(&ga, htild_new, htild_feed);
    return run_gathers(&ga, col_map, s);
  }
};

// Lock-step beam search of n_sent sentences with K >= 1 models.  With K > 1 the models' output distributions are
// averaged and renormalised at every step (ensemble_factory::ensembles_models, src/ensemble_factory.hpp:768-795);
// length limits follow model 0's source lengths (:623).  All models sit on the current device.
int beam_decode_core(zrnn_model* const* models, int K, const int* const* d_src, const int* h_src_len,
                     const int* S_max, int n_sent, int beam, int k_best, float min_ratio, float max_ratio, float penalty,
                     int longest_sent, int* d_out_ids, int* d_out_len, float* d_out_score, int* d_out_align,
                     cudaStream_t s, zrnn_comm* comm = nullptr) {
  ZR_CHECK(K >= 1 && K <= ZR_ENSEMBLE_MAX, "beam_decode: between 1 and 8 models");
  ZR_CHECK(!comm || K == 1, "beam_decode: vocabulary sharding is not combined with ensembles");
  const int V = models[0]->cfg.V_tgt;
  for (int k = 0; k < K; ++k) {
    zrnn_model* m = models[k];
    ZR_CHECK(m, "beam_decode: null model");
    if (!m->finalized) return fail(ZRNN_E_STATE, "beam_decode: model weights not finalized");
    ZR_CHECK(!m->cfg.lm, "beam_decode: needs a sequence-to-sequence model");
    ZR_CHECK(!m->sharded || comm, "beam_decode: the model's softmax is vocabulary-sharded; use zrnn_beam_decode_batch_sharded");
    ZR_CHECK(m->cfg.V_tgt == V, "beam_decode: ensembled models must share the target vocabulary");
    ZR_CHECK(S_max[k] > 0, "beam_decode: bad sizes");
  }
  ZR_CHECK(n_sent >= 0 && beam >= 1 && k_best >= 1 && longest_sent >= 1, "beam_decode: bad sizes");
  if (n_sent == 0) return ZRNN_OK;
  const int cap = (int)std::sqrt((double)V);  // src/ensemble_factory.hpp:19-21
  if (beam > cap) beam = cap;
  ZR_CHECK(beam >= 1 && beam <= ZR_BEAM_MAX, "beam_decode: beam must be in [1,32] after the sqrt(V) cap");
  const int kc = beam + 1;
  ZR_CHECK(kc <= V, "beam_decode: vocabulary smaller than beam+1");
  const int Lmax = longest_sent + 4;  // src/main.cu:408
  const int n = n_sent, NB = n_sent * beam;
  zrnn_model* m0 = models[0];

  // per-sentence step limits (src/ensemble_factory.hpp:637)
  m0->h_tmp.resize(2 * (size_t)n);
  int Tmax = 0;
  for (int i = 0; i < n; ++i) {
    ZR_CHECK(h_src_len[i] >= 1 && h_src_len[i] <= S_max[0], "beam_decode: source length out of range");
    int ms = std::min((int)(max_ratio * h_src_len[i]), Lmax - 2);
    ZR_CHECK(ms >= 1, "beam_decode: max_ratio*source_length must allow at least one step");
    m0->h_tmp[i] = h_src_len[i];
    m0->h_tmp[n + i] = ms;
    Tmax = std::max(Tmax, ms);
  }
  const bool track = d_out_align != nullptr;
  const bool vote = track && K > 1;  // alignment voting over the models of an ensemble
  std::vector<BeamModel> bm(K);
  for (int k = 0; k < K; ++k) {
    BeamModel& b = bm[k];
    b.m = models[k];
    b.g = Geom{models[k]->cfg.H, round64(models[k]->cfg.H), models[k]->eng};
    b.tc = models[k]->eng != ENG_SIMT;
    b.S_max = S_max[k]; b.n = n; b.NB = NB; b.beam = beam;
    size_t bytes = b.bytes(track && k == 0, vote);
    if (k == 0) {  // shared bookkeeping lives in model 0's workspace
      bytes += 2 * aligned(sizeof(int) * n) + 2 * aligned(sizeof(int) * NB) + 2 * aligned(sizeof(int) * (size_t)NB * Lmax);
      bytes += aligned(sizeof(int) * (size_t)NB * kc) + 2 * aligned(sizeof(float) * NB) + aligned(sizeof(float) * (size_t)NB * kc);
      if (track) bytes += 2 * aligned(sizeof(int) * (size_t)NB * Lmax);
      if (K > 1) bytes += aligned(sizeof(float) * (size_t)V * NB);
    }
    ZR_CUDA(models[k]->ws.reserve(bytes));
  }
  Carver cv0(m0->ws.p);
  int* d_len_host = cv0.take<int>(n);
  int* max_steps = cv0.take<int>(n);
  int* cur_ids = cv0.take<int>(NB);
  int* col_map = cv0.take<int>(NB);
  int* top_sent = cv0.take<int>((size_t)NB * Lmax);
  int* top_tmp = cv0.take<int>((size_t)NB * Lmax);
  int* cand_idx = cv0.take<int>((size_t)NB * kc);
  float* scores = cv0.take<float>(NB);
  float* logp_eos = cv0.take<float>(NB);
  float* cand_val = cv0.take<float>((size_t)NB * kc);
  int* vit_rows = track ? cv0.take<int>((size_t)NB * Lmax) : nullptr;
  int* vit_tmp = track ? cv0.take<int>((size_t)NB * Lmax) : nullptr;
  float* mean_logits = K > 1 ? cv0.take<float>((size_t)V * NB) : nullptr;
  bm[0].carve(cv0, track, vote);
  for (int k = 1; k < K; ++k) {
    Carver cv(models[k]->ws.p);
    bm[k].carve(cv, false, vote);
  }

  ZR_CUDA(cudaMemcpyAsync(d_len_host, m0->h_tmp.data(), sizeof(int) * n, cudaMemcpyHostToDevice, s));
  ZR_CUDA(cudaMemcpyAsync(max_steps, m0->h_tmp.data() + n, sizeof(int) * n, cudaMemcpyHostToDevice, s));
  for (int k = 0; k < K; ++k) ZR_TRY(bm[k].encode(d_src[k], s));

  zrnn::BeamArgs ba;
  std::memset(&ba, 0, sizeof(ba));
  ba.n_sent = n; ba.beam = beam; ba.k_cand = kc; ba.Lmax = Lmax; ba.k_best = k_best;
  ba.min_ratio = min_ratio; ba.penalty = penalty;
  ba.cand_val = cand_val; ba.cand_idx = cand_idx; ba.logp_eos = logp_eos; ba.src_len = d_len_host; ba.max_steps = max_steps;
  ba.top_sent = top_sent; ba.top_tmp = top_tmp; ba.scores = scores; ba.cur_ids = cur_ids; ba.col_map = col_map;
  ba.best_ids = d_out_ids; ba.best_len = d_out_len; ba.best_score = d_out_score;
  ba.viterbi = bm[0].vit; ba.vit_rows = vit_rows; ba.vit_tmp = vit_tmp; ba.best_align = d_out_align;
  ZR_CUDA(zrnn::launch_beam_init(ba, s));

  for (int t = 0; t <= Tmax; ++t) {
    if (K == 1) {
      Act top;
      ZR_TRY(bm[0].forward(t, cur_ids, &top, s));
      if (comm) ZR_TRY(softmax_topk_sharded_act(m0->sm, comm, top, NB, kc, cand_val, cand_idx, logp_eos, s));
      else ZR_TRY(softmax_topk_act(m0->sm, top, NB, kc, cand_val, cand_idx, logp_eos, s));
    } else {
      zrnn::EnsembleArgs ea;
      std::memset(&ea, 0, sizeof(ea));
      for (int k = 0; k < K; ++k) {
        Act top;
        ZR_TRY(bm[k].forward(t, cur_ids, &top, s));
        const float* pm = nullptr;
        int np = 0;
        ZR_TRY(softmax_logits_act(models[k]->sm, top, NB, s, &pm, &np));
        ea.logits[k] = models[k]->sm->logits.as<float>();
      }
      ea.K = K; ea.V = V; ea.N = NB; ea.out = mean_logits;
      if (vote) {  // ensembles_models: sum the models' weights per source position, take the largest
        zrnn::EnsembleVitArgs va;
        std::memset(&va, 0, sizeof(va));
        for (int k = 0; k < K; ++k) { va.align[k] = bm[k].align_pos; va.S_max[k] = bm[k].S_max; }
        va.K = K; va.N = NB; va.viterbi_out = bm[0].vit;
        ZR_CUDA(zrnn::launch_ensemble_viterbi(va, s));
      }
      KScope ks(KC_SOFTMAX_REDUCE, s);
      ZR_CUDA(zrnn::launch_ensemble_logmean(ea, s));
      ZR_CUDA(zrnn::launch_topk_logp(mean_logits, V, NB, kc, cand_val, cand_idx, logp_eos, s, nullptr, nullptr, 0));
    }
    ba.step = t;
    {
      KScope ks(KC_BEAM, s);
      ZR_CUDA(zrnn::launch_beam_step(ba, s));
      // the step wrote the surviving rows into the second row buffer: it is the current one from now on
      std::swap(ba.top_sent, ba.top_tmp);
      std::swap(ba.vit_rows, ba.vit_tmp);
    }
    if (t < Tmax)
      for (int k = 0; k < K; ++k) ZR_TRY(bm[k].reorder(col_map, s));
  }
  return ZRNN_OK;
}
}  // namespace

extern "C" {

int zrnn_beam_decode_batch_align_device(zrnn_model* m, const int* d_src, const int* h_src_len, int S_max, int n_sent,
                                        int beam, int k_best, float min_ratio, float max_ratio, float penalty,
                                        int longest_sent, int* d_out_ids, int* d_out_len, float* d_out_score,
                                        int* d_out_align, void* stream) {
  ZR_CHECK(m && d_src && h_src_len && d_out_ids && d_out_len && d_out_score, "beam_decode: null argument");
  return beam_decode_core(&m, 1, &d_src, h_src_len, &S_max, n_sent, beam, k_best, min_ratio, max_ratio, penalty,
                          longest_sent, d_out_ids, d_out_len, d_out_score, d_out_align, (cudaStream_t)stream);
}

int zrnn_beam_decode_batch(zrnn_model* m, const int* src_ids, const int* src_len, int n_sent, int beam, int k_best,
                           float min_ratio, float max_ratio, float penalty, int longest_sent, int* out_ids,
                           int* out_len, float* out_score) {
  return zrnn_beam_decode_batch_align(m, src_ids, src_len, n_sent, beam, k_best, min_ratio, max_ratio, penalty,
                                      longest_sent, out_ids, out_len, out_score, nullptr);
}

static int beam_decode_host(zrnn_model* m, zrnn_comm* comm, const int* src_ids, const int* src_len, int n_sent, int beam,
                            int k_best, float min_ratio, float max_ratio, float penalty, int longest_sent,
                            int* out_ids, int* out_len, float* out_score, int* out_align) {
  ZR_CHECK(m && src_ids && src_len && out_ids && out_len && out_score, "beam_decode: null argument");
  ZR_CHECK(n_sent >= 0 && k_best >= 1 && longest_sent >= 1, "beam_decode: bad sizes");
  if (n_sent == 0) return ZRNN_OK;
  int S_max = 0;
  size_t n_ids = 0;
  for (int i = 0; i < n_sent; ++i) {
    ZR_CHECK(src_len[i] >= 1, "beam_decode: empty source sentence");
    S_max = std::max(S_max, src_len[i]);
    n_ids += (size_t)src_len[i];
  }
  ZR_TRY(check_ids(src_ids, n_ids, m->cfg.V_src, "beam_decode (source)"));
  const int Lmax = longest_sent + 4;
  // pad on the host into the reference's minibatch layout: time-major, left-padded with -1
  std::vector<int> padded((size_t)S_max * n_sent, -1);
  size_t pos = 0;
  for (int i = 0; i < n_sent; ++i) {
    for (int t = 0; t < src_len[i]; ++t) padded[(size_t)(S_max - src_len[i] + t) * n_sent + i] = src_ids[pos + t];
    pos += src_len[i];
  }
  const size_t nO = (size_t)n_sent * k_best;
  ZR_CUDA(m->io.reserve(aligned(sizeof(int) * padded.size()) + 2 * aligned(sizeof(int) * nO * Lmax) +
                        aligned(sizeof(int) * nO) + aligned(sizeof(float) * nO)));
  Carver cv(m->io.p);
  int* d_src = cv.take<int>(padded.size());
  int* d_ids = cv.take<int>(nO * Lmax);
  int* d_len = cv.take<int>(nO);
  float* d_sc = cv.take<float>(nO);
  int* d_al = out_align ? cv.take<int>(nO * Lmax) : nullptr;
  cudaStream_t s = m->stream;
  ZR_CUDA(cudaMemcpyAsync(d_src, padded.data(), sizeof(int) * padded.size(), cudaMemcpyHostToDevice, s));
  const int* d_src_c = d_src;
  ZR_TRY(beam_decode_core(&m, 1, &d_src_c, src_len, &S_max, n_sent, beam, k_best, min_ratio, max_ratio, penalty,
                          longest_sent, d_ids, d_len, d_sc, d_al, s, comm));
  if (out_align) ZR_CUDA(cudaMemcpyAsync(out_align, d_al, sizeof(int) * nO * Lmax, cudaMemcpyDeviceToHost, s));
  ZR_CUDA(cudaMemcpyAsync(out_ids, d_ids, sizeof(int) * nO * Lmax, cudaMemcpyDeviceToHost, s));
  ZR_CUDA(cudaMemcpyAsync(out_len, d_len, sizeof(int) * nO, cudaMemcpyDeviceToHost, s));
  ZR_CUDA(cudaMemcpyAsync(out_score, d_sc, sizeof(float) * nO, cudaMemcpyDeviceToHost, s));
  ZR_CUDA(cudaStreamSynchronize(s));
  ZR_TRY(device_error_status("beam_decode"));
  return ZRNN_OK;
}

int zrnn_beam_decode_batch_align(zrnn_model* m, const int* src_ids, const int* src_len, int n_sent, int beam,
                                 int k_best, float min_ratio, float max_ratio, float penalty, int longest_sent,
                                 int* out_ids, int* out_len, float* out_score, int* out_align) {
  return beam_decode_host(m, nullptr, src_ids, src_len, n_sent, beam, k_best, min_ratio, max_ratio, penalty,
                          longest_sent, out_ids, out_len, out_score, out_align);
}

// ---------------------------------------------------------------- collective layer (vocabulary-sharded softmax)
int zrnn_comm_unique_id(char* id128) {
  ZR_CHECK(id128, "comm_unique_id: null argument");
  static_assert(sizeof(ncclUniqueId) == ZRNN_COMM_ID_BYTES, "the id buffer of the C ABI is the size of NCCL's unique id");
  if (!nccl_api()->ok) return fail(ZRNN_E_NCCL, "the NCCL library (libnccl.so.2) could not be loaded");
  ncclUniqueId id;
  ZR_NCCL(nccl_api()->GetUniqueId(&id));
  std::memcpy(id128, &id, sizeof(id));
  return ZRNN_OK;
}
int zrnn_comm_create(const char* id128, int rank, int world, zrnn_comm** out) {
  ZR_CHECK(out && world >= 1 && rank >= 0 && rank < world, "comm_create: bad arguments");
  ZR_CHECK(world <= ZR_SHARD_MAX, "comm_create: at most 8 ranks");
  ZR_TRY(check_device());
  auto* c = new zrnn_comm();
  c->rank = rank;
  c->world = world;
  if (world > 1) {
    if (!id128) { delete c; return fail(ZRNN_E_ARG, "comm_create: a group of more than one rank needs the unique id"); }
    if (!nccl_api()->ok) { delete c; return fail(ZRNN_E_NCCL, "the NCCL library (libnccl.so.2) could not be loaded"); }
    ncclUniqueId id;
    std::memcpy(&id, id128, sizeof(id));
    const ncclResult_t r = nccl_api()->CommInitRank(&c->comm, world, id, rank);
    if (r != ncclSuccess) {
      delete c;
      return fail(ZRNN_E_NCCL, std::string("ncclCommInitRank: ") + nccl_api()->GetErrorString(r));
    }
  }
  *out = c;
  return ZRNN_OK;
}
int zrnn_comm_from_nccl(void* nccl_comm, int rank, int world, zrnn_comm** out) {
  ZR_CHECK(out && nccl_comm && world >= 2 && rank >= 0 && rank < world, "comm_from_nccl: bad arguments");
  ZR_CHECK(world <= ZR_SHARD_MAX, "comm_from_nccl: at most 8 ranks");
  ZR_TRY(check_device());
  if (!nccl_api()->ok) return fail(ZRNN_E_NCCL, "the NCCL library (libnccl.so.2) could not be loaded");
  auto* c = new zrnn_comm();
  c->comm = (ncclComm_t)nccl_comm;
  c->owned = false;
  c->rank = rank;
  c->world = world;
  *out = c;
  return ZRNN_OK;
}
int zrnn_comm_rank(const zrnn_comm* c, int* rank, int* world) {
  ZR_CHECK(c, "comm_rank: null argument");
  if (rank) *rank = c->rank;
  if (world) *world = c->world;
  return ZRNN_OK;
}
int zrnn_comm_all_gather(zrnn_comm* c, const void* d_send, void* d_recv, size_t bytes_per_rank, void* stream) {
  ZR_CHECK(c && d_send && d_recv, "comm_all_gather: null argument");
  if (!bytes_per_rank) return ZRNN_OK;
  return comm_all_gather(c, d_send, d_recv, bytes_per_rank, (cudaStream_t)stream);
}
int zrnn_comm_last_stage_ms(const zrnn_comm* c, float* ms5) {
  ZR_CHECK(c && ms5, "comm_last_stage_ms: null argument");
  for (int i = 0; i < 5; ++i) ms5[i] = c->stage_ms[i];
  return ZRNN_OK;
}
int zrnn_comm_destroy(zrnn_comm* c) {
  if (!c) return ZRNN_OK;
  if (c->comm && c->owned) nccl_api()->CommDestroy(c->comm);
  delete c;
  return ZRNN_OK;
}
int zrnn_shard_range(int V, int world, int rank, int* lo, int* hi) {
  ZR_CHECK(V >= 0 && world >= 1 && rank >= 0 && rank < world && lo && hi, "shard_range: bad arguments");
  shard_range(V, world, rank, lo, hi);
  return ZRNN_OK;
}

int zrnn_softmax_topk_shard(zrnn_softmax* S, const float* d_h, int N, int k, float* d_logp_out, int* d_idx_out,
                            float* d_lse_out, float* d_logp_eos, void* stream) {
  ZR_CHECK(S && d_h && d_logp_out && d_idx_out && d_lse_out && N >= 0, "softmax_topk_shard: bad arguments");
  ZR_CHECK(k >= 1 && k <= ZR_BEAM_MAX + 1, "softmax_topk_shard: k must be in [1,33]");
  if (!S->loaded) return fail(ZRNN_E_STATE, "softmax_topk_shard: weights not loaded");
  if (N == 0) return ZRNN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  Act h;
  ZR_TRY(softmax_input(S, d_h, N, &h, st));
  return softmax_topk_act(S, h, N, k, d_logp_out, d_idx_out, d_logp_eos, st, d_lse_out);
}
int zrnn_topk_merge(const float* d_val, const int* d_idx, const float* d_lse, const float* d_eos, const int* d_shard_lo,
                    int G, int N, int k, float* d_val_out, int* d_idx_out, float* d_eos_out, void* stream) {
  ZR_CHECK(d_val && d_idx && d_lse && d_shard_lo && d_val_out && d_idx_out && N >= 0, "topk_merge: bad arguments");
  ZR_CHECK(!d_eos_out || d_eos, "topk_merge: an <EOF> output needs the shards' <EOF> values");
  ZR_CHECK(G >= 1 && G <= ZR_SHARD_MAX && k >= 1 && k <= ZR_BEAM_MAX + 1, "topk_merge: 1..8 shards of 1..33 candidates");
  if (N == 0) return ZRNN_OK;
  ZR_CUDA(zrnn::launch_topk_merge(d_val, d_idx, d_lse, d_eos, d_shard_lo, G, N, k, d_val_out, d_idx_out, d_eos_out,
                                  (cudaStream_t)stream));
  return ZRNN_OK;
}
int zrnn_softmax_topk_sharded(zrnn_softmax* S, zrnn_comm* c, const float* d_h, int N, int k, float* d_logp_out,
                              int* d_idx_out, float* d_logp_eos, void* stream) {
  ZR_CHECK(S && c && d_h && d_logp_out && d_idx_out && N >= 0, "softmax_topk_sharded: bad arguments");
  ZR_CHECK(k >= 1 && k <= ZR_BEAM_MAX + 1, "softmax_topk_sharded: k must be in [1,33]");
  if (!S->loaded) return fail(ZRNN_E_STATE, "softmax_topk_sharded: weights not loaded");
  if (N == 0) return ZRNN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  Act h;
  ZR_TRY(softmax_input(S, d_h, N, &h, st));
  return softmax_topk_sharded_act(S, c, h, N, k, d_logp_out, d_idx_out, d_logp_eos, st);
}

int zrnn_beam_decode_batch_sharded(zrnn_model* m, zrnn_comm* c, const int* src_ids, const int* src_len, int n_sent,
                                   int beam, int k_best, float min_ratio, float max_ratio, float penalty,
                                   int longest_sent, int* out_ids, int* out_len, float* out_score) {
  ZR_CHECK(c, "beam_decode_sharded: null communicator");
  return beam_decode_host(m, c, src_ids, src_len, n_sent, beam, k_best, min_ratio, max_ratio, penalty, longest_sent,
                          out_ids, out_len, out_score, nullptr);
}

// Teacher-forced scoring over `world` ranks.  Every rank passes the SAME host batch.  The recurrent stack and the
// attention run data-parallel (rank r takes the columns [B r / world, B (r+1) / world), padded to the widest share);
// the top hidden states are all-gathered; every rank scores all columns against its slice of the vocabulary; one more
// all-gather of (max, sum, target logit) per column and the combine give every rank the whole log-probability matrix.
int zrnn_score_batch_sharded(zrnn_model* m, zrnn_comm* c, const int* src_ids, int S_max, const int* tgt_in,
                             const int* tgt_out, int T, int B, float* logp_out, double* total_logp) {
  ZR_CHECK(m && c && tgt_in && tgt_out && logp_out, "score_batch_sharded: null argument");
  ZR_CHECK(T >= 0 && B >= 0 && S_max >= 0, "score_batch_sharded: negative size");
  if (!m->finalized) return fail(ZRNN_E_STATE, "score_batch_sharded: model weights not finalized");
  {
    int lo, hi;
    shard_range(m->cfg.V_tgt, c->world, c->rank, &lo, &hi);
    ZR_CHECK(m->sm->lo == lo && m->sm->hi == hi, "score_batch_sharded: the model's vocabulary range is not this rank's share");
  }
  if (total_logp) *total_logp = 0.0;
  if (T == 0 || B == 0) return ZRNN_OK;
  const bool lm = m->cfg.lm != 0;
  const int G = c->world, H = m->cfg.H;
  const int S = lm ? 0 : S_max;
  ZR_CHECK(lm || src_ids, "score_batch_sharded: a sequence-to-sequence model needs source ids");
  if (S) ZR_TRY(check_ids(src_ids, (size_t)S * B, m->cfg.V_src, "score_batch_sharded (source)"));
  ZR_TRY(check_ids(tgt_in, (size_t)T * B, m->cfg.V_tgt, "score_batch_sharded (target input)"));
  ZR_TRY(check_ids(tgt_out, (size_t)T * B, m->cfg.V_tgt, "score_batch_sharded (target output)"));
  const int Bp = (B + G - 1) / G;  // columns per rank (the last shares are padded with masked columns)
  int b_lo, b_hi;
  shard_range(B, G, c->rank, &b_lo, &b_hi);
  const size_t nS = (size_t)S * Bp, nT = (size_t)T * Bp, nAll = nT * G;
  // this rank's columns, and the target words of ALL columns in gathered order (rank, step, local column)
  const size_t n_ids = nS + nT + nAll;
  ZR_CUDA(c->pin_reserve(aligned(sizeof(int) * n_ids) + sizeof(float) * nAll));
  int* h_ids = (int*)c->pin;
  float* h_lp = (float*)((char*)c->pin + aligned(sizeof(int) * n_ids));
  std::fill(h_ids, h_ids + n_ids, -1);
  int* l_src = h_ids;
  int* l_tin = l_src + nS;
  int* a_tout = l_tin + nT;
  for (int b = b_lo; b < b_hi; ++b) {
    for (int t = 0; t < S; ++t) l_src[(size_t)t * Bp + (b - b_lo)] = src_ids[(size_t)t * B + b];
    for (int t = 0; t < T; ++t) l_tin[(size_t)t * Bp + (b - b_lo)] = tgt_in[(size_t)t * B + b];
  }
  for (int g = 0; g < G; ++g) {
    int lo, hi;
    shard_range(B, G, g, &lo, &hi);
    for (int t = 0; t < T; ++t)
      for (int b = lo; b < hi; ++b) a_tout[(size_t)g * nT + (size_t)t * Bp + (b - lo)] = tgt_out[(size_t)t * B + b];
  }
  const Geom geo{H, round64(H), m->eng};
  const bool op_gather = m->eng == ENG_BF16;  // the bf16 engine's operand form is half the bytes of the fp32 states
  const size_t col_bytes = op_gather ? (size_t)geo.Kpad * 2 : sizeof(float) * (size_t)H;
  ZR_CUDA(m->io.reserve(aligned(sizeof(int) * n_ids) + 2 * aligned(sizeof(int) * nAll) + aligned(sizeof(float) * nAll)));
  ZR_CUDA(c->recv.reserve(col_bytes * nAll));
  ZR_CUDA(c->send.reserve(3 * sizeof(float) * nAll));
  ZR_CUDA(c->aux.reserve(3 * sizeof(float) * nAll * G));
  Carver cv(m->io.p);
  int* d_ids = cv.take<int>(n_ids);
  int* d_tout = cv.take<int>(nAll);
  int* d_mask = cv.take<int>(nAll);
  float* d_lp = cv.take<float>(nAll);
  cudaStream_t s = m->stream;
  for (auto& e : c->ev) if (!e) ZR_CUDA(cudaEventCreate(&e));
  ZR_CUDA(cudaEventRecord(c->ev[0], s));
  ZR_CUDA(cudaMemcpyAsync(d_ids, h_ids, sizeof(int) * n_ids, cudaMemcpyHostToDevice, s));
  m->drop_graph();
  ZR_TRY(score_batch_body(m, S ? d_ids : nullptr, S, d_ids + nS, d_ids + nS, T, Bp, nullptr, s));
  const Act top = m->last_top_act;
  Act all;
  ZR_CUDA(cudaEventRecord(c->ev[1], s));
  if (op_gather) {
    ZR_TRY(comm_all_gather(c, top.hi, c->recv.p, col_bytes * nT, s));
    all.hi = c->recv.p;
  } else {
    ZR_TRY(comm_all_gather(c, top.f32, c->recv.p, col_bytes * nT, s));
    ZR_TRY(softmax_input(m->sm, c->recv.as<float>(), (int)nAll, &all, s));
  }
  ZR_CUDA(cudaEventRecord(c->ev[2], s));
  ZR_CUDA(zrnn::launch_prep_ids(d_ids + nS + nT, (int)nAll, d_tout, d_mask, s));
  float* mx = c->send.as<float>();
  float* sm = mx + nAll;
  float* tg = sm + nAll;
  {
    int np = 0;
    float *pm, *ps;
    ZR_TRY(softmax_partials_launch(m->sm, all, d_tout, (int)nAll, &np, &pm, &ps, tg, s));
    KScope ks(KC_SOFTMAX_REDUCE, s);
    ZR_CUDA(zrnn::launch_lse_reduce(pm, ps, np, (int)nAll, mx, sm, s));
  }
  ZR_CUDA(cudaEventRecord(c->ev[3], s));
  // one all-gather of [max | sum | target logit]; the combine reads the three [G][N] arrays with the block stride
  ZR_TRY(comm_all_gather(c, c->send.p, c->aux.p, 3 * sizeof(float) * nAll, s));
  const float* r = c->aux.as<float>();
  ZR_CUDA(zrnn::launch_lse_combine_shards(r, r + nAll, r + 2 * nAll, G, (int)nAll, d_mask, d_lp, s, 3 * nAll));
  ZR_CUDA(cudaEventRecord(c->ev[4], s));
  ZR_CUDA(cudaMemcpyAsync(h_lp, d_lp, sizeof(float) * nAll, cudaMemcpyDeviceToHost, s));
  ZR_CUDA(cudaEventRecord(c->ev[5], s));
  ZR_CUDA(cudaStreamSynchronize(s));
  for (int i = 0; i < 5; ++i) ZR_CUDA(cudaEventElapsedTime(&c->stage_ms[i], c->ev[i], c->ev[i + 1]));
  ZR_TRY(device_error_status("score_batch_sharded"));
  double tot = 0;
  for (int g = 0; g < G; ++g) {
    int lo, hi;
    shard_range(B, G, g, &lo, &hi);
    for (int t = 0; t < T; ++t)
      for (int b = lo; b < hi; ++b) {
        const float v = h_lp[(size_t)g * nT + (size_t)t * Bp + (b - lo)];
        logp_out[(size_t)t * B + b] = v;
        tot += v;
      }
  }
  if (total_logp) *total_logp = tot;
  return ZRNN_OK;
}

int zrnn_beam_decode_ensemble(zrnn_model* const* models, int n_models, const int* const* src_ids,
                              const int* const* src_len, int n_sent, int beam, int k_best, float min_ratio,
                              float max_ratio, float penalty, int longest_sent, int* out_ids, int* out_len,
                              float* out_score) {
  return zrnn_beam_decode_ensemble_align(models, n_models, src_ids, src_len, n_sent, beam, k_best, min_ratio, max_ratio,
                                         penalty, longest_sent, out_ids, out_len, out_score, nullptr);
}

int zrnn_beam_decode_ensemble_align(zrnn_model* const* models, int n_models, const int* const* src_ids,
                                    const int* const* src_len, int n_sent, int beam, int k_best, float min_ratio,
                                    float max_ratio, float penalty, int longest_sent, int* out_ids, int* out_len,
                                    float* out_score, int* out_align) {
  ZR_CHECK(models && src_ids && src_len && out_ids && out_len && out_score, "beam_decode_ensemble: null argument");
  ZR_CHECK(n_models >= 1 && n_models <= ZR_ENSEMBLE_MAX, "beam_decode_ensemble: between 1 and 8 models");
  ZR_CHECK(n_sent >= 0 && k_best >= 1 && longest_sent >= 1, "beam_decode_ensemble: bad sizes");
  if (n_sent == 0) return ZRNN_OK;
  const int Lmax = longest_sent + 4;
  const size_t nO = (size_t)n_sent * k_best;
  cudaStream_t s = models[0] ? models[0]->stream : nullptr;
  std::vector<const int*> d_src(n_models);
  std::vector<int> S_max(n_models, 0);
  int *d_ids = nullptr, *d_len = nullptr, *d_al = nullptr;
  float* d_sc = nullptr;
  for (int k = 0; k < n_models; ++k) {
    zrnn_model* m = models[k];
    ZR_CHECK(m && src_ids[k] && src_len[k], "beam_decode_ensemble: null argument");
    size_t n_ids = 0;
    for (int i = 0; i < n_sent; ++i) {
      ZR_CHECK(src_len[k][i] >= 1, "beam_decode_ensemble: empty source sentence");
      S_max[k] = std::max(S_max[k], src_len[k][i]);
      n_ids += (size_t)src_len[k][i];
    }
    ZR_TRY(check_ids(src_ids[k], n_ids, m->cfg.V_src, "beam_decode_ensemble (source)"));
    // pad on the host into the reference's minibatch layout: time-major, left-padded with -1
    std::vector<int> padded((size_t)S_max[k] * n_sent, -1);
    size_t pos = 0;
    for (int i = 0; i < n_sent; ++i) {
      for (int t = 0; t < src_len[k][i]; ++t)
        padded[(size_t)(S_max[k] - src_len[k][i] + t) * n_sent + i] = src_ids[k][pos + t];
      pos += src_len[k][i];
    }
    size_t bytes = aligned(sizeof(int) * padded.size());
    if (k == 0) bytes += 2 * aligned(sizeof(int) * nO * Lmax) + aligned(sizeof(int) * nO) + aligned(sizeof(float) * nO);
    ZR_CUDA(m->io.reserve(bytes));
    Carver cv(m->io.p);
    int* dst = cv.take<int>(padded.size());
    if (k == 0) {
      d_ids = cv.take<int>(nO * Lmax); d_len = cv.take<int>(nO); d_sc = cv.take<float>(nO);
      d_al = out_align ? cv.take<int>(nO * Lmax) : nullptr;
    }
    // pageable source: the copy has left `padded` when the call returns
    ZR_CUDA(cudaMemcpyAsync(dst, padded.data(), sizeof(int) * padded.size(), cudaMemcpyHostToDevice, s));
    ZR_CUDA(cudaStreamSynchronize(s));
    d_src[k] = dst;
  }
  ZR_TRY(beam_decode_core(models, n_models, d_src.data(), src_len[0], S_max.data(), n_sent, beam, k_best, min_ratio,
                          max_ratio, penalty, longest_sent, d_ids, d_len, d_sc, d_al, s));
  if (out_align) ZR_CUDA(cudaMemcpyAsync(out_align, d_al, sizeof(int) * nO * Lmax, cudaMemcpyDeviceToHost, s));
  ZR_CUDA(cudaMemcpyAsync(out_ids, d_ids, sizeof(int) * nO * Lmax, cudaMemcpyDeviceToHost, s));
  ZR_CUDA(cudaMemcpyAsync(out_len, d_len, sizeof(int) * nO, cudaMemcpyDeviceToHost, s));
  ZR_CUDA(cudaMemcpyAsync(out_score, d_sc, sizeof(float) * nO, cudaMemcpyDeviceToHost, s));
  ZR_CUDA(cudaStreamSynchronize(s));
  ZR_TRY(device_error_status("beam_decode_ensemble"));
  return ZRNN_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Allocation-free scoring softmax
// ------------------------------------------------------------------------------------------
// Some hosts of this library must not allocate device memory while they run: a serving process that handed the
// whole GPU to its own arena at start-up (a later cudaMalloc fails or fragments it), and a latency-bound decode
// loop where cudaMalloc / cudaFree would stall every stream of the device.  zrnn_softmax_score grows its
// scratch buffers on demand, so it is off limits for them.  The variant below takes its scratch from a fixed
// array that is part of the library image instead; nothing is allocated, the price is a hard size limit.
#define ZRNN_NOALLOC_SCRATCH_FLOATS (4u * 1024u * 1024u) /* 16 MiB, held by every GPU that loads the library */
static __device__ __align__(256) float g_noalloc_scratch[ZRNN_NOALLOC_SCRATCH_FLOATS];

namespace {
// Device address of g_noalloc_scratch per device.  In host code the array's name is only a handle for the
// runtime, not an address a kernel can use, so the address is looked up once per device (with that device
// current) and passed to the kernels as an ordinary pointer.
const int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};

int noalloc_scratch(float** out) {
  int dev = -1;
  ZR_CUDA(cudaGetDevice(&dev));
  ZR_CHECK(dev >= 0 && dev < kMaxDevices, "softmax_score_noalloc: device index out of range");
  if (!g_noalloc_ptr[dev]) {
    float* p = nullptr;
    ZR_CUDA(cudaGetSymbolAddress((void**)&p, g_noalloc_scratch));
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return ZRNN_OK;
}
}  // namespace

extern "C" {

int zrnn_softmax_score_noalloc_max_floats(void) { return (int)ZRNN_NOALLOC_SCRATCH_FLOATS; }

int zrnn_softmax_score_noalloc(zrnn_softmax* S, const float* d_h, const int* d_targets, const int* d_mask, int N,
                               float* d_logp_out, void* stream) {
  ZR_CHECK(S && d_h && d_targets && d_logp_out && N >= 0, "softmax_score_noalloc: bad arguments");
  if (!S->loaded) return fail(ZRNN_E_STATE, "softmax_score_noalloc: weights not loaded");
  ZR_CHECK(S->lo == 0 && S->hi == S->V, "softmax_score_noalloc: layer is vocabulary-sharded");
  if (N == 0) return ZRNN_OK;
  const int tile = (N >= 96 && S->V >= 512) ? 1 : 0;  // same tiling rule as zrnn_softmax_score
  const int rows = zrnn::gemm_rows_per_tile(1, tile);
  const int np = (S->V + rows - 1) / rows;
  const size_t need = (2 * (size_t)np + 1) * (size_t)N;  // per-tile (max, sum) pairs + one target logit per column
  if (need > ZRNN_NOALLOC_SCRATCH_FLOATS)
    return fail(ZRNN_E_ARG, "softmax_score_noalloc: needs " + std::to_string(need) + " scratch floats for V=" +
                                std::to_string(S->V) + ", N=" + std::to_string(N) + " but the built-in scratch holds " +
                                std::to_string(ZRNN_NOALLOC_SCRATCH_FLOATS) + "; split the columns or use zrnn_softmax_score");
  float* scratch = nullptr;
  ZR_TRY(noalloc_scratch(&scratch));
  cudaStream_t st = (cudaStream_t)stream;
  float* pm = scratch;
  float* ps = scratch + (size_t)np * N;
  float* tgt = scratch + 2 * (size_t)np * N;
  // the array still holds the previous call's numbers: the target logits must start from zero, the partials are
  // fully overwritten by the GEMM epilogue
  ZR_CUDA(cudaMemsetAsync(tgt, 0, sizeof(float) * (size_t)N, st));
  zrnn::GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  g.nsrc = 1;
  g.src[0].A[0] = S->D; g.src[0].lda = S->V; g.src[0].B = d_h; g.src[0].ldb = S->H; g.src[0].K = S->H;
  g.M = S->V; g.N = N; g.bias[0] = S->b;
  g.target = d_targets; g.target_offset = 0;
  g.part_max = pm; g.part_sum = ps; g.tgt_logit = tgt;
  ZR_CUDA(zrnn::launch_fused_gemm(g, 1, zrnn::EPI_LSE, tile, st));
  ZR_CUDA(zrnn::launch_lse_combine(pm, ps, tgt, np, N, d_mask, d_logp_out, st));
  return ZRNN_OK;
}

}  // extern "C"


// ------------------------------------------------------------------------------------------
// Stand-alone GEMM (the reference's cublas_gemm_wrapper, src/BZ_CUDA_UTIL.h:691-696, N/N case):
//   C[n_rows x m_cols] = W[n_rows x K] * X[K x m_cols], all column-major.
// ------------------------------------------------------------------------------------------
extern "C" {

int zrnn_gemm(int mode, int n_rows, int m_cols, int K, const float* d_W, int ldw, const float* d_X, int ldx,
              float* d_C, int ldc, void* stream) {
  ZR_CHECK(d_W && d_X && d_C && n_rows > 0 && m_cols > 0 && K > 0, "gemm: bad arguments");
  ZR_CHECK(ldw >= n_rows && ldx >= K && ldc >= n_rows, "gemm: leading dimension too small");
  ZR_CHECK(mode >= 0 && mode <= 4, "gemm: mode must be 0 (fp32 SIMT), 1 (bf16), 2 (tf32), 3 (3xtf32) or 4 (fp16 split)");
  cudaStream_t st = (cudaStream_t)stream;
  if (mode == 0) {
    zrnn::GemmArgs g;
    std::memset(&g, 0, sizeof(g));
    g.nsrc = 1;
    g.src[0].A[0] = d_W; g.src[0].lda = ldw; g.src[0].B = d_X; g.src[0].ldb = ldx; g.src[0].K = K;
    g.M = n_rows; g.N = m_cols; g.C = d_C; g.ldc = ldc;
    ZR_CUDA(zrnn::launch_fused_gemm(g, 1, zrnn::EPI_STORE, (n_rows >= 256 && m_cols >= 96) ? 1 : 0, st));
    return ZRNN_OK;
  }
  const int tcm = mode == 1 ? zrnn::TC_BF16 : (mode == 2 ? zrnn::TC_TF32 : (mode == 3 ? zrnn::TC_TF32X3 : zrnn::TC_F16X2));
  const int op_mode = mode == 1 ? 0 : (mode == 2 ? 1 : (mode == 3 ? 2 : 3));
  const int eb = (mode == 1 || mode == 4) ? 2 : 4;
  const bool split = mode >= 3;
  const int kb_elems = 128 / eb;
  const int Kpad = (K + 63) / 64 * 64;
  const int BN = n_rows >= 256 ? 256 : (n_rows >= 128 ? 128 : (n_rows >= 64 ? 64 : 32));
  const int n_tiles = (n_rows + BN - 1) / BN;
  const size_t a_elems = (size_t)m_cols * Kpad, b_elems = (size_t)n_tiles * BN * Kpad;
  DevBuf a_hi, a_lo, b_hi, b_lo;
  ZR_CUDA(a_hi.reserve(a_elems * eb));
  ZR_CUDA(b_hi.reserve(b_elems * eb));
  ZR_CUDA(cudaMemsetAsync(a_hi.p, 0, a_elems * eb, st));
  ZR_CUDA(cudaMemsetAsync(b_hi.p, 0, b_elems * eb, st));
  if (split) {
    ZR_CUDA(a_lo.reserve(a_elems * eb));
    ZR_CUDA(b_lo.reserve(b_elems * eb));
    ZR_CUDA(cudaMemsetAsync(a_lo.p, 0, a_elems * eb, st));
    ZR_CUDA(cudaMemsetAsync(b_lo.p, 0, b_elems * eb, st));
  }
  ZR_CUDA(zrnn::launch_convert_rows(d_X, m_cols, K, ldx, op_mode, a_hi.p, a_lo.as<float>(), Kpad, st));
  zrnn::PackArgs pk;
  std::memset(&pk, 0, sizeof(pk));
  pk.src[0] = d_W; pk.G = 1; pk.H = n_rows; pk.K = K; pk.lda = ldw; pk.TH = BN; pk.n_tiles = n_tiles;
  pk.dst_hi = b_hi.p; pk.dst_lo = b_lo.as<float>(); pk.op_mode = op_mode; pk.ld_dst = Kpad; pk.koff = 0;
  ZR_CUDA(zrnn::launch_pack_weights(pk, st));
  zrnn::TcParams tp;
  std::memset(&tp, 0, sizeof(tp));
  bool ok = zrnn::make_kmajor_map(&tp.a[0], a_hi.p, eb, Kpad, m_cols, Kpad, 128) &&
            zrnn::make_kmajor_map(&tp.b, b_hi.p, eb, Kpad, (long long)n_tiles * BN, Kpad, BN);
  if (split)
    ok = ok && zrnn::make_kmajor_map(&tp.a_lo[0], a_lo.p, eb, Kpad, m_cols, Kpad, 128) &&
         zrnn::make_kmajor_map(&tp.b_lo, b_lo.p, eb, Kpad, (long long)n_tiles * BN, Kpad, BN);
  if (!ok) {
    a_hi.release(); a_lo.release(); b_hi.release(); b_lo.release();
    return fail(ZRNN_E_CUDA, "gemm: cannot encode TMA tensor maps");
  }
  tp.nsrc = 1; tp.kblocks[0] = (K + kb_elems - 1) / kb_elems; tp.b_koff[0] = 0;
  tp.M = m_cols; tp.N = n_rows; tp.C = d_C; tp.ldc = ldc; tp.err = tc_error_word();
  cudaError_t e = zrnn::launch_tc_gemm(tp, BN, tcm, zrnn::TC_EPI_STORE, st);
  cudaError_t e2 = cudaStreamSynchronize(st);
  a_hi.release(); a_lo.release(); b_hi.release(); b_lo.release();
  ZR_CUDA(e);
  ZR_CUDA(e2);
  const int code = zrnn_tc_error();
  if (code != 0) return fail(ZRNN_E_TIMEOUT, "gemm: a bounded device wait gave up (role " + std::to_string(code) + ")");
  return ZRNN_OK;
}

}  // extern "C"
