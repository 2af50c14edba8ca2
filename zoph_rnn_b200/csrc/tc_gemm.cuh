// Blackwell tensor-core GEMM family (tcgen05.mma with TMEM accumulators, TMA-fed shared-memory ring):
//   acc[M x N] = sum_s A_s[M x K_s] * B[N x Kcat]^T        (both operands K-major)
// M indexes batch columns (the reference's H x B activations are already "B rows of K contiguous values"),
// N indexes weight rows, so every epilogue thread owns one batch column and sees all N outputs of its row:
// the LSTM gate math, the softmax max / sum-exp and the bias + tanh + mask are thread-local.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace zrnn {

enum { TC_BF16 = 0, TC_TF32 = 1, TC_TF32X3 = 2, TC_F16X2 = 3 };
enum { TC_EPI_STORE = 0, TC_EPI_LSTM = 1, TC_EPI_LSE = 2 };

struct TcParams {
  CUtensorMap a[3];     // A operand per source (bf16, or fp32 "hi" = values representable in tf32)
  CUtensorMap a_lo[3];  // TC_TF32X3: fp32 residuals a - a_hi
  CUtensorMap b;        // weights, rows = packed output rows, K = concatenated (padded) sources
  CUtensorMap b_lo;     // TC_TF32X3
  int nsrc;
  int kblocks[3];  // 128-byte k-blocks per source
  int b_koff[3];   // element offset of each source inside B's K axis
  // > 0: B is stored tile-contiguously (k-blocks per row tile): the box of (row tile n, k-block kb) is the
  // rows [(n * b_tiled_kbtot + kb) * BN, + BN) of a 128-byte-wide 2-D array (tc_gemm_kernel only)
  int b_tiled_kbtot;
  // > 0 and < BN: B was packed for row tiles of this many rows (LSTM: 4 gates x pack/4 hidden units per tile) and the
  // launch uses a wider tile made of BN / b_pack_rows consecutive packed tiles (tc_gemm_kernel, SPLITK == 1)
  int b_pack_rows;
  int M;           // batch columns
  int N;           // STORE / LSE: output rows; LSTM: hidden size H (B holds 4H packed rows)
  const float* bias;  // STORE / LSE: [N]; LSTM: [4][H] gate-major (i,f,g,o)
  const int* mask;    // [M] or null
  // --- STORE: C[n + m*ldc] = act(acc + bias[n]) * mask[m]
  float* C;
  int ldc;
  int act;       // 0 none, 1 tanh
  int act_rows;  // act applies to n < act_rows (0 = all)
  // optional A-operand copies of the output for the next GEMM (row m at + m*ld_op)
  __nv_bfloat16* op_b16;
  float* op_hi;
  float* op_lo;
  __half* op_h_hi;  // TC_F16X2 consumers: fp16 hi part and scaled fp16 lo part
  __half* op_h_lo;
  int ld_op;
  // --- LSTM (gates i,f,g,o): c = f*c_prev + i*g ; h = o*tanh(c) ; (h,c) *= mask ; h -> C (ld = ldc), c -> c_out
  const float* c_prev;
  float* c_out;
  // --- LSE: per (N tile, m) max and sum exp(z - max) of z = acc + bias, plus the logit of target[m]
  const int* target;
  int target_offset;
  float* part_max;  // [n_tiles x M]
  float* part_sum;
  float* tgt_logit;  // [M]
  int* err;          // device error word (0 = ok); set when a bounded wait gives up
  long long* prof;   // optional: 8 globaltimer stamps per CTA (developer profiling)
  int prof_slot;     // >= 0: only CTA (0,0,0) stamps, into prof[prof_slot*8 ..] (timeline of many launches)
};

// BN = N-tile (LSTM: 4*TH). Returns cudaErrorInvalidValue for unsupported (BN, mode, epi) combinations.
// splitk > 1 (BN == 128 only: 2, 4, and 8 for the non-LSTM epilogues) splits the K axis over a thread-block cluster;
// the LSE epilogue then produces n_tiles * splitk partial rows.
cudaError_t launch_tc_gemm(const TcParams& p, int BN, int mode, int epi, cudaStream_t st, int splitk = 1);

// Up to TcMulti::MAX independent LSTM layer-steps (EPI_LSTM, 128-row weight tiles, M <= 128 columns and the same
// hidden size each) in one launch: grid (n, row tiles, splitk).  Nothing orders the problems among themselves.
struct TcMulti {
  enum { MAX = 8 };
  TcParams p[MAX];
};
cudaError_t launch_tc_lstm_multi(const TcMulti& pm, int n, int mode, cudaStream_t st, int splitk);

// Persistent one-CTA-per-SM variant for large problems (store and log-sum-exp epilogues).  The B tensor map must use
// 256-row boxes for TC_BF16 / TC_TF32 and 128-row boxes for the split modes.  Two epilogue warps share each output
// row of a tile, one per half of its columns, so the (max, sum) partials are indexed
// [(n_tile * kPersistentParts + half) x M] and each covers tile width / kPersistentParts consecutive columns.
constexpr int kPersistentParts = 2;
cudaError_t launch_tc_gemm_persistent(const TcParams& p, int mode, int epi, cudaStream_t st);
// One warp waits (bounded by limit_cycles SM cycles) on a barrier that never completes and reports `code` in *err.
cudaError_t launch_wait_probe(int* err, long long limit_cycles, int code, cudaStream_t st);

// Host helpers -------------------------------------------------------------------------------------------
// 2-D K-major tensor map: `rows` rows of `k` elements, row stride ld (elements); box = (128-byte k-block) x box_rows
// elem_bytes 2 (bf16) or 4 (fp32).  Returns false when the driver entry point is unavailable or arguments are
// not encodable (base not 16-byte aligned, ld*elem_bytes not a multiple of 16).
bool make_kmajor_map(CUtensorMap* out, const void* base, int elem_bytes, long long k, long long rows, long long ld,
                     int box_rows);

// round fp32 to the nearest value representable in tf32 (10 mantissa bits), ties away from zero on the bit pattern
inline float tf32_round_host(float x) {
  unsigned u;
  memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;
  u = (u + 0x1000u) & 0xffffe000u;
  float r;
  memcpy(&r, &u, 4);
  return r;
}

}  // namespace zrnn
