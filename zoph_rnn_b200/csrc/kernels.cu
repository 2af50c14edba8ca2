// Hand-written sm_100a kernels (exact-fp32 SIMT family) for the Zoph_RNN inference forward path.
// Layouts follow the reference: column-major, activations H x B, ids time-major int32.
#include "kernels.cuh"
#include "att_device.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cfloat>
#include <cstdint>
#include <cstdlib>
#include <cstring>

namespace zrnn {

static thread_local long long g_launches = 0;
void count_launch(int n) { g_launches += n; }
long long launch_count_value() { return g_launches; }
void launch_count_reset() { g_launches = 0; }

// ------------------------------------------------------------------------------------------
// small helpers
// ------------------------------------------------------------------------------------------
// Programmatic dependent launch for the kernels that sit between tensor-core launches on the scoring / decoding
// chain: the kernel may be scheduled while its predecessor drains (the launch latency disappears from the chain),
// waits for the predecessor's results with griddepcontrol.wait before touching them, and at once allows its own
// successor to be scheduled (that one waits the same way).
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
static const bool g_pdl = std::getenv("ZRNN_NO_PDL") == nullptr;
template <class... KArgs, class... Args>
static cudaError_t launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                Args... args) {
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// block-wide sum; result valid in every thread. `red` needs 32 floats.
__device__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// ------------------------------------------------------------------------------------------
// ids: -1 padding -> (id or 0, mask)
// ------------------------------------------------------------------------------------------
__global__ void prep_ids_kernel(const int* __restrict__ raw, int n, int* __restrict__ nonm1, int* __restrict__ mask01) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int v = raw[i];
    if (nonm1) nonm1[i] = (v == -1) ? 0 : v;
    if (mask01) mask01[i] = (v == -1) ? 0 : 1;
  }
}
cudaError_t launch_prep_ids(const int* raw, int n, int* nonm1, int* mask01, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  const int blocks = (n + 255) / 256;
  prep_ids_kernel<<<blocks > 1184 ? 1184 : blocks, 256, 0, st>>>(raw, n, nonm1, mask01);
  count_launch();
  return cudaGetLastError();
}

// The first launch of a scoring pass: the id preparation of up to three id arrays (-1 -> 0 and a 0/1 mask,
// src/custom_kernels.h:9-50) and the zero fills of the start states, which were one graph node each.
__global__ void __launch_bounds__(256) score_prologue_kernel(const PrologueArgs a) {
  const size_t gtid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, gsz = (size_t)gridDim.x * blockDim.x;
  for (int q = 0; q < 3; ++q) {
    const int* raw = a.raw[q];
    if (!raw) continue;
    for (size_t i = gtid; i < (size_t)a.n[q]; i += gsz) {
      const int v = raw[i];
      a.ids[q][i] = v == -1 ? 0 : v;
      a.mask[q][i] = v == -1 ? 0 : 1;
    }
  }
  for (int z = 0; z < a.n_zero; ++z) {
    uint4* p = reinterpret_cast<uint4*>(a.zero_ptr[z]);
    const size_t n16 = a.zero_bytes[z] >> 4;
    for (size_t i = gtid; i < n16; i += gsz) p[i] = make_uint4(0u, 0u, 0u, 0u);
    // tails shorter than 16 bytes (sizes are multiples of 4)
    const size_t done = n16 << 4, rest = (a.zero_bytes[z] - done) >> 2;
    if (gtid < rest) reinterpret_cast<unsigned*>(reinterpret_cast<char*>(a.zero_ptr[z]) + done)[gtid] = 0u;
  }
}
cudaError_t launch_score_prologue(const PrologueArgs& a, cudaStream_t st) {
  size_t work = 0;
  for (int q = 0; q < 3; ++q) work = a.raw[q] && (size_t)a.n[q] > work ? (size_t)a.n[q] : work;
  for (int z = 0; z < a.n_zero; ++z) {
    if ((reinterpret_cast<uintptr_t>(a.zero_ptr[z]) & 15) || (a.zero_bytes[z] & 3)) return cudaErrorInvalidValue;
    work = (a.zero_bytes[z] >> 4) > work ? (a.zero_bytes[z] >> 4) : work;
  }
  if (work == 0) return cudaSuccess;
  const size_t blocks = (work + 255) / 256;
  score_prologue_kernel<<<(unsigned)(blocks > 1184 ? 1184 : blocks), 256, 0, st>>>(a);
  count_launch();
  return cudaGetLastError();
}

__global__ void fill_int_kernel(int* p, int v, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}
__global__ void src_len_kernel(const int* __restrict__ mask01, int T, int B, int* len, int* offset) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int n = 0;
  for (int t = 0; t < T; ++t) n += mask01[(size_t)t * B + b];
  len[b] = n;
  offset[b] = T - n;
}
cudaError_t launch_src_len(const int* mask01, int T, int B, int* len, int* offset, cudaStream_t st) {
  if (B <= 0) return cudaSuccess;
  src_len_kernel<<<(B + 127) / 128, 128, 0, st>>>(mask01, T, B, len, offset);
  count_launch();
  return cudaGetLastError();
}
__global__ void div_map_kernel(int* map, int n, int div) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) map[i] = i / div;
}
cudaError_t launch_div_map(int* map, int n, int div, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  div_map_kernel<<<(n + 127) / 128, 128, 0, st>>>(map, n, div);
  count_launch();
  return cudaGetLastError();
}
cudaError_t launch_fill_int(int* p, int v, size_t n, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  size_t blocks = (n + 255) / 256;
  fill_int_kernel<<<(unsigned)(blocks > 1184 ? 1184 : blocks), 256, 0, st>>>(p, v, n);
  count_launch();
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// operand preparation for the tensor-core GEMMs
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float tf32_round_prep(float x) {
  unsigned u = __float_as_uint(x);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;
  return __uint_as_float((u + 0x1000u) & 0xffffe000u);
}
__device__ __forceinline__ void store_op(void* hi, float* lo, int mode, size_t idx, float v) {
  if (mode == 0) {
    reinterpret_cast<__nv_bfloat16*>(hi)[idx] = __float2bfloat16(v);
  } else if (mode == 1) {
    reinterpret_cast<float*>(hi)[idx] = v;
  } else if (mode == 3) {  // fp16 split: hi = fp16(v), lo = fp16((v - hi) * 2^11); `lo` points to __half storage
    const __half h = __float2half_rn(v);
    reinterpret_cast<__half*>(hi)[idx] = h;
    reinterpret_cast<__half*>(lo)[idx] = __float2half_rn((v - __half2float(h)) * 2048.0f);
  } else {
    const float h = tf32_round_prep(v);
    reinterpret_cast<float*>(hi)[idx] = h;
    lo[idx] = v - h;
  }
}
__global__ void pack_weights_kernel(const PackArgs a) {
  const int rows_per_tile = a.G * a.TH;
  const long long total = (long long)a.n_tiles * rows_per_tile * a.K;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    // hid fastest so the column-major source is read contiguously
    const int j = (int)(e % a.TH);
    long long r = e / a.TH;
    const int tile = (int)(r % a.n_tiles);
    r /= a.n_tiles;
    const int g = (int)(r % a.G);
    const int k = (int)(r / a.G);
    const int hid = tile * a.TH + j;
    const float v = hid < a.H ? a.src[g][(size_t)k * a.lda + hid] : 0.f;
    const size_t prow = (size_t)tile * rows_per_tile + (size_t)g * a.TH + j;
    size_t at = prow * a.ld_dst + a.koff + k;
    if (a.tiled_kbtot > 0) {
      const int kk = a.koff + k;
      at = (((size_t)tile * a.tiled_kbtot + kk / a.tiled_epk) * rows_per_tile + (size_t)g * a.TH + j) * a.tiled_epk +
           kk % a.tiled_epk;
    }
    store_op(a.dst_hi, a.dst_lo, a.op_mode, at, v);
  }
}
cudaError_t launch_pack_weights(const PackArgs& a, cudaStream_t st) {
  const long long total = (long long)a.n_tiles * a.G * a.TH * a.K;
  if (total <= 0) return cudaSuccess;
  long long blocks = (total + 255) / 256;
  pack_weights_kernel<<<(unsigned)(blocks > 148 * 32 ? 148 * 32 : blocks), 256, 0, st>>>(a);
  count_launch();
  return cudaGetLastError();
}
__global__ void convert_rows_kernel(const float* __restrict__ src, long long rows, int K, long long ld_src, int mode,
                                    void* dst_hi, float* dst_lo, long long ld_dst) {
  const long long total = rows * K;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const long long r = e / K;
    const int k = (int)(e % K);
    store_op(dst_hi, dst_lo, mode, (size_t)(r * ld_dst + k), src[r * ld_src + k]);
  }
}
cudaError_t launch_convert_rows(const float* src, long long rows, int K, long long ld_src, int op_mode, void* dst_hi,
                                float* dst_lo, long long ld_dst, cudaStream_t st) {
  const long long total = rows * K;
  if (total <= 0) return cudaSuccess;
  long long blocks = (total + 255) / 256;
  convert_rows_kernel<<<(unsigned)(blocks > 148 * 32 ? 148 * 32 : blocks), 256, 0, st>>>(src, rows, K, ld_src, op_mode,
                                                                                        dst_hi, dst_lo, ld_dst);
  count_launch();
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// embedding column gather: x[:,n] = W[:,ids[n]] -- a bit copy, 16-byte vectorised when H % 4 == 0.
// One CTA of 128 threads per 4 columns keeps every load/store a full 128-byte line.
// ------------------------------------------------------------------------------------------
__global__ void gather_columns_kernel(const float* __restrict__ W, int H, int V, const int* __restrict__ ids, int n_cols,
                                      float* __restrict__ x, int* err) {
  const int vec = ((H & 3) == 0);
  for (int col = blockIdx.x; col < n_cols; col += gridDim.x) {
    int id = ids[col];
    if (id < 0) id = 0;  // an invalid beam slot; its column is never consumed
    if (V > 0 && id >= V) {  // an id of another vocabulary: read column 0 instead and report it
      id = 0;
      if (err && threadIdx.x == 0) atomicExch(err, kErrBadTokenId);
    }
    const float* src = W + (size_t)id * H;
    float* dst = x + (size_t)col * H;
    if (vec) {
      const float4* s4 = reinterpret_cast<const float4*>(src);
      float4* d4 = reinterpret_cast<float4*>(dst);
      for (int i = threadIdx.x; i < (H >> 2); i += blockDim.x) d4[i] = __ldg(s4 + i);
    } else {
      for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = __ldg(src + i);
    }
  }
}
cudaError_t launch_gather_columns(const float* W, int H, int V, const int* ids, int n_cols, float* x, int* err,
                                  cudaStream_t st) {
  if (n_cols <= 0) return cudaSuccess;
  const int threads = H >= 512 ? 128 : 64;
  gather_columns_kernel<<<n_cols > 148 * 16 ? 148 * 16 : n_cols, threads, 0, st>>>(W, H, V, ids, n_cols, x, err);
  count_launch();
  return cudaGetLastError();
}

__global__ void gather_rows16_kernel(const uint4* __restrict__ src, int vec_per_row, int n_src_rows,
                                     const int* __restrict__ ids, int n_rows, uint4* __restrict__ dst, int* err) {
  for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
    int id = ids[r];
    if (id < 0) id = 0;
    if (n_src_rows > 0 && id >= n_src_rows) {
      id = 0;
      if (err && threadIdx.x == 0) atomicExch(err, kErrBadTokenId);
    }
    const uint4* s = src + (size_t)id * vec_per_row;
    uint4* d = dst + (size_t)r * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) d[i] = __ldg(s + i);
  }
}
cudaError_t launch_gather_rows16(const void* src, size_t row_bytes, int n_src_rows, const int* ids, int n_rows,
                                 void* dst, int* err, cudaStream_t st) {
  if (n_rows <= 0) return cudaSuccess;
  if (row_bytes % 16 != 0) return cudaErrorInvalidValue;
  gather_rows16_kernel<<<n_rows > 148 * 16 ? 148 * 16 : n_rows, 128, 0, st>>>(
      reinterpret_cast<const uint4*>(src), (int)(row_bytes / 16), n_src_rows, ids, n_rows,
      reinterpret_cast<uint4*>(dst), err);
  count_launch();
  return cudaGetLastError();
}

__global__ void col_gather_kernel(ColGatherArgs a) {
  const int arr = blockIdx.y;
  const float* src = a.src[arr];
  float* dst = a.dst[arr];
  const int H = a.h_arr[arr] > 0 ? a.h_arr[arr] : a.H;
  for (int col = blockIdx.x; col < a.n_cols; col += gridDim.x) {
    const int sc = a.map[col];
    const float* s = src + (size_t)sc * H;
    float* d = dst + (size_t)col * H;
    if ((H & 3) == 0) {
      for (int i = threadIdx.x; i < (H >> 2); i += blockDim.x)
        reinterpret_cast<float4*>(d)[i] = reinterpret_cast<const float4*>(s)[i];
    } else {
      for (int i = threadIdx.x; i < H; i += blockDim.x) d[i] = s[i];
    }
  }
}
cudaError_t launch_col_gather(const ColGatherArgs& a, cudaStream_t st) {
  if (a.n_cols <= 0 || a.n_arrays <= 0) return cudaSuccess;
  dim3 grid(a.n_cols > 1184 ? 1184 : a.n_cols, a.n_arrays);
  col_gather_kernel<<<grid, 128, 0, st>>>(a);
  count_launch();
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// fused multi-source fp32 GEMM with LSTM / store / log-sum-exp epilogues
// ------------------------------------------------------------------------------------------
template <int GATES, int EPI, int TM, int TN>
__global__ void __launch_bounds__(256) fused_gemm_kernel(const GemmArgs p) {
  constexpr int BM = 16 * TM, BN = 16 * TN, BK = 16;
  constexpr int TH = BM / GATES;  // rows of each gate block covered by this CTA
  __shared__ __align__(16) float As[2][BK][BM + 4];
  __shared__ __align__(16) float Bs[2][BK][BN + 4];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.x * TH;
  const int n0 = blockIdx.y * BN;
  const int M = p.M, N = p.N;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  int ntiles = 0;
  for (int s = 0; s < p.nsrc; ++s) ntiles += (p.src[s].K + BK - 1) / BK;

  float ra[TM], rb[TN];
  int fs = 0, fk0 = 0;  // fetch cursor: source index, k offset
  auto fetch = [&]() {
    const GemmSrc& S = p.src[fs];
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      const int e = tid + 256 * i;
      const int m = e % BM, k = e / BM;
      const int g = m / TH, row = m0 + (m % TH);
      const int kk = fk0 + k;
      ra[i] = (row < M && kk < S.K) ? __ldg(S.A[g] + (size_t)kk * S.lda + row) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < TN; ++i) {
      const int e = tid + 256 * i;
      const int k = e % BK, n = e / BK;
      const int kk = fk0 + k, col = n0 + n;
      rb[i] = (col < N && kk < S.K) ? S.B[(size_t)col * S.ldb + kk] : 0.f;
    }
    fk0 += BK;
    if (fk0 >= S.K) { fk0 = 0; ++fs; }
  };
  auto stage = [&](int buf) {
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      const int e = tid + 256 * i;
      As[buf][e / BM][e % BM] = ra[i];
    }
#pragma unroll
    for (int i = 0; i < TN; ++i) {
      const int e = tid + 256 * i;
      Bs[buf][e % BK][e / BK] = rb[i];
    }
  };

  if (ntiles > 0) {
    fetch();
    stage(0);
  }
  __syncthreads();
  for (int t = 0; t < ntiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < ntiles) fetch();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[buf][k][tx + 16 * i];
#pragma unroll
      for (int j4 = 0; j4 < TN / 4; ++j4) {
        const float4 v = *reinterpret_cast<const float4*>(&Bs[buf][k][j4 * 64 + ty * 4]);
        b[4 * j4 + 0] = v.x; b[4 * j4 + 1] = v.y; b[4 * j4 + 2] = v.z; b[4 * j4 + 3] = v.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (t + 1 < ntiles) stage(buf ^ 1);
    __syncthreads();
  }

  // ---------------- epilogues ----------------
  if (EPI == EPI_STORE) {
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      const int r = tx + 16 * i;
      const int g = r / TH, row = m0 + (r % TH);
      if (row >= M) continue;
      const float bv = p.bias[g] ? p.bias[g][row] : 0.f;
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        const int col = n0 + (j / 4) * 64 + ty * 4 + (j % 4);
        if (col >= N) continue;
        float v = acc[i][j] + bv;
        if (p.act == 1 && (p.act_rows == 0 || row < p.act_rows)) v = tanhf(v);
        if (p.mask) v *= (float)p.mask[col];
        p.C[(size_t)col * p.ldc + (size_t)g * M + row] = v;
      }
    }
  } else if (EPI == EPI_LSTM) {
    constexpr int U = TM / 4;  // hidden units per thread
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int row = m0 + tx + 16 * u;
      if (row >= M) continue;
      const float b_i = p.bias[0][row], b_f = p.bias[1][row], b_g = p.bias[2][row], b_o = p.bias[3][row];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        const int col = n0 + (j / 4) * 64 + ty * 4 + (j % 4);
        if (col >= N) continue;
        const float gi = sigmoidf_acc(acc[0 * U + u][j] + b_i);
        const float gf = sigmoidf_acc(acc[1 * U + u][j] + b_f);
        const float gg = tanhf(acc[2 * U + u][j] + b_g);
        const float go = sigmoidf_acc(acc[3 * U + u][j] + b_o);
        const size_t idx = (size_t)col * M + row;
        float c = gf * p.c_prev[idx] + gi * gg;
        float h = go * tanhf(c);
        if (p.mask) {
          const float mk = (float)p.mask[col];
          h *= mk;
          c *= mk;
        }
        p.h_out[idx] = h;
        p.c_out[idx] = c;
        if (p.h_out2) p.h_out2[idx] = h;
      }
    }
  } else {  // EPI_LSE
    float (&z)[TM][TN] = acc;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      const int row = m0 + tx + 16 * i;
      const float bv = (row < M && p.bias[0]) ? p.bias[0][row] : 0.f;
#pragma unroll
      for (int j = 0; j < TN; ++j) z[i][j] = (row < M) ? acc[i][j] + bv : -INFINITY;
    }
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int col = n0 + (j / 4) * 64 + ty * 4 + (j % 4);
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < TM; ++i) mx = fmaxf(mx, z[i][j]);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sm = 0.f;
#pragma unroll
      for (int i = 0; i < TM; ++i) sm += (z[i][j] == -INFINITY) ? 0.f : expf(z[i][j] - mx);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
      if (col < N) {
        if (tx == 0) {
          p.part_max[(size_t)blockIdx.x * N + col] = mx;
          p.part_sum[(size_t)blockIdx.x * N + col] = sm;
        }
        if (p.target) {
          const int tg = p.target[col] - p.target_offset;
#pragma unroll
          for (int i = 0; i < TM; ++i)
            if (m0 + tx + 16 * i == tg && tg >= 0 && tg < M) p.tgt_logit[col] = z[i][j];
        }
      }
    }
  }
}

int gemm_rows_per_tile(int gates, int tile) { return (tile ? 128 : 64) / gates; }

template <int GATES, int EPI>
static cudaError_t launch_fused_gemm_t(const GemmArgs& a, int tile, cudaStream_t st) {
  const int TH = gemm_rows_per_tile(GATES, tile);
  const int BN = tile ? 128 : 64;
  dim3 grid((a.M + TH - 1) / TH, (a.N + BN - 1) / BN);
  if (grid.x == 0 || grid.y == 0) return cudaSuccess;
  if (tile) fused_gemm_kernel<GATES, EPI, 8, 8><<<grid, 256, 0, st>>>(a);
  else fused_gemm_kernel<GATES, EPI, 4, 4><<<grid, 256, 0, st>>>(a);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_fused_gemm(const GemmArgs& a, int gates, int epi, int tile, cudaStream_t st) {
  if (gates == 4 && epi == EPI_LSTM) return launch_fused_gemm_t<4, EPI_LSTM>(a, tile, st);
  if (gates == 4 && epi == EPI_STORE) return launch_fused_gemm_t<4, EPI_STORE>(a, tile, st);
  if (gates == 1 && epi == EPI_STORE) return launch_fused_gemm_t<1, EPI_STORE>(a, tile, st);
  if (gates == 1 && epi == EPI_LSE) return launch_fused_gemm_t<1, EPI_LSE>(a, tile, st);
  return cudaErrorInvalidValue;
}

// ------------------------------------------------------------------------------------------
// combine per-tile softmax partials.  A CTA of kLseCx x kLsePy = 8 x 32 threads handles 8 consecutive columns: thread
// (cx, py) walks over parts py, py + 32, ... of column cx (a 32-byte sector per part row), the 32 partial results per
// column meet in shared memory.  Few columns per CTA: the job is a chain of L2 round trips per thread, so what pays is
// many threads per column and many CTAs (280 columns of configuration 1: 35 CTAs of two load batches each).
// exp in float, accumulation and the final log in double.
// ------------------------------------------------------------------------------------------
constexpr int kLseCx = 8, kLsePy = 32;
__device__ __forceinline__ void lse_column_reduce(const float* __restrict__ pm, const float* __restrict__ ps,
                                                  int n_parts, size_t N, int n, bool active, float* s_m /*[kLsePy][kLseCx]*/,
                                                  double* s_s /*[kLsePy][kLseCx]*/, float* mx_out, double* sum_out) {
  // N: distance (in floats) between two parts' rows.  One pass: every thread keeps a running (max, sum) over its
  // parts, rescaling the sum when the maximum moves, and requests four parts' values before it uses any of them (the
  // loop is a chain of L2 round trips otherwise); the kLsePy (max, sum) pairs of a column meet in shared memory.
  const int cx = threadIdx.x, py = threadIdx.y;  // cx < kLseCx, py < kLsePy
  float mx = -INFINITY;
  double sum = 0.0;
  if (active) {
    for (int i0 = py; i0 < n_parts; i0 += 4 * kLsePy) {
      float m4[4], s4[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + kLsePy * u;
        const bool in = i < n_parts;
        m4[u] = in ? pm[(size_t)i * N + n] : -INFINITY;
        s4[u] = in ? ps[(size_t)i * N + n] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float m = m4[u];
        if (m == -INFINITY) continue;
        if (m > mx) {
          sum = sum * (double)expf(mx - m) + (double)s4[u];  // expf(-inf) = 0 on the first part
          mx = m;
        } else {
          sum += (double)(s4[u] * expf(m - mx));
        }
      }
    }
  }
  s_m[py * kLseCx + cx] = mx;
  s_s[py * kLseCx + cx] = sum;
  __syncthreads();
  if (py == 0) {
    float M = mx;
#pragma unroll
    for (int q = 1; q < kLsePy; ++q) M = fmaxf(M, s_m[q * kLseCx + cx]);
    double S = 0.0;
#pragma unroll
    for (int q = 0; q < kLsePy; ++q) {
      const float mq = s_m[q * kLseCx + cx];
      if (mq != -INFINITY) S += s_s[q * kLseCx + cx] * (double)expf(mq - M);
    }
    mx = M;
    sum = S;
  }
  *mx_out = mx;
  *sum_out = sum;
}
__global__ void __launch_bounds__(256) lse_combine_kernel(const float* __restrict__ pm, const float* __restrict__ ps,
                                                           const float* __restrict__ tgt, int n_parts, int n_tgt, int N,
                                                           size_t part_stride, const int* __restrict__ mask,
                                                           float* __restrict__ logp) {
  __shared__ float s_m[kLsePy * kLseCx];
  __shared__ double s_s[kLsePy * kLseCx];
  const int n = blockIdx.x * kLseCx + threadIdx.x;
  const bool in = n < N;
  const bool active = in && !(mask && mask[n] != 1);
  float mx;
  double sum;
  lse_column_reduce(pm, ps, n_parts, part_stride, n, active, s_m, s_s, &mx, &sum);
  if (threadIdx.y != 0 || !in) return;
  if (!active) { logp[n] = 0.f; return; }
  double tg = 0.0;
  for (int i = 0; i < n_tgt; ++i) tg += (double)tgt[(size_t)i * part_stride + n];
  logp[n] = (float)((tg - (double)mx) - log(sum));
}
__global__ void __launch_bounds__(256) lse_reduce_kernel(const float* __restrict__ pm, const float* __restrict__ ps,
                                                          int n_parts, int N, float* __restrict__ out_max,
                                                          float* __restrict__ out_sum) {
  __shared__ float s_m[kLsePy * kLseCx];
  __shared__ double s_s[kLsePy * kLseCx];
  const int n = blockIdx.x * kLseCx + threadIdx.x;
  const bool in = n < N;
  float mx;
  double sum;
  lse_column_reduce(pm, ps, n_parts, N, n, in, s_m, s_s, &mx, &sum);
  if (threadIdx.y != 0 || !in) return;
  out_max[n] = mx;
  out_sum[n] = (float)sum;
}
cudaError_t launch_lse_reduce(const float* pm, const float* ps, int n_parts, int N, float* out_max, float* out_sum,
                              cudaStream_t st) {
  if (N <= 0) return cudaSuccess;
  lse_reduce_kernel<<<(N + kLseCx - 1) / kLseCx, dim3(kLseCx, kLsePy), 0, st>>>(pm, ps, n_parts, N, out_max, out_sum);
  count_launch();
  return cudaGetLastError();
}
cudaError_t launch_lse_combine_shards(const float* pm, const float* ps, const float* tgt, int G, int N, const int* mask,
                                      float* logp, cudaStream_t st, size_t shard_stride) {
  if (N <= 0) return cudaSuccess;
  lse_combine_kernel<<<(N + kLseCx - 1) / kLseCx, dim3(kLseCx, kLsePy), 0, st>>>(pm, ps, tgt, G, G, N, shard_stride ? shard_stride : (size_t)N, mask,
                                                            logp);
  count_launch();
  return cudaGetLastError();
}
cudaError_t launch_lse_combine(const float* pm, const float* ps, const float* tgt, int n_parts, int N, const int* mask,
                               float* logp, cudaStream_t st) {
  if (N <= 0) return cudaSuccess;
  lse_combine_kernel<<<(N + kLseCx - 1) / kLseCx, dim3(kLseCx, kLsePy), 0, st>>>(pm, ps, tgt, n_parts, 1, N, (size_t)N, mask, logp);
  count_launch();
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// per-column top-k of log-softmax(z): one CTA per column
// ------------------------------------------------------------------------------------------
#define ZR_TOPK_MAX 33
#define ZR_TOPK_CAND 512
// Two passes over the column.  Pass 1: per-thread online (max, sum exp) and per-thread maximum; the k-th largest of
// the 256 thread maxima is a lower bound of the column's k-th largest value.  Pass 2: every element >= that bound
// becomes a candidate (a handful for real logits), and the k best candidates are picked by k block-wide argmax
// rounds.  Only if more than ZR_TOPK_CAND elements reach the bound (massive ties) the bound is raised and pass 2
// repeated.
// With part_max / part_sum (n_parts row-tile partials per column, laid out [part][N], as the GEMM epilogue writes
// them) pass 1 reads those few values instead of the whole column.  With both partials and the tiles' width
// (part_width rows per tile) pass 2 also skips every tile whose maximum is below the bound: it reads about k tiles
// of the column instead of all of it.
#define ZR_TOPK_TILES 1024
__global__ void __launch_bounds__(256) topk_logp_kernel(const float* __restrict__ z, int V, int N, int k,
                                                         const float* __restrict__ part_max,
                                                         const float* __restrict__ part_sum, int n_parts,
                                                         int part_width, float* __restrict__ val_out,
                                                         int* __restrict__ idx_out, float* __restrict__ logp_eos,
                                                         int eos_row, float* __restrict__ lse_out) {
  __shared__ int sel[ZR_TOPK_TILES];
  __shared__ int s_nsel;
  __shared__ float tmax[256];
  __shared__ float cval[ZR_TOPK_CAND];
  __shared__ int cidx[ZR_TOPK_CAND];
  __shared__ float red_m[8], red_s[8];
  __shared__ float s_M, s_logS, s_thr;
  __shared__ int s_count;
  const int col = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const float* zc = z + (size_t)col * V;
  float m = -INFINITY, s = 0.f;
  const bool sum_in_pass2 = part_max && !part_sum;  // only tile maxima are known: sum exp(v - M) during the scan
  // the value the <EOF> probability needs, requested early by the thread that will use it
  const bool has_eos = eos_row >= 0 && eos_row < V;  // the <EOF> row lies among these rows (false on other shards)
  const float z_eos = (logp_eos && tid == 32 && has_eos) ? zc[eos_row] : 0.f;
  float pmv[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // this thread's tile maxima (n_parts <= 1024)
  if (part_max && n_parts <= ZR_TOPK_TILES) {
    float psv[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int q = 0; q < 4; ++q) {  // all loads in flight together
      const int j = tid + 256 * q;
      if (j < n_parts) {
        pmv[q] = part_max[(size_t)j * N + col];
        psv[q] = part_sum ? part_sum[(size_t)j * N + col] : 0.f;
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float pm = pmv[q], ps = psv[q];
      if (pm > m) { s = s * expf(m - pm) + ps; m = pm; }
      else if (pm != -INFINITY) s += ps * expf(pm - m);
    }
  } else if (part_max) {
    for (int j = tid; j < n_parts; j += 256) {
      const float pm = part_max[(size_t)j * N + col];
      const float ps = part_sum ? part_sum[(size_t)j * N + col] : 0.f;
      if (pm > m) { s = s * expf(m - pm) + ps; m = pm; }
      else if (pm != -INFINITY) s += ps * expf(pm - m);
    }
  } else {
    for (int i = tid; i < V; i += 256) {
      const float v = zc[i];
      if (v > m) { s = s * expf(m - v) + 1.f; m = v; }
      else s += expf(v - m);
    }
  }
  tmax[tid] = m;
  float wm = m;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
  float ws = (m == -INFINITY) ? 0.f : s * expf(m - wm);
  ws = warp_sum(ws);
  if (lane == 0) { red_m[w] = wm; red_s[w] = ws; }
  if (tid == 0) { s_count = 0; s_nsel = 0; }
  __syncthreads();
  if (w == 1) {  // the normaliser, by the second warp (one warp's term per lane) while the first selects the bound
    float M = -INFINITY;
    for (int i = 0; i < 8; ++i) M = fmaxf(M, red_m[i]);
    double S = (lane < 8 && red_m[lane] != -INFINITY) ? (double)red_s[lane] * exp((double)red_m[lane] - (double)M) : 0.0;
    S += __shfl_xor_sync(0xffffffffu, S, 1);
    S += __shfl_xor_sync(0xffffffffu, S, 2);
    S += __shfl_xor_sync(0xffffffffu, S, 4);
    if (lane == 0) {
      s_M = M;
      s_logS = (float)log(S);
      if (logp_eos) logp_eos[col] = has_eos ? (z_eos - M) - s_logS : -INFINITY;
      if (lse_out) lse_out[col] = M + s_logS;
    }
  }
  // the k-th largest of the 256 thread maxima (duplicates count): k rounds of a warp-wide argmax over 8 values per
  // lane, the winner's owner dropping it
  if (w == 0) {
    float loc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) loc[i] = tmax[lane + 32 * i];
    const int rounds = k < 256 ? k : 256;
    float kth = -INFINITY;
    for (int r = 0; r < rounds; ++r) {
      float bm = loc[0];
      int bi = 0;
#pragma unroll
      for (int i = 1; i < 8; ++i)
        if (loc[i] > bm) { bm = loc[i]; bi = i; }
      float wmax = bm;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, o));
      kth = wmax;
      if (wmax == -INFINITY) break;
      const unsigned owners = __ballot_sync(0xffffffffu, bm == wmax);
      if (lane == __ffs(owners) - 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (i == bi) loc[i] = -INFINITY;
      }
    }
    if (lane == 0) s_thr = kth;
  }
  __syncthreads();
  float thr = s_thr;
  float s2 = 0.f;
  const float Mall = s_M;
  const bool vec4 = (V & 3) == 0 && ((reinterpret_cast<uintptr_t>(zc) & 15) == 0);
  const bool skip = part_max && part_sum && part_width > 0 && n_parts <= ZR_TOPK_TILES;
  if (skip) {  // the tiles that can hold one of the k largest values (at least k of them, more only on ties)
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (tid + 256 * q < n_parts && pmv[q] >= thr) sel[atomicAdd(&s_nsel, 1)] = tid + 256 * q;
    __syncthreads();
  }
  for (int attempt = 0; attempt < 4; ++attempt) {
    if (skip && vec4 && (part_width & 3) == 0) {
      const float4* z4 = reinterpret_cast<const float4*>(zc);
      const int w4 = part_width >> 2, n4 = V >> 2, tot = s_nsel * w4;
      for (int e = tid; e < tot; e += 256) {
        const int i4 = sel[e / w4] * w4 + e % w4;
        if (i4 >= n4) continue;
        const float4 v = __ldcs(z4 + i4);
        if (fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)) >= thr) {
          const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (vv[u] >= thr && vv[u] != -INFINITY) {
              const int p = atomicAdd(&s_count, 1);
              if (p < ZR_TOPK_CAND) { cval[p] = vv[u]; cidx[p] = 4 * i4 + u; }
            }
        }
      }
    } else if (skip) {
      const int tot = s_nsel * part_width;
      for (int e = tid; e < tot; e += 256) {
        const int i = sel[e / part_width] * part_width + e % part_width;
        if (i >= V) continue;
        const float v = zc[i];
        if (v >= thr && v != -INFINITY) {
          const int p = atomicAdd(&s_count, 1);
          if (p < ZR_TOPK_CAND) { cval[p] = v; cidx[p] = i; }
        }
      }
    } else if (vec4) {
      // 16-byte loads, four independent exp chains per thread
      const float4* z4 = reinterpret_cast<const float4*>(zc);
      float e0 = 0.f, e1 = 0.f, e2 = 0.f, e3 = 0.f;
      const int n4 = V >> 2;
      for (int base = tid; base < n4; base += 256 * 4) {
        float4 v[4];  // four 16-byte loads in flight per thread
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int i4 = base + q * 256;
          v[q] = i4 < n4 ? __ldcs(z4 + i4) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int i4 = base + q * 256;
          if (sum_in_pass2 && attempt == 0) {  // exp(-inf) = 0 for the padding of the last group
            e0 += expf(v[q].x - Mall); e1 += expf(v[q].y - Mall); e2 += expf(v[q].z - Mall); e3 += expf(v[q].w - Mall);
          }
          if (fmaxf(fmaxf(v[q].x, v[q].y), fmaxf(v[q].z, v[q].w)) >= thr) {
            const float vv[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
#pragma unroll
            for (int u = 0; u < 4; ++u)
              if (vv[u] >= thr && vv[u] != -INFINITY) {
                const int p = atomicAdd(&s_count, 1);
                if (p < ZR_TOPK_CAND) { cval[p] = vv[u]; cidx[p] = 4 * i4 + u; }
              }
          }
        }
      }
      s2 += (e0 + e1) + (e2 + e3);
    } else {
      for (int i = tid; i < V; i += 256) {
        const float v = zc[i];
        if (sum_in_pass2 && attempt == 0) s2 += expf(v - Mall);
        if (v >= thr && v != -INFINITY) {
          const int p = atomicAdd(&s_count, 1);
          if (p < ZR_TOPK_CAND) { cval[p] = v; cidx[p] = i; }
        }
      }
    }
    __syncthreads();
    if (s_count <= ZR_TOPK_CAND) break;
    // too many candidates (massive ties): raise the bound just above the k-th largest distinct stored value, which
    // is still a lower bound of the column's k-th largest distinct value, and collect again
    if (tid < 32) {
      float best = INFINITY;
      for (int r = 0; r < k; ++r) {
        float vmax = -INFINITY;
        for (int j = lane; j < ZR_TOPK_CAND; j += 32)
          if (cval[j] < best) vmax = fmaxf(vmax, cval[j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
        if (vmax == -INFINITY) break;
        best = vmax;
      }
      if (lane == 0) {
        s_thr = (best > thr && best != INFINITY) ? best : nextafterf(thr, INFINITY);
        s_count = 0;
      }
    }
    __syncthreads();
    thr = s_thr;
  }
  if (sum_in_pass2) {  // finish the normaliser now that the whole column has been seen
    s2 = warp_sum(s2);
    if (lane == 0) red_s[w] = s2;
    __syncthreads();
    if (tid == 0) {
      double S = 0.0;
      for (int i = 0; i < 8; ++i) S += (double)red_s[i];
      s_logS = (float)log(S);
      if (logp_eos) logp_eos[col] = has_eos ? (zc[eos_row] - s_M) - s_logS : -INFINITY;
      if (lse_out) lse_out[col] = s_M + s_logS;
    }
    __syncthreads();
  }
  const int nc = s_count < ZR_TOPK_CAND ? s_count : ZR_TOPK_CAND;
  // k rounds of argmax over the candidates (value, then lower word id) by one warp: the candidate list is short, and
  // a warp needs no block barrier between rounds
  const float M = s_M, logS = s_logS;
  if (nc <= 256) {
    // few candidates (the normal case): every candidate counts the ones that beat it and writes itself at that rank
    if (tid < nc) {
      const float v = cval[tid];
      const int id = cidx[tid];
      int rank = 0;
      for (int i = 0; i < nc; ++i) {
        const float o = cval[i];
        rank += (o > v || (o == v && cidx[i] < id)) ? 1 : 0;
      }
      if (rank < k) {
        val_out[(size_t)col * k + rank] = (v - M) - logS;
        idx_out[(size_t)col * k + rank] = id;
      }
    } else if (tid < k) {  // fewer candidates than k: the tail stays empty
      val_out[(size_t)col * k + tid] = -INFINITY;
      idx_out[(size_t)col * k + tid] = -1;
    }
    return;
  }
  if (w != 0) return;
  for (int r = 0; r < k; ++r) {
    float v = -INFINITY;
    int id = 0x7fffffff, pos = -1;
    for (int jj = lane; jj < nc; jj += 32) {
      const float cv = cval[jj];
      const int ci = cidx[jj];
      if (cv > v || (cv == v && ci < id)) { v = cv; id = ci; pos = jj; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, id, o);
      const int op = __shfl_xor_sync(0xffffffffu, pos, o);
      if (ov > v || (ov == v && oi < id)) { v = ov; id = oi; pos = op; }
    }
    if (lane == 0) {
      const bool ok = pos >= 0 && v != -INFINITY;
      val_out[(size_t)col * k + r] = ok ? (v - M) - logS : -INFINITY;
      idx_out[(size_t)col * k + r] = ok ? id : -1;
      if (pos >= 0) cval[pos] = -INFINITY;  // remove the winner
    }
    __syncwarp();
  }
}
cudaError_t launch_topk_logp(const float* logits, int V, int N, int k, float* val_out, int* idx_out, float* logp_eos,
                             cudaStream_t st, const float* part_max, const float* part_sum, int n_parts,
                             int part_width, int eos_row, float* lse_out) {
  if (N <= 0) return cudaSuccess;
  if (k < 1 || k > ZR_TOPK_MAX) return cudaErrorInvalidValue;
  topk_logp_kernel<<<N, 256, 0, st>>>(logits, V, N, k, part_max, part_sum, n_parts, part_width, val_out, idx_out,
                                      logp_eos, eos_row, lse_out);
  count_launch();
  return cudaGetLastError();
}

// Merge of G vocabulary shards' candidates.  Shard g reports, per column, its k best rows as log-probabilities under
// its OWN normaliser (val, sorted), their row numbers inside the shard (idx), the log of its normaliser (lse) and the
// <EOF> log-probability under that normaliser (-inf where the shard does not hold the row).  The global normaliser is
// log sum_g exp(lse_g); a candidate's global log-probability is val + lse_g - that.  One warp per column picks the
// k largest of the G * k candidates (ties: lower word id), sorted.
__global__ void __launch_bounds__(128) topk_merge_kernel(const float* __restrict__ val, const int* __restrict__ idx,
                                                          const float* __restrict__ lse, const float* __restrict__ eos,
                                                          const int* __restrict__ shard_lo, int G, int N, int k,
                                                          size_t cand_stride, size_t col_stride,
                                                          float* __restrict__ val_out, int* __restrict__ idx_out,
                                                          float* __restrict__ eos_out) {
  // cand_stride: words between two shards' val (idx) blocks; col_stride: words between two shards' lse (eos) blocks
  const int col = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (col >= N) return;
  float M = -INFINITY;
  for (int g = 0; g < G; ++g) M = fmaxf(M, lse[g * col_stride + col]);
  double S = 0.0;
  for (int g = 0; g < G; ++g) S += exp((double)lse[g * col_stride + col] - (double)M);
  const float LSE = M + (float)log(S);
  if (eos_out && lane == 0) {
    float e = -INFINITY;
    for (int g = 0; g < G; ++g) {
      const float eg = eos[g * col_stride + col];
      if (eg != -INFINITY) e = eg + lse[g * col_stride + col] - LSE;
    }
    eos_out[col] = e;
  }
  // candidate c = g * k + r lives in lane c % 32, register c / 32 (G * k <= 8 * 33 = 264)
  float cv[9];
  int ci[9];
#pragma unroll
  for (int q = 0; q < 9; ++q) {
    const int c = lane + 32 * q;
    cv[q] = -INFINITY;
    ci[q] = 0x7fffffff;
    if (c < G * k) {
      const int g = c / k, r = c - g * k;
      const size_t at = g * cand_stride + (size_t)col * k + r;
      const int id = idx[at];
      if (id >= 0) {
        cv[q] = val[at] + lse[g * col_stride + col] - LSE;
        ci[q] = id + shard_lo[g];
      }
    }
  }
  for (int r = 0; r < k; ++r) {
    float bv = cv[0];
    int bi = ci[0], bq = 0;
#pragma unroll
    for (int q = 1; q < 9; ++q)
      if (cv[q] > bv || (cv[q] == bv && ci[q] < bi)) { bv = cv[q]; bi = ci[q]; bq = q; }
    float wv = bv;
    int wi = bi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, wv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
      if (ov > wv || (ov == wv && oi < wi)) { wv = ov; wi = oi; }
    }
    if (lane == 0) {
      val_out[(size_t)col * k + r] = wv;
      idx_out[(size_t)col * k + r] = wv == -INFINITY ? -1 : wi;
    }
    if (bv == wv && bi == wi) {  // the winner's owner drops it (word ids are unique, so exactly one lane)
#pragma unroll
      for (int q = 0; q < 9; ++q)
        if (q == bq) { cv[q] = -INFINITY; ci[q] = 0x7fffffff; }
    }
  }
}
cudaError_t launch_topk_merge(const float* val, const int* idx, const float* lse, const float* eos, const int* shard_lo,
                              int G, int N, int k, float* val_out, int* idx_out, float* eos_out, cudaStream_t st,
                              size_t cand_stride, size_t col_stride) {
  if (N <= 0) return cudaSuccess;
  if (k < 1 || k > ZR_TOPK_MAX || G < 1 || G * k > 288) return cudaErrorInvalidValue;
  if (!cand_stride) cand_stride = (size_t)N * k;
  if (!col_stride) col_stride = (size_t)N;
  topk_merge_kernel<<<(N + 3) / 4, 128, 0, st>>>(val, idx, lse, eos, shard_lo, G, N, k, cand_stride, col_stride, val_out,
                                                 idx_out, eos_out);
  count_launch();
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// attention: window / global scores, masked softmax, context.  One CTA per target column.
// ------------------------------------------------------------------------------------------
#define ZR_ATT_MAXW 64
__global__ void __launch_bounds__(256) att_local_kernel(const AttArgs a) {
  pdl_enter();
  __shared__ float red[32];
  __shared__ float s_al[ZR_ATT_MAXW];
  __shared__ int s_slot[ZR_ATT_MAXW];
  __shared__ float s_p;
  __shared__ int s_lo, s_hi;
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5, nw = blockDim.x >> 5;
  const int H = a.H, Wn = 2 * a.D + 1, sb = b / a.cols_per_sent;
  float* c = a.c_t + (size_t)b * H;
  if (a.mask && a.mask[b] != 1) {  // create_indicies_kernel: every window slot is -1 -> context 0
    for (int i = tid; i < H; i += blockDim.x) { c[i] = 0.f; att_store_op(a, b, i, 0.f); }
    if (a.align_out) {
      const int n_out = a.align_by_pos ? a.S_max : Wn;
      for (int j = tid; j < n_out; j += blockDim.x) a.align_out[(size_t)j * a.B + b] = 0.f;
    }
    if (a.viterbi_out && tid == 0) a.viterbi_out[b] = -1;
    return;
  }
  float part = 0.f;
  for (int i = tid; i < H; i += blockDim.x) part += a.v_p[i] * a.tanh1[(size_t)b * a.ld_tq + i];
  const float tot = block_sum(part, red);
  const int len = a.len[sb], off = a.offset[sb];
  if (tid == 0) {
    const float sg = (float)(1.0 / (1.0 + exp(-1.0 * (double)tot)));
    const float pt = len * sg;
    const int ip = (int)pt;
    s_p = pt;
    s_lo = (0 > ip - a.D) ? 0 : (ip - a.D);
    s_hi = ((len - 1) < ip + a.D) ? (len - 1) : (ip + a.D);
  }
  __syncthreads();
  const int lo = s_lo, hi = s_hi;
  const float* q = a.q + (size_t)b * a.ld_tq;
  for (int j = w; j < Wn; j += nw) {
    const int pos = lo + j;
    int slot = -1;
    float sc = 0.f;
    if (pos <= hi) {
      slot = len - 1 - pos + off;
      const float* hv = a.hs + ((size_t)slot * a.B_src + sb) * H;
      for (int i = lane; i < H; i += 32) sc += hv[i] * q[i];
      sc = warp_sum(sc);
    }
    if (lane == 0) { s_al[j] = sc; s_slot[j] = slot; }
  }
  __syncthreads();
  if (tid == 0) {
    float sum = 0.f, mx = 0.f;  // the reference starts the max at 0
    for (int j = 0; j < Wn; ++j)
      if (s_slot[j] != -1 && s_al[j] > mx) mx = s_al[j];
    for (int j = 0; j < Wn; ++j) {
      if (s_slot[j] != -1) { s_al[j] = expf(s_al[j] - mx); sum += s_al[j]; }
      else s_al[j] = 0.f;
    }
    const float sigma_sq = (float)((a.D * a.D) / 4.0);
    for (int j = 0; j < Wn; ++j) {
      if (s_slot[j] != -1) {
        const float d = s_p - (float)(lo + j);
        const float gs = expf((-1.f * d * d) / (2.f * sigma_sq));
        if (sum != 0.f) s_al[j] = (s_al[j] / sum) * gs;
      }
    }
    if (a.viterbi_out) {  // only a strictly larger weight replaces the running maximum
      float best = a.viterbi_init;
      int best_pos = -1;
      for (int j = 0; j < Wn; ++j)
        if (best < s_al[j]) { best = s_al[j]; best_pos = (s_slot[j] != -1) ? lo + j : -1; }
      a.viterbi_out[b] = best_pos;
    }
  }
  __syncthreads();
  if (a.align_out) {
    if (a.align_by_pos) {
      for (int s = tid; s < a.S_max; s += blockDim.x) {
        const int j = s - lo;
        a.align_out[(size_t)s * a.B + b] = (j >= 0 && j < Wn && s <= hi) ? s_al[j] : 0.f;
      }
    } else {
      for (int j = tid; j < Wn; j += blockDim.x) a.align_out[(size_t)j * a.B + b] = s_al[j];
    }
  }
  for (int i = tid; i < H; i += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < Wn; ++j) {
      const int slot = s_slot[j];
      if (slot != -1) acc += s_al[j] * a.hs[((size_t)slot * a.B_src + sb) * H + i];
    }
    c[i] = acc;
    att_store_op(a, b, i, acc);
  }
}
// att_local_fast_body (att_device.cuh): the same arithmetic for H % 4 == 0, H <= 1024 with 16-byte loads.
__global__ void __launch_bounds__(256) att_local_fast_kernel(const AttArgs a) {
  pdl_enter();
  __shared__ __align__(16) unsigned char scratch[kAttLocalScratchBytes];
  att_local_fast_body(a, (int)blockIdx.x, (int)threadIdx.x, scratch, SyncCta());
}
cudaError_t launch_att_local(const AttArgs& a, cudaStream_t st) {
  if (a.B <= 0) return cudaSuccess;
  if (2 * a.D + 1 > ZR_ATT_MAXW) return cudaErrorInvalidValue;
  if ((a.H & 3) == 0 && a.H <= 1024 && (a.ld_tq & 3) == 0) {
    count_launch();
    return launch_chain(att_local_fast_kernel, dim3(a.B), dim3(256), 0, st, a);
  }
  count_launch();
  return launch_chain(att_local_kernel, dim3(a.B), dim3(256), 0, st, a);
}

__global__ void __launch_bounds__(256) att_global_kernel(const AttArgs a) {
  pdl_enter();
  extern __shared__ float s_sc[];  // S_max scores
  __shared__ float red[32];
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5, nw = blockDim.x >> 5;
  const int H = a.H, sb = b / a.cols_per_sent;
  float* c = a.c_t + (size_t)b * H;
  if (a.align_out)
    for (int s = tid; s < a.S_max; s += blockDim.x) a.align_out[(size_t)s * a.B + b] = 0.f;
  if (a.mask && a.mask[b] != 1) {
    for (int i = tid; i < H; i += blockDim.x) { c[i] = 0.f; att_store_op(a, b, i, 0.f); }
    if (a.viterbi_out && tid == 0) a.viterbi_out[b] = -1;
    return;
  }
  const int len = a.len[sb], off = a.offset[sb];
  const float* h = a.h_t + (size_t)b * H;
  for (int pos = w; pos < len; pos += nw) {
    const float* hv = a.hs + ((size_t)(len - 1 - pos + off) * a.B_src + sb) * H;
    float sc = 0.f;
    for (int i = lane; i < H; i += 32) sc += hv[i] * h[i];
    sc = warp_sum(sc);
    if (lane == 0) s_sc[pos] = sc;
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int pos = tid; pos < len; pos += blockDim.x) mx = fmaxf(mx, s_sc[pos]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[w] = mx;
  __syncthreads();
  mx = red[0];
  for (int i = 1; i < nw; ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float part = 0.f;
  for (int pos = tid; pos < len; pos += blockDim.x) {
    const float e = expf(s_sc[pos] - mx);
    s_sc[pos] = e;
    part += e;
  }
  const float sum = block_sum(part, red);
  const float inv = 1.0f / sum;
  if (a.align_out)
    for (int pos = tid; pos < len; pos += blockDim.x) a.align_out[(size_t)pos * a.B + b] = s_sc[pos] * inv;
  if (a.viterbi_out && tid == 0) {
    float best = a.viterbi_init;
    int best_pos = -1;
    for (int pos = 0; pos < len; ++pos)
      if (best < s_sc[pos] * inv) { best = s_sc[pos] * inv; best_pos = pos; }
    a.viterbi_out[b] = best_pos;
  }
  for (int i = tid; i < H; i += blockDim.x) {
    float acc = 0.f;
    for (int pos = 0; pos < len; ++pos)
      acc += (s_sc[pos] * inv) * a.hs[((size_t)(len - 1 - pos + off) * a.B_src + sb) * H + i];
    c[i] = acc;
    att_store_op(a, b, i, acc);
  }
}
// att_global_fast_body (att_device.cuh): single pass for H % 4 == 0, H <= 1024, one CTA of 256 threads per column.
__global__ void __launch_bounds__(256) att_global_fast_kernel(const AttArgs a) {
  pdl_enter();
  extern __shared__ __align__(16) unsigned char att_dyn_scratch[];
  att_global_fast_body(a, (int)blockIdx.x, (int)threadIdx.x, att_dyn_scratch, SyncCta());
}
cudaError_t launch_att_global(const AttArgs& a, cudaStream_t st) {
  if (a.B <= 0) return cudaSuccess;
  if ((a.H & 3) == 0 && a.H <= 1024) {
    count_launch();
    return launch_chain(att_global_fast_kernel, dim3(a.B), dim3(256), (size_t)kAttGlobalScratchBytes, st, a);
  }
  const size_t smem = sizeof(float) * (size_t)(a.S_max > 0 ? a.S_max : 1);
  if (smem > 40 * 1024) return cudaErrorInvalidValue;
  count_launch();
  return launch_chain(att_global_kernel, dim3(a.B), dim3(256), smem, st, a);
}

// ------------------------------------------------------------------------------------------
// resident-weight LSTM sequence kernel (small layers)
// ------------------------------------------------------------------------------------------
// Input-side products of ALL steps: xp[n][j] = (M_i, M_f, M_g, M_o)[:, j] . x_n for every column n = (step, sentence).
// A CTA takes 8 columns at a time (their x vectors staged in shared memory) and 128 hidden units; its 256 threads are
// two halves of the k range, each thread accumulating 4 gates x 8 columns, so that a weight value fetched from L2 is
// used 8 times and the loads of ten k values are in flight together (one column per CTA and one load per FMA made this
// launch as long as the whole recurrent loop it prepares).
constexpr int kSeqXpartMaxH = 320;
__global__ void __launch_bounds__(256) lstm_seq_xpart_kernel(const SeqArgs a) {
  __shared__ __align__(16) float xs[kSeqXpartMaxH * 8];
  __shared__ __align__(16) float red[32 * 128];
  // the sequence kernel that follows may start now: its set-up (weights into registers or shared memory, barriers)
  // needs nothing from this launch, and it waits (griddepcontrol.wait) before it reads the first product
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int H = a.H, N = a.S * a.B;
  const int tid = threadIdx.x, jt = tid & 127, half = tid >> 7;
  const int j = blockIdx.x * 128 + jt;
  const size_t HH = (size_t)H * H;
  const int k_lo = half ? H / 2 : 0, k_hi = half ? H : H / 2;
  for (int n0 = blockIdx.y * 8; n0 < N; n0 += gridDim.y * 8) {
    __syncthreads();  // the previous group's xs and red are free
    for (int c = 0; c < 8; ++c) {
      const int n = n0 + c;
      const float* x = nullptr;
      if (n < N) {
        if (a.x_seq) {
          x = a.x_seq + (size_t)n * H;
        } else {
          int id = a.ids[n];
          if (id < 0) id = 0;
          if (a.V > 0 && id >= a.V) {
            id = 0;
            if (a.err && tid == 0 && blockIdx.x == 0) atomicExch(a.err, kErrBadTokenId);
          }
          x = a.emb + (size_t)id * H;
        }
      }
      for (int k = tid; k < H; k += 256) xs[k * 8 + c] = x ? __ldg(x + k) : 0.f;
    }
    __syncthreads();
    float acc[4][8];
#pragma unroll
    for (int g = 0; g < 4; ++g)
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[g][c] = 0.f;
    if (j < H) {
#pragma unroll 10
      for (int k = k_lo; k < k_hi; ++k) {
        const size_t at = (size_t)k * H + j;
        const float w0 = __ldg(a.Mx + at), w1 = __ldg(a.Mx + HH + at), w2 = __ldg(a.Mx + 2 * HH + at), w3 = __ldg(a.Mx + 3 * HH + at);
        const float4 xa = *reinterpret_cast<const float4*>(xs + k * 8), xb = *reinterpret_cast<const float4*>(xs + k * 8 + 4);
        const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          acc[0][c] = fmaf(w0, xv[c], acc[0][c]);
          acc[1][c] = fmaf(w1, xv[c], acc[1][c]);
          acc[2][c] = fmaf(w2, xv[c], acc[2][c]);
          acc[3][c] = fmaf(w3, xv[c], acc[3][c]);
        }
      }
    }
    if (half == 1) {
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int c = 0; c < 8; ++c) red[(g * 8 + c) * 128 + jt] = acc[g][c];
    }
    __syncthreads();
    if (half == 0 && j < H) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int n = n0 + c;
        if (n < N)
          reinterpret_cast<float4*>(a.xp)[(size_t)n * H + j] =
              make_float4(acc[0][c] + red[(0 * 8 + c) * 128 + jt], acc[1][c] + red[(1 * 8 + c) * 128 + jt],
                          acc[2][c] + red[(2 * 8 + c) * 128 + jt], acc[3][c] + red[(3 * 8 + c) * 128 + jt]);
      }
    }
  }
}

__device__ __forceinline__ void seq_store_op(const SeqArgs& a, size_t n, int i, float v) {
  const size_t idx = n * a.ld_op + i;
  if (a.op_b16) reinterpret_cast<__nv_bfloat16*>(a.op_b16)[idx] = __float2bfloat16(v);
  if (a.op_h_hi) {
    const __half h = __float2half_rn(v);
    reinterpret_cast<__half*>(a.op_h_hi)[idx] = h;
    reinterpret_cast<__half*>(a.op_h_lo)[idx] = __float2half_rn((v - __half2float(h)) * 2048.0f);
  }
  if (a.op_hi) {
    unsigned u = __float_as_uint(v);
    const float hi = ((u & 0x7f800000u) == 0x7f800000u) ? v : __uint_as_float((u + 0x1000u) & 0xffffe000u);
    a.op_hi[idx] = hi;
    if (a.op_lo) a.op_lo[idx] = v - hi;
  }
}

// One cluster of C CTAs per launch.  CTA r keeps Wt[k][jl] = (Wh_i, Wh_f, Wh_g, Wh_o)[j0 + jl, k] for its Hc hidden
// units in shared memory; thread (jl, cg) owns the cell of unit j0 + jl for CPT consecutive columns.  h_{t-1} lives in
// every CTA's shared memory (hb[buf][k][column], double-buffered); after a step each thread sends its new h values
// into all C copies with st.async, and the bytes arriving complete the receiving copy's transaction barrier (see the
// exchange protocol inside).
// A thread reads its unit's four weights once per k for all of its columns, so the more columns a thread owns the
// fewer times the weight slice is read per step (CPT = 8: once for 8 columns) - and the longer its instruction
// stream; with few columns more threads win.
template <int CPT>
__global__ void __launch_bounds__(CPT >= 4 ? 256 : 1024, 1) lstm_seq_resident_kernel(const SeqArgs a, int Hc, int CG) {
  extern __shared__ __align__(16) unsigned char seq_smem[];
  const int H = a.H, B = a.B, Bp = CG * CPT;
  float4* Wt = reinterpret_cast<float4*>(seq_smem);                       // [H][Hc]
  float* hb = reinterpret_cast<float*>(seq_smem + (size_t)H * Hc * 16);   // [2][H][Bp]
  // one transaction barrier per copy of h: the bytes of a step's exchange complete it (no cluster barrier per step)
  uint64_t* hbar = reinterpret_cast<uint64_t*>(seq_smem + (size_t)H * Hc * 16 + ((2 * (size_t)H * Bp * 4 + 15) / 16) * 16);
  unsigned rank, csize;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(csize));
  const int j0 = (int)rank * Hc;
  const int nj = H - j0 < Hc ? (H - j0 > 0 ? H - j0 : 0) : Hc;  // units of this CTA
  const int tid = threadIdx.x;
  const size_t HH = (size_t)H * H;
  for (int e = tid; e < H * Hc; e += blockDim.x) {
    const int k = e / Hc, jl = e - k * Hc;
    float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
    if (jl < nj) {
      const size_t at = (size_t)k * H + j0 + jl;
      w = make_float4(__ldg(a.Wh + at), __ldg(a.Wh + HH + at), __ldg(a.Wh + 2 * HH + at), __ldg(a.Wh + 3 * HH + at));
    }
    Wt[e] = w;
  }
  for (int e = tid; e < H * Bp; e += blockDim.x) {
    const int k = e / Bp, c = e - k * Bp;
    hb[e] = c < B ? a.h0[(size_t)c * H + k] : 0.f;
    hb[(size_t)H * Bp + e] = 0.f;
  }
  if (tid == 0) {
    const uint32_t b0 = (uint32_t)__cvta_generic_to_shared(hbar);
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b0));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b0 + 8));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const int jl = tid % Hc, cg = tid / Hc;
  const bool active = cg < CG && jl < nj;
  const int j = j0 + jl, cb = cg * CPT;  // unit and first column of this thread
  float cst[CPT];
  float bi = 0.f, bf = 0.f, bg = 0.f, bo = 0.f;
#pragma unroll
  for (int c = 0; c < CPT; ++c) cst[c] = (active && cb + c < B) ? a.c0[(size_t)(cb + c) * H + j] : 0.f;
  if (active) { bi = a.bias[j]; bf = a.bias[H + j]; bg = a.bias[2 * H + j]; bo = a.bias[3 * H + j]; }
  // every copy of h_0 is in place before anybody reads or overwrites one
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  uint32_t hb_remote[8], bar_remote[8];
  const uint32_t bar_local = (uint32_t)__cvta_generic_to_shared(hbar);
  {
    const uint32_t local = (uint32_t)__cvta_generic_to_shared(hb);
    for (unsigned q = 0; q < 8; ++q) {
      uint32_t r = local, rb = bar_local;
      if (q < csize) {
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(q));
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rb) : "r"(bar_local), "r"(q));
      }
      hb_remote[q] = r;
      bar_remote[q] = rb;
    }
  }
  // Exchange protocol.  Step t reads h_t from copy t & 1 and sends h_(t+1) into copy (t + 1) & 1 of EVERY CTA of the
  // cluster (its own included) with st.async, whose bytes count on the receiver's barrier of that copy; a step
  // starts when the barrier of its copy has all H * B values.  Two copies suffice: a CTA sends h_(t+2) into the copy
  // that held h_t only after it has received every h_(t+1), and each of those was sent after its sender's last read
  // of h_t.  The wait is bounded; a thread that gives up sets the error word and leaves (so do all others, in turn).
  const uint32_t step_bytes = (uint32_t)H * (uint32_t)B * 4u;
  bool alive = true;
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the input-side products (the launch before this one) are complete
  for (int t = 0; t < a.S && alive; ++t) {
    // with the last step under way the next launch may be scheduled: it sets itself up beside this kernel's few CTAs
    // and waits for this grid to complete before it touches its results
    if (t == a.S - 1) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const float* hcur = hb + (size_t)(t & 1) * H * Bp;
    const size_t nb = (size_t)t * B;
    if (tid == 0 && nj > 0 && t + 1 < a.S)  // (a CTA without units neither waits nor is sent to: it must not arm)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_local + 8u * ((t + 1) & 1)), "r"(step_bytes)
                   : "memory");
    float4 xp[CPT];
    float mk[CPT];
    if (active) {  // the inputs of the epilogue do not depend on the recurrence: request them before the k loop
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const bool okc = cb + c < B;
        xp[c] = okc ? reinterpret_cast<const float4*>(a.xp)[(nb + cb + c) * H + j] : make_float4(0.f, 0.f, 0.f, 0.f);
        mk[c] = okc ? (float)a.mask[nb + cb + c] : 0.f;
      }
    }
    float ai[CPT], af[CPT], ag[CPT], ao[CPT], hnew[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) ai[c] = af[c] = ag[c] = ao[c] = hnew[c] = 0.f;
    if (active && t > 0) {  // h_t complete in this CTA's copy?
      const uint32_t bar = bar_local + 8u * (t & 1), parity = (uint32_t)((t - 1) >> 1) & 1u;
      const long long t0 = clock64();
      for (int spins = 0;; ++spins) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) break;
        if ((spins & 63) == 63 && clock64() - t0 > 400000000LL) {
          if (a.err) atomicExch(a.err, 88);
          alive = false;
          break;
        }
      }
    }
    if (active && alive) {
      const float4* wp = Wt + jl;
      const float* hp = hcur + cb;
#pragma unroll 4
      for (int k = 0; k < H; ++k) {
        const float4 w = wp[(size_t)k * Hc];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          const float hv = hp[(size_t)k * Bp + c];
          ai[c] = fmaf(w.x, hv, ai[c]);
          af[c] = fmaf(w.y, hv, af[c]);
          ag[c] = fmaf(w.z, hv, ag[c]);
          ao[c] = fmaf(w.w, hv, ao[c]);
        }
      }
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        if (cb + c < B) {
          const float gi = sigmoidf_acc(ai[c] + xp[c].x + bi);
          const float gf = sigmoidf_acc(af[c] + xp[c].y + bf);
          const float gg = tanhf(ag[c] + xp[c].z + bg);
          const float go = sigmoidf_acc(ao[c] + xp[c].w + bo);
          const float cn = gf * cst[c] + gi * gg;
          const float hn = go * tanhf(cn) * mk[c];
          cst[c] = cn * mk[c];
          hnew[c] = hn;
          // the new h into every CTA's copy of the other buffer (nobody reads the last step's)
          if (t + 1 < a.S) {
            const uint32_t off = (uint32_t)((((size_t)((t + 1) & 1) * H + j) * Bp + cb + c) * 4);
            const uint32_t boff = 8u * ((t + 1) & 1);
            for (unsigned q = 0; q < csize && (int)q * Hc < H; ++q)
              asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(hb_remote[q] + off),
                           "r"(__float_as_uint(hn)), "r"(bar_remote[q] + boff)
                           : "memory");
          }
        }
      }
      // the copies for the consumers outside the kernel, off the step's critical path
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        if (cb + c < B) {
          const size_t n = nb + cb + c;
          a.h_seq[n * H + j] = hnew[c];
          seq_store_op(a, n, j, hnew[c]);
        }
      }
    }
  }
  // no CTA leaves while a peer may still write into its shared memory or wait for its bytes
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (active)
#pragma unroll
    for (int c = 0; c < CPT; ++c)
      if (cb + c < B) a.c_out[(size_t)(cb + c) * H + j] = cst[c];
}

// The same time loop for the narrowest case (at most 8 columns, 64 <= H <= 128: configuration 1), with the recurrent
// weights in REGISTERS and a warp per hidden unit.  In the kernel above a step is one long dependent instruction
// stream per thread (a thousand instructions at one warp per scheduler: every stall is exposed), and every thread
// re-reads its unit's weights from shared memory at every k.  Here lane s of a unit's warp keeps the unit's 4 x 4
// weights of k = s, s + 32, s + 64, s + 96 in registers for the whole sequence, reads h_t[k][0..7] (32 bytes) and
// accumulates all 8 columns: 128 FMAs per lane and step.  A 31-shuffle butterfly leaves lane s with gate s / 8 of
// column s % 8; lanes 0..7 fetch their column's other three gates, do the gate math, keep c, and send h.  Thirteen
// to sixteen warps per CTA hide each other's latencies.  Cluster of 8 CTAs, exchange and barriers as above.
__global__ void __launch_bounds__(512, 1) lstm_seq_reg_kernel(const SeqArgs a, int Hc) {
  extern __shared__ __align__(16) unsigned char seq_smem[];
  constexpr int KI = 4, Bp = 8;
  const int H = a.H, B = a.B;
  float* hb = reinterpret_cast<float*>(seq_smem);                               // [2][H][8]
  uint64_t* hbar = reinterpret_cast<uint64_t*>(seq_smem + 2 * (size_t)H * Bp * 4);
  unsigned rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int tid = threadIdx.x, s = tid & 31, jl = tid >> 5;
  const int j0 = (int)rank * Hc;
  const int nj = H - j0 < Hc ? (H - j0 > 0 ? H - j0 : 0) : Hc;
  const bool active = jl < nj;  // per warp
  const int j = j0 + jl;
  // CTAs of the cluster that own hidden units.  The others (a cluster larger than H / Hc) take no part in the
  // exchange: nobody sends to them, and they must not arm their barriers (a thread that arrives step after step on a
  // barrier nobody completes overflows its arrival count).
  const unsigned n_recv = (unsigned)((H + Hc - 1) / Hc);
  for (int e = tid; e < H * Bp; e += blockDim.x) {
    const int k = e >> 3, c = e & 7;
    hb[e] = c < B ? a.h0[(size_t)c * H + k] : 0.f;
    hb[(size_t)H * Bp + e] = 0.f;
  }
  if (tid == 0) {
    const uint32_t b0 = (uint32_t)__cvta_generic_to_shared(hbar);
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b0));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b0 + 8));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  float w[4][KI];
  const size_t HH = (size_t)H * H;
#pragma unroll
  for (int i = 0; i < KI; ++i) {
    const int k = i * 32 + s;
    const bool in = active && k < H;
    const size_t at = in ? (size_t)k * H + j : 0;
#pragma unroll
    for (int g = 0; g < 4; ++g) w[g][i] = in ? __ldg(a.Wh + g * HH + at) : 0.f;
  }
  const bool col = active && s < B;  // this lane finishes column s of unit j
  float cst = col ? a.c0[(size_t)s * H + j] : 0.f;
  float bi = 0.f, bf = 0.f, bg = 0.f, bo = 0.f;
  if (col) { bi = a.bias[j]; bf = a.bias[H + j]; bg = a.bias[2 * H + j]; bo = a.bias[3 * H + j]; }
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  const uint32_t bar_local = (uint32_t)__cvta_generic_to_shared(hbar);
  const uint32_t hb_local = (uint32_t)__cvta_generic_to_shared(hb);
  const uint32_t step_bytes = (uint32_t)H * (uint32_t)B * 4u;
  bool alive = true;
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the input-side products (the launch before this one) are complete
  for (int t = 0; t < a.S && alive; ++t) {
    // with the last step under way the next launch may be scheduled: it sets itself up beside this kernel's few CTAs
    // and waits for this grid to complete before it touches its results
    if (t == a.S - 1) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const float* hcur = hb + (size_t)(t & 1) * H * Bp;
    const size_t nb = (size_t)t * B;
    if (tid == 0 && nj > 0 && t + 1 < a.S)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_local + 8u * ((t + 1) & 1)), "r"(step_bytes)
                   : "memory");
    float4 xp = make_float4(0.f, 0.f, 0.f, 0.f);
    float mk = 0.f;
    if (col) {
      xp = reinterpret_cast<const float4*>(a.xp)[(nb + s) * H + j];
      mk = (float)a.mask[nb + s];
    }
    if (active && t > 0) {
      const uint32_t bar = bar_local + 8u * (t & 1), parity = (uint32_t)((t - 1) >> 1) & 1u;
      const long long t0 = clock64();
      for (int spins = 0;; ++spins) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) break;
        if ((spins & 63) == 63 && clock64() - t0 > 400000000LL) {
          if (a.err) atomicExch(a.err, 88);
          alive = false;
          break;
        }
      }
      alive = __all_sync(0xffffffffu, alive);  // a warp gives up as a whole
    }
    if (active && alive) {
      float acc[4][8];
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[g][c] = 0.f;
#pragma unroll
      for (int i = 0; i < KI; ++i) {
        const int k = i * 32 + s;
        if (k < H) {
          const float4* h4 = reinterpret_cast<const float4*>(hcur + (size_t)k * Bp);
          const float4 ha = h4[0], hc = h4[1];
          const float hv[8] = {ha.x, ha.y, ha.z, ha.w, hc.x, hc.y, hc.z, hc.w};
#pragma unroll
          for (int g = 0; g < 4; ++g)
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[g][c] = fmaf(w[g][i], hv[c], acc[g][c]);
        }
      }
      // butterfly over the warp: value index g * 8 + c; every round a lane keeps the half selected by one bit of its id
      float v16[16], v8[8], v4[4], v2[2], v1;
      {
        const bool up = (s & 16) != 0;
#pragma unroll
        for (int x = 0; x < 16; ++x) {
          const float lo = acc[x >> 3][x & 7], hi = acc[2 + (x >> 3)][x & 7];
          v16[x] = (up ? hi : lo) + __shfl_xor_sync(0xffffffffu, up ? lo : hi, 16);
        }
      }
      {
        const bool up = (s & 8) != 0;
#pragma unroll
        for (int x = 0; x < 8; ++x) v8[x] = (up ? v16[8 + x] : v16[x]) + __shfl_xor_sync(0xffffffffu, up ? v16[x] : v16[8 + x], 8);
      }
      {
        const bool up = (s & 4) != 0;
#pragma unroll
        for (int x = 0; x < 4; ++x) v4[x] = (up ? v8[4 + x] : v8[x]) + __shfl_xor_sync(0xffffffffu, up ? v8[x] : v8[4 + x], 4);
      }
      {
        const bool up = (s & 2) != 0;
#pragma unroll
        for (int x = 0; x < 2; ++x) v2[x] = (up ? v4[2 + x] : v4[x]) + __shfl_xor_sync(0xffffffffu, up ? v4[x] : v4[2 + x], 2);
      }
      {
        const bool up = (s & 1) != 0;
        v1 = (up ? v2[1] : v2[0]) + __shfl_xor_sync(0xffffffffu, up ? v2[0] : v2[1], 1);
      }
      // lane s now holds gate s >> 3 of column s & 7; lanes 0..7 collect their column's four gates
      const int c8 = s & 7;
      const float si = __shfl_sync(0xffffffffu, v1, c8), sf = __shfl_sync(0xffffffffu, v1, 8 + c8);
      const float sg = __shfl_sync(0xffffffffu, v1, 16 + c8), so = __shfl_sync(0xffffffffu, v1, 24 + c8);
      if (col) {
        const float gi = sigmoidf_acc(si + xp.x + bi);
        const float gf = sigmoidf_acc(sf + xp.y + bf);
        const float gg = tanhf(sg + xp.z + bg);
        const float go = sigmoidf_acc(so + xp.w + bo);
        const float cn = gf * cst + gi * gg;
        const float hn = go * tanhf(cn) * mk;
        cst = cn * mk;
        if (t + 1 < a.S) {
          const uint32_t off = (uint32_t)((((size_t)((t + 1) & 1) * H + j) * Bp + s) * 4);
          const uint32_t boff = 8u * ((t + 1) & 1);
#pragma unroll
          for (unsigned q = 0; q < 16; ++q) {
            if (q < n_recv) {
              uint32_t ra, rb;
              asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(hb_local + off), "r"(q));
              asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rb) : "r"(bar_local + boff), "r"(q));
              asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(ra),
                           "r"(__float_as_uint(hn)), "r"(rb)
                           : "memory");
            }
          }
        }
        const size_t n = nb + s;
        a.h_seq[n * H + j] = hn;
        seq_store_op(a, n, j, hn);
      }
    }
  }
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (col) a.c_out[(size_t)s * H + j] = cst;
}

namespace {
struct SeqPlan { int C, Hc, CG, CPT, threads; size_t smem; };
bool seq_plan(int H, int B, SeqPlan* p) {
  if (H < 1 || H > kSeqXpartMaxH || B < 1 || B > 32) return false;
  // A step is a chain of short dependent stages (matrix-vector product, gate math, exchange), so what pays is
  // parallelism: the largest cluster that leaves every CTA a few hidden units, and one column per thread as long as
  // the block holds that many threads (measured at H = 100, B = 8: 8 CTAs x 1 column per thread 3.7 us per step,
  // 1 CTA x 8 columns per thread 9.7 us).
  static const int force_cpt = std::getenv("ZRNN_SEQ_CPT") ? std::atoi(std::getenv("ZRNN_SEQ_CPT")) : 0;
  static const int force_c = std::getenv("ZRNN_SEQ_C") ? std::atoi(std::getenv("ZRNN_SEQ_C")) : 0;
  int C = 8;
  while (C > 1 && (H + C - 1) / C < 8) C /= 2;
  if (force_c == 1 || force_c == 2 || force_c == 4 || force_c == 8) C = force_c;
  for (; C <= 8; C *= 2) {
    const int Hc = (H + C - 1) / C;
    for (int CPT = 1; CPT <= 8; CPT *= 2) {
      if (force_cpt && CPT != force_cpt) continue;
      const int CG = (B + CPT - 1) / CPT;
      const int threads = (Hc * CG + 31) / 32 * 32;
      const size_t smem = (size_t)H * Hc * 16 + (2 * (size_t)H * CG * CPT * 4 + 15) / 16 * 16 + 16;
      if (threads <= (CPT >= 4 ? 256 : 1024) && smem <= 200 * 1024) {
        *p = SeqPlan{C, Hc, CG, CPT, threads, smem};
        return true;
      }
    }
  }
  return false;
}
template <int CPT>
cudaError_t launch_seq_t(const SeqArgs& a, const SeqPlan& pl, cudaStream_t st) {
  static bool configured[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(lstm_seq_resident_kernel<CPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(lstm_seq_resident_kernel<CPT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(pl.C);
  cfg.blockDim = dim3(pl.threads);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = pl.C;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl ? 2 : 1;
  count_launch();
  return cudaLaunchKernelEx(&cfg, lstm_seq_resident_kernel<CPT>, a, pl.Hc, pl.CG);
}
}  // namespace

// the register-weight variant: 8 columns at most, 8 CTAs of at most 16 units (one warp each), 4 k values per lane
static bool seq_reg_fits(int H, int B) {
  static const bool off = std::getenv("ZRNN_SEQ_NO_REG") != nullptr;
  return !off && B <= 8 && H >= 64 && H <= 128;
}
bool lstm_seq_resident_supported(int H, int B) {
  SeqPlan pl;
  return seq_plan(H, B, &pl);
}
cudaError_t launch_lstm_seq_resident(const SeqArgs& a, cudaStream_t st) {
  SeqPlan pl;
  if (!seq_plan(a.H, a.B, &pl) || a.S < 1) return cudaErrorInvalidValue;
  const int N = a.S * a.B, groups = (N + 7) / 8;
  if (a.H > kSeqXpartMaxH) return cudaErrorInvalidValue;
  dim3 grid((a.H + 127) / 128, groups > 1024 ? 1024 : groups);
  lstm_seq_xpart_kernel<<<grid, 256, 0, st>>>(a);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (seq_reg_fits(a.H, a.B)) {
    // a cluster of 16 CTAs (non-portable size) where the device schedules one, else 8: half the warps per SM
    static int cluster_size[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 2 : 1;
    cfg.dynamicSmemBytes = 2 * (size_t)a.H * 8 * 4 + 16;
    cfg.stream = st;
    if (cluster_size[dev] == 0) {
      cluster_size[dev] = 8;
      static const bool no16 = std::getenv("ZRNN_SEQ_NO_C16") != nullptr;
      if (!no16 && cudaFuncSetAttribute(lstm_seq_reg_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
        const int Hc16 = (a.H + 15) / 16;
        cfg.gridDim = dim3(16);
        cfg.blockDim = dim3(32 * Hc16);
        attr[0].val.clusterDim.x = 16;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, lstm_seq_reg_kernel, &cfg) == cudaSuccess && n >= 1) cluster_size[dev] = 16;
      }
      (void)cudaGetLastError();
    }
    const int C = cluster_size[dev], Hc = (a.H + C - 1) / C;
    cfg.gridDim = dim3(C);
    cfg.blockDim = dim3(32 * Hc);
    attr[0].val.clusterDim.x = C;
    count_launch();
    return cudaLaunchKernelEx(&cfg, lstm_seq_reg_kernel, a, Hc);
  }
  switch (pl.CPT) {
    case 1: return launch_seq_t<1>(a, pl, st);
    case 2: return launch_seq_t<2>(a, pl, st);
    case 4: return launch_seq_t<4>(a, pl, st);
    case 8: return launch_seq_t<8>(a, pl, st);
  }
  return cudaErrorInvalidValue;
}

// ------------------------------------------------------------------------------------------
// ensemble: log of the mean of K softmax distributions, one CTA per column
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ensemble_logmean_kernel(const EnsembleArgs a) {
  __shared__ float red[32];
  __shared__ float s_max[ZR_ENSEMBLE_MAX], s_inv[ZR_ENSEMBLE_MAX];
  const int n = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5, nw = blockDim.x >> 5;
  const size_t col = (size_t)n * a.V;
  for (int k = 0; k < a.K; ++k) {
    const float* z = a.logits[k] + col;
    float mx = -INFINITY;
    for (int v = tid; v < a.V; v += blockDim.x) mx = fmaxf(mx, z[v]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[w] = mx;
    __syncthreads();
    mx = red[0];
    for (int i = 1; i < nw; ++i) mx = fmaxf(mx, red[i]);
    __syncthreads();
    float part = 0.f;
    for (int v = tid; v < a.V; v += blockDim.x) part += expf(z[v] - mx);
    const float sum = block_sum(part, red);
    if (tid == 0) { s_max[k] = mx; s_inv[k] = 1.0f / (sum * (float)a.K); }
    __syncthreads();
  }
  for (int v = tid; v < a.V; v += blockDim.x) {
    float p = 0.f;
    for (int k = 0; k < a.K; ++k) p += expf(a.logits[k][col + v] - s_max[k]) * s_inv[k];
    a.out[col + v] = logf(p);
  }
}
__global__ void ensemble_viterbi_kernel(const EnsembleVitArgs a) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= a.N) return;
  int smax = 0;
  for (int k = 0; k < a.K; ++k) smax = a.S_max[k] > smax ? a.S_max[k] : smax;
  float best = 0.f;
  int best_pos = -1;
  for (int s = 0; s < smax; ++s) {
    float sum = 0.f;
    for (int k = 0; k < a.K; ++k)
      if (s < a.S_max[k]) sum += a.align[k][(size_t)s * a.N + n];
    if (sum > best) { best = sum; best_pos = s; }
  }
  a.viterbi_out[n] = best_pos;
}
cudaError_t launch_ensemble_viterbi(const EnsembleVitArgs& a, cudaStream_t st) {
  if (a.N <= 0) return cudaSuccess;
  if (a.K < 1 || a.K > ZR_ENSEMBLE_MAX) return cudaErrorInvalidValue;
  ensemble_viterbi_kernel<<<(a.N + 127) / 128, 128, 0, st>>>(a);
  count_launch();
  return cudaGetLastError();
}
cudaError_t launch_ensemble_logmean(const EnsembleArgs& a, cudaStream_t st) {
  if (a.N <= 0) return cudaSuccess;
  if (a.K < 1 || a.K > ZR_ENSEMBLE_MAX) return cudaErrorInvalidValue;
  ensemble_logmean_kernel<<<a.N, 256, 0, st>>>(a);
  count_launch();
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// beam bookkeeping, one CTA per sentence
// ------------------------------------------------------------------------------------------
__global__ void beam_init_kernel(const BeamArgs a) {
  const int s = blockIdx.x, tid = threadIdx.x;
  const size_t rowbase = (size_t)s * a.beam * a.Lmax;
  for (int i = tid; i < a.beam * a.Lmax; i += blockDim.x) { a.top_sent[rowbase + i] = 0; a.top_tmp[rowbase + i] = 0; }
  if (a.vit_rows) {
    for (int i = tid; i < a.beam * a.Lmax; i += blockDim.x) { a.vit_rows[rowbase + i] = -20; a.vit_tmp[rowbase + i] = -20; }
    for (int i = tid; i < a.k_best * a.Lmax; i += blockDim.x) a.best_align[(size_t)s * a.k_best * a.Lmax + i] = -1;
  }
  for (int i = tid; i < a.beam; i += blockDim.x) {
    a.scores[s * a.beam + i] = 0.f;
    a.cur_ids[s * a.beam + i] = 0;
    a.col_map[s * a.beam + i] = s * a.beam + i;
  }
  for (int i = tid; i < a.k_best * a.Lmax; i += blockDim.x) a.best_ids[(size_t)s * a.k_best * a.Lmax + i] = -1;
  for (int i = tid; i < a.k_best; i += blockDim.x) { a.best_len[s * a.k_best + i] = 0; a.best_score[s * a.k_best + i] = 0.f; }
}
cudaError_t launch_beam_init(const BeamArgs& a, cudaStream_t st) {
  if (a.n_sent <= 0) return cudaSuccess;
  beam_init_kernel<<<a.n_sent, 128, 0, st>>>(a);
  count_launch();
  return cudaGetLastError();
}

// insert (prefix of `row` up to position last_pos, then <EOF>) with `score` into the sentence's k-best list
// vrow / last_align: the alignments stored with the prefix and the one of the step that produced <EOF> (tracking on)
__device__ void beam_insert_hyp(const BeamArgs& a, int s, const int* row, int last_pos, float score, const int* vrow,
                                int last_align) {
  const int len = last_pos + 2;
  const float ratio = ((float)len) / (float)a.src_len[s];
  if (!(ratio > a.min_ratio)) return;
  int* ids = a.best_ids + (size_t)s * a.k_best * a.Lmax;
  int* lens = a.best_len + s * a.k_best;
  float* sc = a.best_score + s * a.k_best;
  int pos = 0;
  while (pos < a.k_best && lens[pos] != 0 && !(score > sc[pos])) ++pos;
  if (pos >= a.k_best) return;
  int* al = a.best_align ? a.best_align + (size_t)s * a.k_best * a.Lmax : nullptr;
  for (int j = a.k_best - 1; j > pos; --j) {
    if (lens[j - 1] == 0) continue;
    for (int i = 0; i < a.Lmax; ++i) ids[(size_t)j * a.Lmax + i] = ids[(size_t)(j - 1) * a.Lmax + i];
    if (al)
      for (int i = 0; i < a.Lmax; ++i) al[(size_t)j * a.Lmax + i] = al[(size_t)(j - 1) * a.Lmax + i];
    lens[j] = lens[j - 1];
    sc[j] = sc[j - 1];
  }
  for (int i = 0; i < a.Lmax; ++i) ids[(size_t)pos * a.Lmax + i] = (i <= last_pos) ? row[i] : (i == last_pos + 1 ? 1 : -1);
  if (al)
    for (int i = 0; i < a.Lmax; ++i)
      al[(size_t)pos * a.Lmax + i] = (i <= last_pos) ? vrow[i] : (i == last_pos + 1 ? last_align : -1);
  lens[pos] = len;
  sc[pos] = score;
}

// NL: candidates per lane of the selecting warp: 8 covers beam * (beam + 1) <= 256 (beam <= 15), 33 covers beam <= 32
template <int NL>
__global__ void __launch_bounds__(256) beam_step_kernel(const BeamArgs a) {
  __shared__ float cv[32 * NL];
  __shared__ int ci[32 * NL];
  __shared__ int n_chg[ZR_BEAM_MAX], n_cur[ZR_BEAM_MAX];
  __shared__ float n_sc[ZR_BEAM_MAX];
  const int s = blockIdx.x, tid = threadIdx.x, beam = a.beam, kc = a.k_cand, t = a.step;
  const int base = s * beam;
  const int max_steps = a.max_steps[s];
  int* rows = a.top_sent + (size_t)base * a.Lmax;
  int* tmp = a.top_tmp + (size_t)base * a.Lmax;
  int* vrows = a.vit_rows ? a.vit_rows + (size_t)base * a.Lmax : nullptr;
  int* vtmp = a.vit_rows ? a.vit_tmp + (size_t)base * a.Lmax : nullptr;
  if (t > max_steps) {
    if (tid < beam) a.col_map[base + tid] = base + tid;
    return;
  }
  if (t == max_steps) {  // finish_current_hypotheses
    if (tid == 0)
      for (int i = 0; i < beam; ++i) {
        if (a.cur_ids[base + i] == -1) continue;
        const float sc = a.scores[base + i] + (a.logp_eos[base + i] + a.penalty);
        beam_insert_hyp(a, s, rows + (size_t)i * a.Lmax, t, sc, vrows ? vrows + (size_t)i * a.Lmax : nullptr,
                        vrows ? a.viterbi[base + i] : -1);
      }
    if (tid < beam) a.col_map[base + tid] = base + tid;
    return;
  }
  // ---- expand
  // live columns: the leading ones whose current word is set (one load per lane, not a chain of dependent ones)
  int ncols = (t == 0) ? 1 : beam;
  {
    const int l = tid & 31;
    const bool dead = l < ncols && a.cur_ids[base + l] == -1;
    const unsigned db = __ballot_sync(0xffffffffu, dead);
    if (db) ncols = __ffs(db) - 1;
  }
  for (int c = tid; c < 32 * NL; c += 256) {
    const int i = c / kc, r = c % kc;
    float v = -INFINITY;
    int wd = -1;
    if (i < ncols) {
      const float lp = a.cand_val[(size_t)(base + i) * kc + r];
      wd = a.cand_idx[(size_t)(base + i) * kc + r];
      if (wd >= 0 && lp != -INFINITY) v = lp + a.scores[base + i];
    }
    cv[c] = v;   // candidate c = beam column * kc + candidate rank
    ci[c] = wd;  // its word, kept on chip: the selection below reads one per pick
  }
  __syncthreads();
  // One warp walks the candidates in descending score (the lower candidate index wins a tie) until the beam is full:
  // a warp-wide argmax per pick, the winner's owner dropping it.
  if (tid < 32) {
    const int lane = tid;
    float loc[NL];
#pragma unroll
    for (int j = 0; j < NL; ++j) loc[j] = cv[lane + 32 * j];
    int filled = 0;
    while (filled < beam) {
      float bv = loc[0];
      int bj = 0;
#pragma unroll
      for (int j = 1; j < NL; ++j)
        if (loc[j] > bv) { bv = loc[j]; bj = j; }
      int bidx = lane + 32 * bj;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
        if (ov > bv || (ov == bv && oi < bidx)) { bv = ov; bidx = oi; }
      }
      if (bv == -INFINITY) {  // no candidate left: the remaining slots stay empty
        if (lane == 0)
          for (; filled < beam; ++filled) { n_cur[filled] = -1; n_chg[filled] = 0; n_sc[filled] = 0.f; }
        break;
      }
      if ((bidx & 31) == lane) {
#pragma unroll
        for (int j = 0; j < NL; ++j)
          if (j == (bidx >> 5)) loc[j] = -INFINITY;
      }
      const int i = bidx / kc;
      const int wd = ci[bidx];
      if (wd == 0) continue;  // <START> is never extended
      if (wd == 1) {          // <EOF>: finished hypothesis, does not take a slot
        if (lane == 0)
          beam_insert_hyp(a, s, rows + (size_t)i * a.Lmax, t, bv + a.penalty, vrows ? vrows + (size_t)i * a.Lmax : nullptr,
                          vrows ? a.viterbi[base + i] : -1);
        __syncwarp();
      } else {
        if (lane == 0) { n_cur[filled] = wd; n_chg[filled] = i; n_sc[filled] = bv + a.penalty; }
        ++filled;
      }
    }
  }
  __syncthreads();
  // the surviving hypotheses' rows go to the other row buffer, which the host makes the current one for the next step
  for (int e = tid; e < beam * a.Lmax; e += blockDim.x) {
    const int f = e / a.Lmax, i = e % a.Lmax;
    int v = rows[(size_t)n_chg[f] * a.Lmax + i];
    if (i == t + 1) v = (n_cur[f] == -1) ? 0 : n_cur[f];
    tmp[e] = v;
    if (vrows) {
      int al = vrows[(size_t)n_chg[f] * a.Lmax + i];
      if (i == t + 1 && n_cur[f] != -1) al = a.viterbi[base + n_chg[f]];
      vtmp[e] = al;
    }
  }
  if (tid < beam) {
    a.cur_ids[base + tid] = n_cur[tid];
    a.col_map[base + tid] = base + n_chg[tid];
    a.scores[base + tid] = n_sc[tid];
  }
}
cudaError_t launch_beam_step(const BeamArgs& a, cudaStream_t st) {
  if (a.n_sent <= 0) return cudaSuccess;
  if (a.beam < 1 || a.beam > ZR_BEAM_MAX || a.k_cand > ZR_BEAM_MAX + 1 || a.beam * a.k_cand > 32 * 33) return cudaErrorInvalidValue;
  if (a.beam * a.k_cand <= 256) beam_step_kernel<8><<<a.n_sent, 256, 0, st>>>(a);
  else beam_step_kernel<33><<<a.n_sent, 256, 0, st>>>(a);
  count_launch();
  return cudaGetLastError();
}

}  // namespace zrnn
