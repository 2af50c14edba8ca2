// tcgen05 / TMEM / TMA GEMM kernels for sm_100a.  See tc_gemm.cuh for the operand convention.
//
// CTA = 6 warps: warps 0-3 run the epilogue (one TMEM lane quadrant each), warp 4 is the TMA producer,
// warp 5 owns the TMEM allocation and issues tcgen05.mma.  A ring of shared-memory stages is guarded by
// full/empty mbarriers; every wait is bounded (about a second of SM clock) and reports through p.err
// instead of spinning forever.
#include "tc_gemm.cuh"

#include <cstdint>
#include <cstring>

#include "kernels.cuh"

namespace zrnn {
namespace {

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Gives up after ~2e9 SM cycles or as soon as another role has given up (*abort_flag != 0).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > 2000000000LL) {
        *abort_flag = 1;
        if (err) atomicExch(err, code);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// K-major operand tile, 128-byte rows, SWIZZLE_128B, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major), bits [16,30)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                    // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                    // layout type SWIZZLE_128B
  return d;
}
// instruction descriptor: D = f32, A/B format fmt (1 = bf16, 2 = tf32), both K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, uint32_t n) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}
template <int KIND_TF32>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  if (KIND_TF32) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        :
        : "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        :
        : "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
  }
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float* v) {
  uint32_t r0, r1, r2, r3, r4, r5, r6, r7;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3), "=r"(r4), "=r"(r5), "=r"(r6), "=r"(r7)
               : "r"(taddr));
  v[0] = __uint_as_float(r0); v[1] = __uint_as_float(r1); v[2] = __uint_as_float(r2); v[3] = __uint_as_float(r3);
  v[4] = __uint_as_float(r4); v[5] = __uint_as_float(r5); v[6] = __uint_as_float(r6); v[7] = __uint_as_float(r7);
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ float sigmoid_acc(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float tf32_round_dev(float x) {
  uint32_t u = __float_as_uint(x);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;
  return __uint_as_float((u + 0x1000u) & 0xffffe000u);
}
// write the A-operand copies (for the next GEMM) of value v at element index idx
__device__ __forceinline__ void store_operand(const TcParams& p, size_t idx, float v) {
  if (p.op_b16) p.op_b16[idx] = __float2bfloat16(v);
  if (p.op_hi) {
    const float hi = tf32_round_dev(v);
    p.op_hi[idx] = hi;
    if (p.op_lo) p.op_lo[idx] = v - hi;
  }
}

constexpr int kABytes = 128 * 128;  // A tile: 128 rows x 128-byte k-block
__host__ __device__ constexpr int stage_bytes(int BN, int mode) { return (mode == TC_TF32X3 ? 2 : 1) * (kABytes + BN * 128); }
__host__ __device__ constexpr int num_stages(int BN, int mode) {
  int s = (200 * 1024) / stage_bytes(BN, mode);
  return s > 8 ? 8 : s;
}

// 3xTF32 keeps fp32-level accuracy only if the tensor core's accumulator is not asked to absorb hundreds of
// additions: its fp32 accumulation truncates toward zero (measured: a relative shrink of ~8e-6 after 375
// additions).  So in that mode the hi*hi products are spread round-robin over NACC TMEM accumulators (each sees
// 1/NACC of the additions on a smaller partial sum), the two small cross terms go to an accumulator of their own,
// and the epilogue adds the partial sums with round-to-nearest fp32.
__host__ __device__ constexpr int num_acc(int BN, int mode) {
  return mode != TC_TF32X3 ? 1 : (BN <= 32 ? 8 : (BN <= 64 ? 4 : (BN <= 128 ? 2 : 1)));
}
__host__ __device__ constexpr int tmem_cols(int BN, int mode) {
  int need = (mode == TC_TF32X3 ? num_acc(BN, mode) + 1 : 1) * BN;
  int c = 32;
  while (c < need) c *= 2;
  return c;
}

template <int BN, int MODE, int EPI>
__global__ void __launch_bounds__(192, 1) tc_gemm_kernel(const __grid_constant__ TcParams p) {
  constexpr int ST = num_stages(BN, MODE);
  constexpr int STAGE = stage_bytes(BN, MODE);
  constexpr int BBYTES = BN * 128;
  constexpr uint32_t IDESC = make_idesc(MODE == TC_BF16 ? 1u : 2u, BN);
  constexpr int NACC = num_acc(BN, MODE);
  constexpr int TMEM_COLS = tmem_cols(BN, MODE);
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[ST];
  __shared__ __align__(8) uint64_t empty_bar[ST];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const int m0 = blockIdx.x * 128;
  const int n_tile = blockIdx.y;
  int total_kb = 0;
  for (int s = 0; s < p.nsrc; ++s) total_kb += p.kblocks[s];

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&accum_bar, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int s = 0; s < p.nsrc && ok; ++s) {
        for (int kb = 0; kb < p.kblocks[s]; ++kb, ++it) {
          const int st = it % ST;
          const uint32_t ph = (uint32_t)((it / ST) & 1);
          if (!mbar_wait(&empty_bar[st], ph ^ 1u, &abort_s, p.err, 1)) { ok = false; break; }
          uint8_t* base = tiles + (size_t)st * STAGE;
          mbar_expect_tx(&full_bar[st], (uint32_t)STAGE);
          const int kx = kb * (MODE == TC_BF16 ? 64 : 32);
          tma_load_2d(base, &p.a[s], &full_bar[st], kx, m0);
          tma_load_2d(base + kABytes, &p.b, &full_bar[st], p.b_koff[s] + kx, n_tile * BN);
          if (MODE == TC_TF32X3) {
            tma_load_2d(base + kABytes + BBYTES, &p.a_lo[s], &full_bar[st], kx, m0);
            tma_load_2d(base + 2 * kABytes + BBYTES, &p.b_lo, &full_bar[st], p.b_koff[s] + kx, n_tile * BN);
          }
        }
      }
      if (!ok) {
        // wait (bounded) for copies already in flight before the CTA may retire
        for (int st = 0; st < ST; ++st) {
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000LL) {}
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = true;
      for (int it = 0; it < total_kb; ++it) {
        const int st = it % ST;
        const uint32_t ph = (uint32_t)((it / ST) & 1);
        if (!mbar_wait(&full_bar[st], ph, &abort_s, p.err, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(tiles + (size_t)st * STAGE);
        const uint32_t b_addr = a_addr + kABytes;
        const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(b_addr);
        const uint32_t d_main = tmem_base + (uint32_t)((it % NACC) * BN);  // round-robin over the main accumulators
#pragma unroll
        for (int k = 0; k < 4; ++k) {  // 4 x 32 bytes of K per 128-byte k-block
          const uint32_t acc = (it >= NACC || k > 0) ? 1u : 0u;
          umma<MODE != TC_BF16>(d_main, da + 2 * k, db + 2 * k, IDESC, acc);
          if (MODE == TC_TF32X3) {
            const uint64_t dal = make_smem_desc(b_addr + BBYTES), dbl = make_smem_desc(b_addr + BBYTES + kABytes);
            const uint32_t d_cross = tmem_base + (uint32_t)(NACC * BN);
            umma<1>(d_cross, dal + 2 * k, db + 2 * k, IDESC, (it > 0 || k > 0) ? 1u : 0u);
            umma<1>(d_cross, da + 2 * k, dbl + 2 * k, IDESC, 1u);
          }
        }
        umma_commit(&empty_bar[st]);
      }
      if (ok) umma_commit(&accum_bar);
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 0-3)
    const int row = m0 + warp * 32 + lane;
    const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
    const bool ready = (total_kb == 0) ? false : mbar_wait(&accum_bar, 0, &abort_s, p.err, 3);
    tc_fence_after();
    const int n_main = total_kb < NACC ? total_kb : NACC;  // main accumulators that were written
    // 8 accumulator columns starting at `col`, summed over the partial accumulators
    auto load8 = [&](int col, float* v) {
      tmem_ld8(taddr + col, v);
      if (MODE == TC_TF32X3) {
        float t[8];
        for (int a = 1; a < n_main; ++a) {
          tmem_ld8(taddr + a * BN + col, t);
          tmem_wait_ld();
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] += t[u];
        }
        tmem_ld8(taddr + NACC * BN + col, t);
        tmem_wait_ld();
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] += t[u];
      }
      tmem_wait_ld();
    };
    if (ready) {
      const bool row_ok = row < p.M;
      const float mk = (p.mask && row_ok) ? (float)p.mask[row] : 1.0f;
      if (EPI == TC_EPI_LSTM) {
        constexpr int TH = BN / 4;
        const int H = p.N;
        const int hid0 = n_tile * TH;
        for (int j0 = 0; j0 < TH; j0 += 8) {
          float g[4][8];
#pragma unroll
          for (int q = 0; q < 4; ++q) load8(q * TH + j0, g[q]);
          if (row_ok) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int hid = hid0 + j0 + u;
              if (hid < H) {
                const float gi = sigmoid_acc(g[0][u] + p.bias[hid]);
                const float gf = sigmoid_acc(g[1][u] + p.bias[H + hid]);
                const float gg = tanhf(g[2][u] + p.bias[2 * H + hid]);
                const float go = sigmoid_acc(g[3][u] + p.bias[3 * H + hid]);
                const size_t idx = (size_t)row * H + hid;
                float c = gf * p.c_prev[idx] + gi * gg;
                float h = go * tanhf(c);
                h *= mk;
                c *= mk;
                p.c_out[idx] = c;
                if (p.C) p.C[(size_t)row * p.ldc + hid] = h;
                store_operand(p, (size_t)row * p.ld_op + hid, h);
              }
            }
          }
        }
      } else if (EPI == TC_EPI_STORE) {
        const int n0 = n_tile * BN;
        for (int c0 = 0; c0 < BN; c0 += 8) {
          float v[8];
          load8(c0, v);
          if (row_ok) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int n = n0 + c0 + u;
              if (n < p.N) {
                float x = v[u] + (p.bias ? p.bias[n] : 0.f);
                if (p.act == 1 && (p.act_rows == 0 || n < p.act_rows)) x = tanhf(x);
                x *= mk;
                if (p.C) p.C[(size_t)row * p.ldc + n] = x;
                store_operand(p, (size_t)row * p.ld_op + n, x);
              }
            }
          }
        }
      } else {  // TC_EPI_LSE
        const int n0 = n_tile * BN;
        const int tg = (p.target && row_ok) ? p.target[row] - p.target_offset : -1;
        float mx = -INFINITY, sm = 0.f;
        for (int c0 = 0; c0 < BN; c0 += 8) {
          float v[8];
          load8(c0, v);
          float cm = -INFINITY;
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int n = n0 + c0 + u;
            v[u] = (n < p.N) ? v[u] + (p.bias ? p.bias[n] : 0.f) : -INFINITY;
            cm = fmaxf(cm, v[u]);
            if (n == tg && n < p.N) p.tgt_logit[row] = v[u];
          }
          if (cm > mx) {
            sm *= expf(mx - cm);  // expf(-inf) = 0 on the first chunk
            mx = cm;
          }
          if (mx != -INFINITY) {
#pragma unroll
            for (int u = 0; u < 8; ++u) sm += expf(v[u] - mx);
          }
        }
        if (row_ok) {
          p.part_max[(size_t)n_tile * p.M + row] = mx;
          p.part_sum[(size_t)n_tile * p.M + row] = sm;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

template <int BN, int MODE, int EPI>
cudaError_t launch_t(const TcParams& p, cudaStream_t st) {
  const size_t smem = (size_t)num_stages(BN, MODE) * stage_bytes(BN, MODE) + 1024;
  static bool configured = false;  // once per instantiation (one device per process)
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(tc_gemm_kernel<BN, MODE, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int n_rows = (EPI == TC_EPI_LSTM) ? p.N * 4 : p.N;
  dim3 grid((p.M + 127) / 128, (n_rows + BN - 1) / BN);
  if (grid.x == 0 || grid.y == 0) return cudaSuccess;
  tc_gemm_kernel<BN, MODE, EPI><<<grid, 192, smem, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

template <int MODE, int EPI>
cudaError_t launch_bn(const TcParams& p, int BN, cudaStream_t st) {
  switch (BN) {
    case 32: return launch_t<32, MODE, EPI>(p, st);
    case 64: return launch_t<64, MODE, EPI>(p, st);
    case 128: return launch_t<128, MODE, EPI>(p, st);
    case 256: return launch_t<256, MODE, EPI>(p, st);
  }
  return cudaErrorInvalidValue;
}
template <int MODE>
cudaError_t launch_epi(const TcParams& p, int BN, int epi, cudaStream_t st) {
  switch (epi) {
    case TC_EPI_STORE: return launch_bn<MODE, TC_EPI_STORE>(p, BN, st);
    case TC_EPI_LSTM: return launch_bn<MODE, TC_EPI_LSTM>(p, BN, st);
    case TC_EPI_LSE: return launch_bn<MODE, TC_EPI_LSE>(p, BN, st);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_tc_gemm(const TcParams& p, int BN, int mode, int epi, cudaStream_t st) {
  switch (mode) {
    case TC_BF16: return launch_epi<TC_BF16>(p, BN, epi, st);
    case TC_TF32: return launch_epi<TC_TF32>(p, BN, epi, st);
    case TC_TF32X3: return launch_epi<TC_TF32X3>(p, BN, epi, st);
  }
  return cudaErrorInvalidValue;
}

// ------------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

bool make_kmajor_map(CUtensorMap* out, const void* base, int elem_bytes, long long k, long long rows, long long ld,
                     int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || !base || k <= 0 || rows <= 0 || box_rows <= 0 || box_rows > 256) return false;
  if (((uintptr_t)base & 15) != 0 || ((ld * elem_bytes) & 15) != 0) return false;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld * elem_bytes)};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace zrnn
