// Device-side building blocks shared by the tensor-core kernels (tc_gemm.cu, tc_decoder.cu): PTX wrappers for
// mbarriers, TMA, tcgen05 / TMEM and clusters, the operand-form store helpers and the per-mode traits.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "tc_gemm.cuh"

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
// Bounded wait.  Gives up after `limit` SM cycles (about a second by default) or as soon as another role has given up
// (*abort_flag != 0); the first role to give up leaves `code` in the device error word.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err, int code,
                                          long long limit = 2000000000LL) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) {
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
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ float tf32_round_dev(float x) {
  uint32_t u = __float_as_uint(x);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;
  return __uint_as_float((u + 0x1000u) & 0xffffe000u);
}
// 8 consecutive outputs of one row: vector stores when the group is complete and 16-byte aligned
__device__ __forceinline__ void store8_f32(float* base, size_t idx, const float* v, int nvalid) {
  if (nvalid == 8 && (idx & 3) == 0) {
    float4* d = reinterpret_cast<float4*>(base + idx);
    d[0] = make_float4(v[0], v[1], v[2], v[3]);
    d[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    for (int u = 0; u < nvalid; ++u) base[idx + u] = v[u];
  }
}
template <class P>
__device__ __forceinline__ void store8_operand(const P& p, size_t idx, const float* v, int nvalid) {
  if (p.op_b16) {
    if (nvalid == 8 && (idx & 7) == 0) {
      __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
      __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
      uint4 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&a); pk.y = *reinterpret_cast<uint32_t*>(&b);
      pk.z = *reinterpret_cast<uint32_t*>(&c); pk.w = *reinterpret_cast<uint32_t*>(&d);
      *reinterpret_cast<uint4*>(p.op_b16 + idx) = pk;
    } else {
      for (int u = 0; u < nvalid; ++u) p.op_b16[idx + u] = __float2bfloat16(v[u]);
    }
  }
  if (p.op_h_hi) {  // fp16 split operands: hi = fp16(v), lo = fp16((v - hi) * 2^11)
    __align__(16) __half hi[8];
    __align__(16) __half lo[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      hi[u] = __float2half_rn(v[u]);
      lo[u] = __float2half_rn((v[u] - __half2float(hi[u])) * 2048.0f);
    }
    if (nvalid == 8 && (idx & 7) == 0) {
      *reinterpret_cast<uint4*>(p.op_h_hi + idx) = *reinterpret_cast<const uint4*>(hi);
      *reinterpret_cast<uint4*>(p.op_h_lo + idx) = *reinterpret_cast<const uint4*>(lo);
    } else {
      for (int u = 0; u < nvalid; ++u) { p.op_h_hi[idx + u] = hi[u]; p.op_h_lo[idx + u] = lo[u]; }
    }
  }
  if (p.op_hi) {
    float hi[8], lo[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) { hi[u] = tf32_round_dev(v[u]); lo[u] = v[u] - hi[u]; }
    store8_f32(p.op_hi, idx, hi, nvalid);
    if (p.op_lo) store8_f32(p.op_lo, idx, lo, nvalid);
  }
}
// four consecutive values (the 8-warp LSTM epilogue): same destinations as store8_f32 / store8_operand
__device__ __forceinline__ void store4_f32(float* base, size_t idx, const float* v, int nvalid) {
  if (nvalid == 4 && (idx & 3) == 0) {
    *reinterpret_cast<float4*>(base + idx) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
    for (int u = 0; u < nvalid; ++u) base[idx + u] = v[u];
  }
}
template <class P>
__device__ __forceinline__ void store4_operand(const P& p, size_t idx, const float* v, int nvalid) {
  const bool vec = nvalid == 4 && (idx & 3) == 0;
  if (p.op_b16) {
    if (vec) {
      __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&a); pk.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(p.op_b16 + idx) = pk;
    } else {
      for (int u = 0; u < nvalid; ++u) p.op_b16[idx + u] = __float2bfloat16(v[u]);
    }
  }
  if (p.op_h_hi) {
    __align__(8) __half hi[4];
    __align__(8) __half lo[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      hi[u] = __float2half_rn(v[u]);
      lo[u] = __float2half_rn((v[u] - __half2float(hi[u])) * 2048.0f);
    }
    if (vec) {
      *reinterpret_cast<uint2*>(p.op_h_hi + idx) = *reinterpret_cast<const uint2*>(hi);
      *reinterpret_cast<uint2*>(p.op_h_lo + idx) = *reinterpret_cast<const uint2*>(lo);
    } else {
      for (int u = 0; u < nvalid; ++u) { p.op_h_hi[idx + u] = hi[u]; p.op_h_lo[idx + u] = lo[u]; }
    }
  }
  if (p.op_hi) {
    float hi[4], lo[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) { hi[u] = tf32_round_dev(v[u]); lo[u] = v[u] - hi[u]; }
    store4_f32(p.op_hi, idx, hi, nvalid);
    if (p.op_lo) store4_f32(p.op_lo, idx, lo, nvalid);
  }
}

// Mode traits.  "Split" modes keep every operand as a hi part plus a residual lo part and spend three MMAs per
// k-step (hi*hi into the main accumulators, lo*hi and hi*lo into the cross accumulator):
//   TC_TF32X3: fp32 storage, hi = value rounded to tf32, lo = value - hi
//   TC_F16X2 : fp16 storage, hi = value rounded to fp16, lo = (value - hi) * 2^11 rounded to fp16; the cross
//              accumulator is scaled back by 2^-11 in the epilogue.  Same 11 + 11 significant bits, half the bytes
//              and half the tensor time; operands must stay inside the fp16 range (|x| < 65504).
__host__ __device__ constexpr bool mode_split(int mode) { return mode == TC_TF32X3 || mode == TC_F16X2; }
__host__ __device__ constexpr bool mode_exact_math(int mode) { return mode_split(mode); }
__host__ __device__ constexpr bool mode_kind_tf32(int mode) { return mode == TC_TF32 || mode == TC_TF32X3; }
__host__ __device__ constexpr int mode_epk(int mode) { return mode_kind_tf32(mode) ? 32 : 64; }  // elements per k-block
__host__ __device__ constexpr uint32_t mode_fmt(int mode) { return mode == TC_BF16 ? 1u : (mode == TC_F16X2 ? 0u : 2u); }
__host__ __device__ constexpr float mode_cross_scale(int mode) { return mode == TC_F16X2 ? (1.0f / 2048.0f) : 1.0f; }

// activations: exact for the fp32-accurate mode, hardware approximations (tanh.approx, ~2^-11) for bf16 / tf32
template <int MODE>
__device__ __forceinline__ float act_tanh(float x) {
  if (mode_exact_math(MODE)) return tanhf(x);
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <int MODE>
__device__ __forceinline__ float act_sigmoid(float x) {
  if (mode_exact_math(MODE)) return 1.0f / (1.0f + expf(-x));
  return fmaf(0.5f, act_tanh<MODE>(0.5f * x), 0.5f);
}

constexpr int kABytes = 128 * 128;  // A tile: 128 rows x 128-byte k-block
__host__ __device__ constexpr int stage_bytes(int BN, int mode) { return (mode_split(mode) ? 2 : 1) * (kABytes + BN * 128); }
// bytes of the split-K exchange slots: SPLITK slots of (BN/SPLITK)/4 x 128 rows of float4.  They must not overlap
// the stage ring: a peer that finishes its main loop early pushes into them while this CTA may still be loading.
__host__ __device__ constexpr int slot_bytes(int BN, int splitk) {
  return splitk > 1 ? splitk * 128 * (BN / splitk) * 4 : 0;
}
// 3xTF32 stages are twice as large (hi + lo parts), and with exchange slots of their own only two would fit, too few
// bytes in flight to keep HBM busy.  In that mode the slots alias the ring instead, which costs one more cluster
// barrier (nobody may push into a peer's ring before that peer's MMAs have consumed it).
__host__ __device__ constexpr bool slots_alias_ring(int mode, int splitk) { return mode_split(mode) && splitk > 1; }
__host__ __device__ constexpr int num_stages(int BN, int mode, int splitk = 1) {
  int s = (225 * 1024 - 1024 - (slots_alias_ring(mode, splitk) ? 0 : slot_bytes(BN, splitk))) / stage_bytes(BN, mode);
  return s > 8 ? 8 : s;
}
__host__ __device__ constexpr int smem_bytes(int BN, int mode, int splitk) {
  return num_stages(BN, mode, splitk) * stage_bytes(BN, mode) + (slots_alias_ring(mode, splitk) ? 0 : slot_bytes(BN, splitk)) + 1024;
}

// The split modes keep fp32-level accuracy only if the tensor core's accumulator is not asked to absorb hundreds of
// additions: its fp32 accumulation truncates toward zero (measured: a relative shrink of ~8e-6 after 375
// additions).  So in those modes the hi*hi products are spread round-robin over NACC TMEM accumulators (each sees
// 1/NACC of the additions on a smaller partial sum), the two small cross terms go to an accumulator of their own,
// and the epilogue adds the partial sums with round-to-nearest fp32.  128-column tiles use all 512 TMEM columns:
// three main accumulators and the cross one (against two: log-prob error at H = 1000, 4 layers 2.0e-6 -> 1.4e-6).
__host__ __device__ constexpr int num_acc(int BN, int mode) {
  return !mode_split(mode) ? 1 : (BN <= 32 ? 8 : (BN <= 64 ? 4 : (BN <= 128 ? 3 : 1)));  // (NACC + 1) BN <= 512 columns
}
__host__ __device__ constexpr int tmem_cols(int BN, int mode) {
  int need = (mode_split(mode) ? num_acc(BN, mode) + 1 : 1) * BN;
  int c = 32;
  while (c < need) c *= 2;
  return c;
}

__device__ __forceinline__ long long gtime() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define ZR_STAMP(i)                                                                                           \
  do {                                                                                                        \
    if (p.prof && (threadIdx.x == 0)) {                                                                       \
      if (p.prof_slot < 0)                                                                                    \
        p.prof[((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + (i)] = gtime(); \
      else if (blockIdx.x + blockIdx.y + blockIdx.z == 0)                                                     \
        p.prof[(size_t)p.prof_slot * 8 + (i)] = gtime();                                                      \
    }                                                                                                         \
  } while (0)

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may start while
// its predecessor is still draining; pdl_wait() blocks until the predecessor has completed and its writes are
// visible, pdl_trigger() tells the runtime that the successor may be scheduled.  Both are no-ops otherwise.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t cluster_map(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

}  // namespace
}  // namespace zrnn
