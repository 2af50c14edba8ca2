// tcgen05 / TMEM / TMA GEMM kernels for sm_100a.  See tc_gemm.cuh for the operand convention.
//
// CTA = 6 warps: warps 0-3 run the epilogue (one TMEM lane quadrant each), warp 4 is the TMA producer,
// warp 5 owns the TMEM allocation and issues tcgen05.mma.  A ring of shared-memory stages is guarded by
// full/empty mbarriers; every wait is bounded (about a second of SM clock) and reports through p.err
// instead of spinning forever.
#include "tc_gemm.cuh"

#include <cstdint>
#include <cstdlib>
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
__device__ __forceinline__ void store8_operand(const TcParams& p, size_t idx, const float* v, int nvalid) {
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
__device__ __forceinline__ void store4_operand(const TcParams& p, size_t idx, const float* v, int nvalid) {
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

// SPLITK > 1: the CTAs of a (1,1,SPLITK) cluster each accumulate a slice of the K axis for the same output tile.
// Each CTA then finishes 1/SPLITK of the tile's columns: every CTA pushes the matching columns of its partial tile
// into a slot of the owner's shared memory with remote stores (distributed shared memory; stores need no round
// trip, remote loads measured ~1.4 us each), a cluster barrier publishes them, and the owner adds its SPLITK slots
// in a fixed order.  This keeps the number of CTAs high for skinny problems (one 128-row M tile) without every CTA
// re-reading the whole A operand.
// The body is a device function over a reference to the kernel parameters, so that one launch can also carry several
// independent problems (tc_gemm_multi_kernel below).
template <int BN, int MODE, int EPI, int SPLITK>
__device__ __forceinline__ void tc_gemm_body(const TcParams& p, const int m_block) {
  constexpr int ST = num_stages(BN, MODE, SPLITK);
  constexpr int STAGE = stage_bytes(BN, MODE);
  constexpr int BBYTES = BN * 128;
  static_assert(ST >= 2, "need at least a double-buffered ring");
  constexpr uint32_t IDESC = make_idesc(mode_fmt(MODE), BN);
  constexpr int NACC = num_acc(BN, MODE);
  constexpr int TMEM_COLS = tmem_cols(BN, MODE);
  constexpr int OWNC = BN / SPLITK;  // columns finished by each CTA of the cluster
  static_assert(SPLITK == 1 || SPLITK * OWNC * 128 * 4 == slot_bytes(BN, SPLITK), "slot size mismatch");
  constexpr bool ALIAS = slots_alias_ring(MODE, SPLITK);
  static_assert(!ALIAS || ST * STAGE >= slot_bytes(BN, SPLITK), "ring too small to hold the exchange slots");
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[ST];
  __shared__ __align__(8) uint64_t empty_bar[ST];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  // the tile's bias values, read by every epilogue thread for every column: staged once (a weight, so it does not
  // wait for the predecessor kernel).  LSE: -inf beyond the last valid row, which removes the column from max / sum.
  __shared__ float s_bias[BN];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const int m0 = m_block * 128;
  const int n_tile = blockIdx.y;
  for (int i = threadIdx.x; i < BN; i += blockDim.x) {
    float bv;
    if (EPI == TC_EPI_LSTM) {
      constexpr int TH = BN / 4;
      const int hid = n_tile * TH + (i % TH);
      bv = hid < p.N ? p.bias[(i / TH) * p.N + hid] : 0.f;
    } else {
      const int n = n_tile * BN + i;
      bv = n < p.N ? (p.bias ? p.bias[n] : 0.f) : (EPI == TC_EPI_LSE ? -INFINITY : 0.f);
    }
    s_bias[i] = bv;
  }
  const int rank = SPLITK > 1 ? (int)blockIdx.z : 0;  // cluster dims (1,1,SPLITK): rank in cluster == blockIdx.z
  int all_kb = 0;
  for (int s = 0; s < p.nsrc; ++s) all_kb += p.kblocks[s];
  // this CTA's slice [kb_lo, kb_hi) of the global k-block sequence
  const int kb_lo = (int)(((long long)all_kb * rank) / SPLITK);
  const int kb_hi = (int)(((long long)all_kb * (rank + 1)) / SPLITK);
  const int total_kb = kb_hi - kb_lo;

  ZR_STAMP(0);
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
  ZR_STAMP(1);
  pdl_wait();  // everything above touched only this CTA's shared memory and TMEM

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int it = 0, g = 0;
      bool ok = true;
      for (int s = 0; s < p.nsrc && ok; ++s) {
        for (int kb = 0; kb < p.kblocks[s]; ++kb, ++g) {
          if (g < kb_lo || g >= kb_hi) continue;
          const int st = it % ST;
          const uint32_t ph = (uint32_t)((it / ST) & 1);
          if (!mbar_wait(&empty_bar[st], ph ^ 1u, &abort_s, p.err, 1)) { ok = false; break; }
          uint8_t* base = tiles + (size_t)st * STAGE;
          mbar_expect_tx(&full_bar[st], (uint32_t)STAGE);
          constexpr int EPK = mode_epk(MODE);  // elements per 128-byte k-block
          const int kx = kb * EPK;
          const int bx = p.b_tiled_kbtot > 0 ? 0 : p.b_koff[s] + kx;
          const int by = p.b_tiled_kbtot > 0 ? (n_tile * p.b_tiled_kbtot + (p.b_koff[s] + kx) / EPK) * BN : n_tile * BN;
          tma_load_2d(base, &p.a[s], &full_bar[st], kx, m0);
          if (mode_split(MODE)) tma_load_2d(base + kABytes + BBYTES, &p.a_lo[s], &full_bar[st], kx, m0);
          if (p.b_pack_rows > 0 && p.b_pack_rows < BN) {
            // B was packed for narrower row tiles: this tile is BN / pack consecutive packed tiles, one box each
            const int parts = BN / p.b_pack_rows, kbg = (p.b_koff[s] + kx) / EPK;
            for (int h = 0; h < parts; ++h) {
              const int pt = n_tile * parts + h;
              const int byh = p.b_tiled_kbtot > 0 ? (pt * p.b_tiled_kbtot + kbg) * p.b_pack_rows : pt * p.b_pack_rows;
              const size_t off = (size_t)h * p.b_pack_rows * 128;
              tma_load_2d(base + kABytes + off, &p.b, &full_bar[st], bx, byh);
              if (mode_split(MODE)) tma_load_2d(base + 2 * kABytes + BBYTES + off, &p.b_lo, &full_bar[st], bx, byh);
            }
          } else {
            tma_load_2d(base + kABytes, &p.b, &full_bar[st], bx, by);
            if (mode_split(MODE)) tma_load_2d(base + 2 * kABytes + BBYTES, &p.b_lo, &full_bar[st], bx, by);
          }
          ++it;
        }
      }
      if (!ok) {
        // give copies already in flight time to land before the CTA may retire
        const long long t0 = clock64();
        while (clock64() - t0 < 20000000LL) {}
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
          umma<mode_kind_tf32(MODE)>(d_main, da + 2 * k, db + 2 * k, IDESC, acc);
          if (mode_split(MODE)) {
            const uint64_t dal = make_smem_desc(b_addr + BBYTES), dbl = make_smem_desc(b_addr + BBYTES + kABytes);
            const uint32_t d_cross = tmem_base + (uint32_t)(NACC * BN);
            umma<mode_kind_tf32(MODE)>(d_cross, dal + 2 * k, db + 2 * k, IDESC, (it > 0 || k > 0) ? 1u : 0u);
            umma<mode_kind_tf32(MODE)>(d_cross, da + 2 * k, dbl + 2 * k, IDESC, 1u);
          }
        }
        umma_commit(&empty_bar[st]);
      }
      if (ok) umma_commit(&accum_bar);
    }
  }

  __syncwarp();  // lanes of the producer / MMA warps rejoin lane 0 before any warp-aligned barrier
  // ------------------------------------------------------------ epilogue (warps 0-3 do the math)
  const bool epi_warp = warp < 4;
  const int row = m0 + warp * 32 + lane;  // meaningful for epilogue warps only
  const int lrow = warp * 32 + lane;
  const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
  // the LSTM epilogue's global operands do not depend on the accumulators: fetch them while the main loop runs
  // With a 256-thread block (split-K LSTM cells that own 8 hidden units per CTA) the math after the exchange is
  // spread over all 8 warps: thread t finishes row t % 128, hidden units 4 * (t / 128) .. + 4 of the CTA's 8.
  const bool wide = EPI == TC_EPI_LSTM && SPLITK > 1 && BN / 4 / SPLITK == 8 && blockDim.x == 256;
  const int wrow = m0 + (threadIdx.x & 127), whalf = threadIdx.x >> 7;
  float pre_c[8];
  if constexpr (EPI == TC_EPI_LSTM) {
    constexpr int TH = BN / 4;
    constexpr int TH_OWN = TH / SPLITK;
    if (wide) {
      const int H = p.N;
      const int hidb = n_tile * TH + rank * TH_OWN + whalf * 4;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int hid = hidb + u;
        pre_c[u] = (hid < H && wrow < p.M) ? p.c_prev[(size_t)wrow * H + hid] : 0.f;
      }
    } else if (TH_OWN == 8 && epi_warp) {
      const int H = p.N;
      const int hidb = n_tile * TH + rank * TH_OWN;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int hid = hidb + u;
        const bool okh = hid < H;
        pre_c[u] = (okh && row < p.M) ? p.c_prev[(size_t)row * H + hid] : 0.f;
      }
    }
  }
  bool ready = false;
  if (epi_warp) {
    ready = (total_kb == 0) ? (SPLITK > 1) : mbar_wait(&accum_bar, 0, &abort_s, p.err, 3);
    tc_fence_after();
  }
  ZR_STAMP(2);
  pdl_trigger();  // the successor may begin its prologue while this kernel runs its epilogue
  const int n_main = total_kb < NACC ? total_kb : NACC;  // main accumulators that were written
  // 8 accumulator columns starting at `col` from TMEM, summed over the partial accumulators
  auto load8_tmem = [&](int col, float* v) {
    if (total_kb == 0) {
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = 0.f;
      return;
    }
    tmem_ld8(taddr + col, v);
    if (mode_split(MODE)) {
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
      for (int u = 0; u < 8; ++u) v[u] = fmaf(t[u], mode_cross_scale(MODE), v[u]);
    }
    tmem_wait_ld();
  };
  // the same for 32 columns with one wait per accumulator (the split-K exchange reads the whole tile)
  auto load32_tmem = [&](int col, float* v) {
    if (total_kb == 0) {
#pragma unroll
      for (int u = 0; u < 32; ++u) v[u] = 0.f;
      return;
    }
    tmem_ld32(taddr + col, v);
    if (mode_split(MODE)) {
      float t[32];
      for (int a = 1; a < n_main; ++a) {
        tmem_ld32(taddr + a * BN + col, t);
        tmem_wait_ld();
#pragma unroll
        for (int u = 0; u < 32; ++u) v[u] += t[u];
      }
      tmem_ld32(taddr + NACC * BN + col, t);
      tmem_wait_ld();
#pragma unroll
      for (int u = 0; u < 32; ++u) v[u] = fmaf(t[u], mode_cross_scale(MODE), v[u]);
    }
    tmem_wait_ld();
  };
  // slots[q][c4][row] (float4 units): contribution of cluster rank q to this CTA's columns (split-K only), placed
  // after the ring.  Rows are the fastest index, so the 32 lanes of a warp push 512 contiguous bytes per remote store
  // and read back without bank conflicts.  Column order inside a slot: LSTM -> gate*TH_OWN + j (this CTA's hidden
  // units, all four gates); otherwise the CTA's OWNC consecutive columns.
  float4* slots = reinterpret_cast<float4*>(ALIAS ? tiles : tiles + (size_t)ST * STAGE);
  if (SPLITK > 1) {
    if (ALIAS) {
      // every CTA of the cluster is past its main loop (its ring is dead) before anybody pushes into it
      tc_fence_before();
      cluster_sync_all();
    }
    if (epi_warp && ready) {
      const uint32_t my_slot = smem_u32(slots + (size_t)rank * (OWNC / 4) * 128 + lrow);
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        load32_tmem(c0, v);
#pragma unroll
        for (int u = 0; u < 32; u += 4) {
          const int c = c0 + u;
          int owner, lcol;
          if (EPI == TC_EPI_LSTM) {
            constexpr int TH = BN / 4, TH_OWN = TH / SPLITK;
            const int gate = c / TH, j = c % TH;
            owner = j / TH_OWN;
            lcol = gate * TH_OWN + (j % TH_OWN);
          } else {
            owner = c / OWNC;
            lcol = c % OWNC;
          }
          const uint32_t local = my_slot + (uint32_t)((lcol / 4) * 128 * 16);
          if (owner == rank) {
            slots[((size_t)rank * (OWNC / 4) + lcol / 4) * 128 + lrow] = make_float4(v[u], v[u + 1], v[u + 2], v[u + 3]);
          } else {
            st_cluster_v4(cluster_map(local, (uint32_t)owner), v[u], v[u + 1], v[u + 2], v[u + 3]);
          }
        }
      }
    }
    tc_fence_before();
    ZR_STAMP(3);
    cluster_sync_all();  // release/acquire: every CTA's pushes are visible to their owners
    ZR_STAMP(4);
  }
  // 8 finished accumulator columns: `col` is a tile column (SPLITK == 1) or a slot column (SPLITK > 1)
  auto load8 = [&](int col, float* v) {
    if (SPLITK == 1) {
      load8_tmem(col, v);
    } else {
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = 0.f;
#pragma unroll
      for (int q = 0; q < SPLITK; ++q) {
        const float4* src = slots + ((size_t)q * (OWNC / 4) + col / 4) * 128 + lrow;
        const float4 a = src[0], b = src[128];
        v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
        v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
      }
    }
  };
  if constexpr (EPI == TC_EPI_LSTM && SPLITK > 1) {
    if (wide) {
      constexpr int TH = BN / 4, TH_OWN = TH / SPLITK;
      const int H = p.N;
      if (!abort_s && wrow < p.M) {
        const int r = threadIdx.x & 127;
        float g[4][4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int rk = 0; rk < SPLITK; ++rk) {  // fixed order: deterministic sums
            const float4 t = slots[((size_t)rk * (OWNC / 4) + (q * TH_OWN) / 4 + whalf) * 128 + r];
            acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
          }
          g[q][0] = acc.x; g[q][1] = acc.y; g[q][2] = acc.z; g[q][3] = acc.w;
        }
        ZR_STAMP(5);
        const float mk = p.mask ? (float)p.mask[wrow] : 1.0f;
        const int jb = rank * TH_OWN + whalf * 4;  // first hidden unit inside the tile
        const int hb = n_tile * TH + jb;
        const int nvalid = H - hb >= 4 ? 4 : (H - hb > 0 ? H - hb : 0);
        float hv[4], cvv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float gi = act_sigmoid<MODE>(g[0][u] + s_bias[jb + u]);
          const float gf = act_sigmoid<MODE>(g[1][u] + s_bias[TH + jb + u]);
          const float gg = act_tanh<MODE>(g[2][u] + s_bias[2 * TH + jb + u]);
          const float go = act_sigmoid<MODE>(g[3][u] + s_bias[3 * TH + jb + u]);
          const float c = gf * pre_c[u] + gi * gg;
          hv[u] = go * act_tanh<MODE>(c) * mk;
          cvv[u] = c * mk;
        }
        ZR_STAMP(6);
        if (nvalid > 0) {
          store4_f32(p.c_out, (size_t)wrow * H + hb, cvv, nvalid);
          if (p.C) store4_f32(p.C, (size_t)wrow * p.ldc + hb, hv, nvalid);
          store4_operand(p, (size_t)wrow * p.ld_op + hb, hv, nvalid);
        }
      }
      ready = false;  // the 4-warp epilogue below is skipped
    }
  }
  if (epi_warp && ready) {
    const bool row_ok = row < p.M;
    const float mk = (p.mask && row_ok) ? (float)p.mask[row] : 1.0f;
    if constexpr (EPI == TC_EPI_LSTM) {
      constexpr int TH = BN / 4;
      constexpr int TH_OWN = TH / SPLITK;  // hidden units finished by this CTA
      static_assert(TH_OWN % 8 == 0, "each CTA must own a multiple of 8 hidden units");
      const int H = p.N;
      const int hid0 = n_tile * TH;
      for (int j0 = rank * TH_OWN; j0 < (rank + 1) * TH_OWN; j0 += 8) {
        float g[4][8];
        // accumulator column of (gate q, hidden j0): gate blocks of THP hidden units, THP = the packing's tile
        // (the tile itself unless the weights were packed for narrower tiles)
        const int THP = (p.b_pack_rows > 0 && p.b_pack_rows < BN) ? p.b_pack_rows / 4 : TH;
#pragma unroll
        for (int q = 0; q < 4; ++q)
          load8(SPLITK == 1 ? (j0 / THP) * (4 * THP) + q * THP + (j0 % THP) : q * TH_OWN + (j0 - rank * TH_OWN), g[q]);
        ZR_STAMP(5);
        if (row_ok) {
          const int hb = hid0 + j0;
          const int nvalid = H - hb >= 8 ? 8 : (H - hb > 0 ? H - hb : 0);
          const bool pf = (TH_OWN == 8);  // operands were prefetched
          float hv[8], cvv[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int hid = hb + u;
            const bool okh = u < nvalid;
            const float b0 = s_bias[j0 + u], b1 = s_bias[TH + j0 + u], b2 = s_bias[2 * TH + j0 + u], b3 = s_bias[3 * TH + j0 + u];
            const float cp = pf ? pre_c[u] : (okh ? p.c_prev[(size_t)row * H + hid] : 0.f);
            const float gi = act_sigmoid<MODE>(g[0][u] + b0);
            const float gf = act_sigmoid<MODE>(g[1][u] + b1);
            const float gg = act_tanh<MODE>(g[2][u] + b2);
            const float go = act_sigmoid<MODE>(g[3][u] + b3);
            const float c = gf * cp + gi * gg;
            hv[u] = go * act_tanh<MODE>(c) * mk;
            cvv[u] = c * mk;
          }
          ZR_STAMP(6);
          if (nvalid > 0) {
            store8_f32(p.c_out, (size_t)row * H + hb, cvv, nvalid);
            if (p.C) store8_f32(p.C, (size_t)row * p.ldc + hb, hv, nvalid);
            store8_operand(p, (size_t)row * p.ld_op + hb, hv, nvalid);
          }
        }
      }
    } else if constexpr (EPI == TC_EPI_STORE) {
      constexpr int OWN = BN / SPLITK;
      static_assert(OWN % 8 == 0, "each CTA must own a multiple of 8 columns");
      const int n0 = n_tile * BN;
      for (int c0 = rank * OWN; c0 < (rank + 1) * OWN; c0 += 8) {
        float v[8];
        load8(SPLITK == 1 ? c0 : c0 - rank * OWN, v);
        if (row_ok) {
          const int nb = n0 + c0;
          const int nvalid = p.N - nb >= 8 ? 8 : (p.N - nb > 0 ? p.N - nb : 0);
          float x[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int n = nb + u;
            float t = v[u] + s_bias[c0 + u];
            if (p.act == 1 && (p.act_rows == 0 || n < p.act_rows)) t = act_tanh<MODE>(t);
            x[u] = t * mk;
          }
          if (nvalid > 0) {
            if (p.C) store8_f32(p.C, (size_t)row * p.ldc + nb, x, nvalid);
            store8_operand(p, (size_t)row * p.ld_op + nb, x, nvalid);
          }
        }
      }
    } else {  // TC_EPI_LSE
      constexpr int OWN = BN / SPLITK;
      const int n0 = n_tile * BN;
      const int tg = (p.target && row_ok) ? p.target[row] - p.target_offset : -1;
      float mx = -INFINITY, sm = 0.f;
      for (int c0 = rank * OWN; c0 < (rank + 1) * OWN; c0 += 8) {
        float v[8];
        load8(SPLITK == 1 ? c0 : c0 - rank * OWN, v);
        float cm = -INFINITY;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          v[u] += s_bias[c0 + u];
          cm = fmaxf(cm, v[u]);
        }
        const int rel = tg - (n0 + c0);
        if ((unsigned)rel < 8u && tg < p.N) {  // the target's logit lies in this chunk (once per row at most)
          float t = 0.f;
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (u == rel) t = v[u];
          p.tgt_logit[row] = t;
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
        const size_t pi = ((size_t)n_tile * SPLITK + rank) * p.M + row;
        p.part_max[pi] = mx;
        p.part_sum[pi] = sm;
      }
    }
  }
  tc_fence_before();
  ZR_STAMP(7);
  // A CTA's shared memory is written by its peers only before the cluster barrier above and read by nobody else, so
  // no second cluster barrier is needed before it retires.
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

template <int BN, int MODE, int EPI, int SPLITK>
__global__ void __launch_bounds__(256, 1) tc_gemm_kernel(const __grid_constant__ TcParams p) {
  tc_gemm_body<BN, MODE, EPI, SPLITK>(p, (int)blockIdx.x);
}
// Several independent problems of one column tile each (M <= 128) in one launch: blockIdx.x selects the problem.  The
// encoder uses it for the LSTM cells of one anti-diagonal (layer l at step t, layer l-1 at step t+1, ...), which do
// not depend on one another: together they fill the SMs without splitting K, so no partial tiles are exchanged.
template <int BN, int MODE, int EPI, int SPLITK>
__global__ void __launch_bounds__(256, 1) tc_gemm_multi_kernel(const __grid_constant__ TcMulti pm) {
  tc_gemm_body<BN, MODE, EPI, SPLITK>(pm.p[blockIdx.x], 0);
}

// ------------------------------------------------------------------ persistent variant for large GEMMs
// One CTA per SM walks over output tiles (M tile fastest, so concurrently running CTAs share the same rows of B in
// L2).  The TMA producer runs ahead across tile boundaries and the accumulator is double-buffered in TMEM, so the
// epilogue of tile i overlaps the main loop of tile i+1 and the load pipe never drains.
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Warp roles: warps 0-7 run the epilogue (warp w reads TMEM lanes 32 (w % 4) .. +31, the only ones it may access, and
// the column half w / 4 of the tile), warp 8 is the TMA producer, warp 9 issues the MMAs and owns the TMEM allocation.
// Every tile therefore leaves kPersistentParts = 2 (max, sum) partials per output row, one per column half.
constexpr int kXposeBytes = 8 * 32 * 32 * 4;  // one 32 x 32 fp32 transposition buffer per epilogue warp
__host__ __device__ constexpr int persistent_stages(int BN, int mode) {
  return (225 * 1024 - 1024 - kXposeBytes) / stage_bytes(BN, mode);
}

template <int BN, int MODE, int EPI>
__global__ void __launch_bounds__(320, 1) tc_gemm_persistent_kernel(const __grid_constant__ TcParams p, int m_tiles,
                                                                     int n_tiles) {
  constexpr int ST = persistent_stages(BN, MODE);
  constexpr int STAGE = stage_bytes(BN, MODE);
  constexpr int BBYTES = BN * 128;
  constexpr uint32_t IDESC = make_idesc(mode_fmt(MODE), BN);
  constexpr int ACC_COLS = (mode_split(MODE) ? 2 : 1) * BN;  // main accumulator (+ cross-term accumulator)
  constexpr int TMEM_COLS = 2 * ACC_COLS;                       // double-buffered
  constexpr int HC = BN / kPersistentParts;                     // columns per epilogue warp
  static_assert(ST >= 2, "need at least a double-buffered ring");
  static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM budget");
  static_assert(HC % 32 == 0, "the epilogue works on chunks of 32 columns");
  static_assert(EPI != TC_EPI_LSTM, "the persistent variant has store and log-sum-exp epilogues only");
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[ST];
  __shared__ __align__(8) uint64_t empty_bar[ST];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  // bias values of the tile whose epilogue is running (two named barriers per tile order its refill)
  __shared__ __align__(16) float s_bias[BN];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const int total_tiles = m_tiles * n_tiles;
  ZR_STAMP(0);
  int kb_per_tile = 0;
  for (int s = 0; s < p.nsrc; ++s) kb_per_tile += p.kblocks[s];

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);  // one arrival per epilogue warp
    }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  pdl_wait();

  if (warp == 8) {
    // ------------------------------------------------------------ TMA producer (runs ahead across tiles)
    if (lane == 0 && kb_per_tile > 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * 128, n0 = (tile / m_tiles) * BN;
        for (int s = 0; s < p.nsrc && ok; ++s) {
          for (int kb = 0; kb < p.kblocks[s]; ++kb, ++it) {
            const int st = it % ST;
            const uint32_t ph = (uint32_t)((it / ST) & 1);
            if (!mbar_wait(&empty_bar[st], ph ^ 1u, &abort_s, p.err, 1)) { ok = false; break; }
            uint8_t* base = tiles + (size_t)st * STAGE;
            mbar_expect_tx(&full_bar[st], (uint32_t)STAGE);
            const int kx = kb * mode_epk(MODE);
            tma_load_2d(base, &p.a[s], &full_bar[st], kx, m0);
            tma_load_2d(base + kABytes, &p.b, &full_bar[st], p.b_koff[s] + kx, n0);
            if (mode_split(MODE)) {
              tma_load_2d(base + kABytes + BBYTES, &p.a_lo[s], &full_bar[st], kx, m0);
              tma_load_2d(base + 2 * kABytes + BBYTES, &p.b_lo, &full_bar[st], p.b_koff[s] + kx, n0);
            }
          }
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 20000000LL) {}
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && kb_per_tile > 0) {
      int it = 0, ti = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++ti) {
        const int buf = ti & 1;
        // wait until the epilogue has drained this accumulator buffer (passes at once on its first use)
        if (!mbar_wait(&acc_empty[buf], (uint32_t)(((ti >> 1) & 1) ^ 1), &abort_s, p.err, 4)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_main = tmem_base + (uint32_t)(buf * ACC_COLS);
        for (int kk = 0; kk < kb_per_tile; ++kk, ++it) {
          const int st = it % ST;
          const uint32_t ph = (uint32_t)((it / ST) & 1);
          if (!mbar_wait(&full_bar[st], ph, &abort_s, p.err, 2)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + (size_t)st * STAGE);
          const uint32_t b_addr = a_addr + kABytes;
          const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(b_addr);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t acc = (kk > 0 || k > 0) ? 1u : 0u;
            umma<mode_kind_tf32(MODE)>(d_main, da + 2 * k, db + 2 * k, IDESC, acc);
            if (mode_split(MODE)) {
              const uint64_t dal = make_smem_desc(b_addr + BBYTES), dbl = make_smem_desc(b_addr + BBYTES + kABytes);
              umma<mode_kind_tf32(MODE)>(d_main + BN, dal + 2 * k, db + 2 * k, IDESC, acc);
              umma<mode_kind_tf32(MODE)>(d_main + BN, da + 2 * k, dbl + 2 * k, IDESC, 1u);
            }
          }
          umma_commit(&empty_bar[st]);
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else if (kb_per_tile > 0) {
    // ------------------------------------------------------------ epilogue warps 0-7
    const int q = warp & 3, half = warp >> 2;
    float* xp = reinterpret_cast<float*>(tiles + (size_t)ST * STAGE) + warp * 1024;
    // Stores go through the warp's transposition buffer so that every store instruction writes whole 128-byte lines
    // (a thread per output row would scatter 16-byte pieces over 32 lines).  That needs 16-byte aligned rows; any
    // other layout, and launches that also emit operand copies, take the per-row path.
    const bool fast_store = EPI == TC_EPI_STORE && p.C && (p.ldc & 3) == 0 && (p.N & 3) == 0 &&
                            (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 && !p.op_b16 && !p.op_hi && !p.op_h_hi;
    int ti = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++ti) {
      const int buf = ti & 1;
      const int m_tile = tile % m_tiles, n_tile = tile / m_tiles;
      const int row = m_tile * 128 + q * 32 + lane;
      const bool row_ok = row < p.M;
      asm volatile("bar.sync 1, 256;" ::: "memory");  // all epilogue threads have finished with the previous bias
      for (int i = threadIdx.x; i < BN; i += 256) {
        const int n = n_tile * BN + i;
        s_bias[i] = n < p.N ? (p.bias ? __ldg(p.bias + n) : 0.f) : (EPI == TC_EPI_LSE ? -INFINITY : 0.f);
      }
      if (!mbar_wait(&acc_full[buf], (uint32_t)((ti >> 1) & 1), &abort_s, p.err, 3)) break;
      tc_fence_after();
      asm volatile("bar.sync 1, 256;" ::: "memory");  // the new bias values are visible
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * ACC_COLS + half * HC);
      const float mk = (p.mask && row_ok) ? (float)p.mask[row] : 1.0f;
      const int n0 = n_tile * BN + half * HC;  // first output column of this warp
      const float* sb = s_bias + half * HC;
      const size_t pi = (size_t)(n_tile * kPersistentParts + half) * p.M + row;
      if constexpr (EPI == TC_EPI_STORE) {
        const bool want_max = p.part_max != nullptr;  // also emit the maximum of this warp's stored values per row
        const bool want_lse = want_max && p.part_sum != nullptr;  // ... and sum exp(x - max)
        float mx = -INFINITY, sm = 0.f;
        for (int c0 = 0; c0 < HC; c0 += 32) {
          float v[32];
          tmem_ld32(taddr + c0, v);
          if (mode_split(MODE)) {
            float t[32];
            tmem_ld32(taddr + BN + c0, t);
            tmem_wait_ld();
#pragma unroll
            for (int u = 0; u < 32; ++u) v[u] = fmaf(t[u], mode_cross_scale(MODE), v[u]);
          }
          tmem_wait_ld();
          const int nb = n0 + c0;
          const int nvalid = p.N - nb >= 32 ? 32 : (p.N - nb > 0 ? p.N - nb : 0);
          float cm = -INFINITY;
#pragma unroll
          for (int u = 0; u < 32; u += 4) {
            const float4 b4 = *reinterpret_cast<const float4*>(sb + c0 + u);
            const float bb[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float t = v[u + e] + bb[e];
              if (p.act == 1 && (p.act_rows == 0 || nb + u + e < p.act_rows)) t = act_tanh<MODE>(t);
              t *= mk;
              v[u + e] = t;
              if (u + e < nvalid) cm = fmaxf(cm, t);
            }
          }
          if (want_lse) {
            if (cm > mx) { sm *= expf(mx - cm); mx = cm; }
            if (mx != -INFINITY) {
              float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
              for (int u = 0; u < 32; u += 4) {
                s0 += u < nvalid ? expf(v[u] - mx) : 0.f;
                s1 += u + 1 < nvalid ? expf(v[u + 1] - mx) : 0.f;
                s2 += u + 2 < nvalid ? expf(v[u + 2] - mx) : 0.f;
                s3 += u + 3 < nvalid ? expf(v[u + 3] - mx) : 0.f;
              }
              sm += (s0 + s1) + (s2 + s3);
            }
          } else if (want_max) {
            mx = fmaxf(mx, cm);
          }
          if (fast_store) {
            // row `lane` of the 32 x 32 chunk, its eight 16-byte pieces XOR-swizzled by the row so that neither
            // these writes nor the transposed reads below collide on a bank
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<float4*>(xp + lane * 32 + ((j ^ (lane & 7)) << 2)) =
                  make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {  // eight lanes per row, four rows per instruction
              const int r = 4 * i + (lane >> 3), j = lane & 7;
              const float4 o = *reinterpret_cast<const float4*>(xp + r * 32 + ((j ^ (r & 7)) << 2));
              const int grow = m_tile * 128 + q * 32 + r, n = nb + 4 * j;
              // streaming stores: the consumer reads a few tiles of the logits once, the weights should stay in L2
              if (grow < p.M && n < p.N) __stcs(reinterpret_cast<float4*>(p.C + (size_t)grow * p.ldc + n), o);
            }
            __syncwarp();
          } else if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int nv = nvalid - 8 * g >= 8 ? 8 : (nvalid - 8 * g > 0 ? nvalid - 8 * g : 0);
              if (nv > 0) {
                float x8[8];  // a copy: the ragged tail indexes it dynamically, which must not push v out of registers
#pragma unroll
                for (int u = 0; u < 8; ++u) x8[u] = v[8 * g + u];
                if (p.C) store8_f32(p.C, (size_t)row * p.ldc + nb + 8 * g, x8, nv);
                store8_operand(p, (size_t)row * p.ld_op + nb + 8 * g, x8, nv);
              }
            }
          }
        }
        if (want_max && row_ok) {
          p.part_max[pi] = mx;
          if (want_lse) p.part_sum[pi] = sm;
        }
      } else {  // TC_EPI_LSE
        const int tg = (p.target && row_ok) ? p.target[row] - p.target_offset : -1;
        float mx = -INFINITY, sm = 0.f;
        for (int c0 = 0; c0 < HC; c0 += 32) {
          float v[32];
          tmem_ld32(taddr + c0, v);
          if (mode_split(MODE)) {
            float t[32];
            tmem_ld32(taddr + BN + c0, t);
            tmem_wait_ld();
#pragma unroll
            for (int u = 0; u < 32; ++u) v[u] = fmaf(t[u], mode_cross_scale(MODE), v[u]);
          }
          tmem_wait_ld();
          float cm = -INFINITY;
#pragma unroll
          for (int u = 0; u < 32; u += 4) {
            const float4 b4 = *reinterpret_cast<const float4*>(sb + c0 + u);
            v[u] += b4.x; v[u + 1] += b4.y; v[u + 2] += b4.z; v[u + 3] += b4.w;
            cm = fmaxf(fmaxf(cm, fmaxf(v[u], v[u + 1])), fmaxf(v[u + 2], v[u + 3]));
          }
          const int rel = tg - (n0 + c0);
          if ((unsigned)rel < 32u && tg < p.N) {  // the target's logit lies in this chunk (once per row at most)
            float t = 0.f;
#pragma unroll
            for (int u = 0; u < 32; ++u)
              if (u == rel) t = v[u];
            p.tgt_logit[row] = t;
          }
          if (cm > mx) {
            sm *= expf(mx - cm);
            mx = cm;
          }
          if (mx != -INFINITY) {
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int u = 0; u < 32; u += 4) {
              s0 += expf(v[u] - mx); s1 += expf(v[u + 1] - mx); s2 += expf(v[u + 2] - mx); s3 += expf(v[u + 3] - mx);
            }
            sm += (s0 + s1) + (s2 + s3);
          }
        }
        if (row_ok) {
          p.part_max[pi] = mx;
          p.part_sum[pi] = sm;
        }
      }
      // this warp's TMEM reads are complete: hand the buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  ZR_STAMP(7);
  if (warp == 9) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

constexpr int kMaxDevices = 64;
static int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  return dev;
}
static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int BN, int MODE, int EPI>
cudaError_t launch_persistent_t(const TcParams& p, cudaStream_t st) {
  const size_t smem = (size_t)persistent_stages(BN, MODE) * stage_bytes(BN, MODE) + 1024 + kXposeBytes;
  static bool configured[kMaxDevices] = {false};  // the attribute is per device
  const int dev = current_device();
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tc_gemm_persistent_kernel<BN, MODE, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int m_tiles = (p.M + 127) / 128, n_tiles = (p.N + BN - 1) / BN;
  const int total = m_tiles * n_tiles;
  if (total == 0) return cudaSuccess;
  const int grid = total < sm_count() ? total : sm_count();
  tc_gemm_persistent_kernel<BN, MODE, EPI><<<grid, 320, smem, st>>>(p, m_tiles, n_tiles);
  count_launch();
  return cudaGetLastError();
}

static const bool g_use_pdl = std::getenv("ZRNN_NO_PDL") == nullptr;

template <int BN, int MODE, int EPI, int SPLITK>
cudaError_t launch_t(const TcParams& p, cudaStream_t st) {
  const size_t smem = (size_t)smem_bytes(BN, MODE, SPLITK);
  static bool configured[kMaxDevices] = {false};  // once per instantiation and device
  const int dev = current_device();
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tc_gemm_kernel<BN, MODE, EPI, SPLITK>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int n_rows = (EPI == TC_EPI_LSTM) ? p.N * 4 : p.N;
  dim3 grid((p.M + 127) / 128, (n_rows + BN - 1) / BN, SPLITK);
  if (grid.x == 0 || grid.y == 0) return cudaSuccess;
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = dim3((EPI == TC_EPI_LSTM && SPLITK > 1 && BN / 4 / SPLITK == 8) ? 256 : 192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (g_use_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (SPLITK > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = SPLITK;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, tc_gemm_kernel<BN, MODE, EPI, SPLITK>, p);
  count_launch();
  return e;
}

template <int MODE, int SPLITK>
cudaError_t launch_multi_t(const TcMulti& pm, int n, cudaStream_t st) {
  constexpr int BN = 128;
  const size_t smem = (size_t)smem_bytes(BN, MODE, SPLITK);
  static bool configured[kMaxDevices] = {false};
  const int dev = current_device();
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tc_gemm_multi_kernel<BN, MODE, TC_EPI_LSTM, SPLITK>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  dim3 grid(n, (pm.p[0].N * 4 + BN - 1) / BN, SPLITK);
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = dim3((SPLITK > 1 && BN / 4 / SPLITK == 8) ? 256 : 192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (g_use_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (SPLITK > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = SPLITK;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, tc_gemm_multi_kernel<BN, MODE, TC_EPI_LSTM, SPLITK>, pm);
  count_launch();
  return e;
}
template <int MODE>
cudaError_t launch_multi_mode(const TcMulti& pm, int n, int splitk, cudaStream_t st) {
  switch (splitk) {
    case 1: return launch_multi_t<MODE, 1>(pm, n, st);
    case 2: return launch_multi_t<MODE, 2>(pm, n, st);
    case 4: return launch_multi_t<MODE, 4>(pm, n, st);
  }
  return cudaErrorInvalidValue;
}

template <int MODE, int EPI>
cudaError_t launch_bn(const TcParams& p, int BN, int splitk, cudaStream_t st) {
  if (splitk == 1) {
    switch (BN) {
      case 32: return launch_t<32, MODE, EPI, 1>(p, st);
      case 64: return launch_t<64, MODE, EPI, 1>(p, st);
      case 128: return launch_t<128, MODE, EPI, 1>(p, st);
      case 256: return launch_t<256, MODE, EPI, 1>(p, st);
    }
  } else if (BN == 128) {  // split-K variants exist for the 128-column tile only
    switch (splitk) {
      case 2: return launch_t<128, MODE, EPI, 2>(p, st);
      case 4: return launch_t<128, MODE, EPI, 4>(p, st);
    }
    if constexpr (EPI != TC_EPI_LSTM) {
      if (splitk == 8) return launch_t<128, MODE, EPI, 8>(p, st);
    }
  }
  return cudaErrorInvalidValue;
}
template <int MODE>
cudaError_t launch_epi(const TcParams& p, int BN, int epi, int splitk, cudaStream_t st) {
  switch (epi) {
    case TC_EPI_STORE: return launch_bn<MODE, TC_EPI_STORE>(p, BN, splitk, st);
    case TC_EPI_LSTM: return launch_bn<MODE, TC_EPI_LSTM>(p, BN, splitk, st);
    case TC_EPI_LSE: return launch_bn<MODE, TC_EPI_LSE>(p, BN, splitk, st);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_tc_gemm_persistent(const TcParams& p, int mode, int epi, cudaStream_t st) {
  // tile widths: 256 columns for bf16 / tf32, 128 for 3xTF32 (its second, cross-term accumulator doubles the TMEM need)
  if (epi == TC_EPI_LSE) {
    if (mode == TC_BF16) return launch_persistent_t<256, TC_BF16, TC_EPI_LSE>(p, st);
    if (mode == TC_TF32) return launch_persistent_t<256, TC_TF32, TC_EPI_LSE>(p, st);
    if (mode == TC_TF32X3) return launch_persistent_t<128, TC_TF32X3, TC_EPI_LSE>(p, st);
    if (mode == TC_F16X2) return launch_persistent_t<128, TC_F16X2, TC_EPI_LSE>(p, st);
  } else if (epi == TC_EPI_STORE) {
    if (mode == TC_BF16) return launch_persistent_t<256, TC_BF16, TC_EPI_STORE>(p, st);
    if (mode == TC_TF32) return launch_persistent_t<256, TC_TF32, TC_EPI_STORE>(p, st);
    if (mode == TC_TF32X3) return launch_persistent_t<128, TC_TF32X3, TC_EPI_STORE>(p, st);
    if (mode == TC_F16X2) return launch_persistent_t<128, TC_F16X2, TC_EPI_STORE>(p, st);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_tc_lstm_multi(const TcMulti& pm, int n, int mode, cudaStream_t st, int splitk) {
  if (n < 1 || n > TcMulti::MAX) return cudaErrorInvalidValue;
  for (int i = 0; i < n; ++i)
    if (pm.p[i].M > 128 || pm.p[i].M < 1 || pm.p[i].N != pm.p[0].N) return cudaErrorInvalidValue;
  switch (mode) {
    case TC_BF16: return launch_multi_mode<TC_BF16>(pm, n, splitk, st);
    case TC_TF32: return launch_multi_mode<TC_TF32>(pm, n, splitk, st);
    case TC_TF32X3: return launch_multi_mode<TC_TF32X3>(pm, n, splitk, st);
    case TC_F16X2: return launch_multi_mode<TC_F16X2>(pm, n, splitk, st);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_tc_gemm(const TcParams& p, int BN, int mode, int epi, cudaStream_t st, int splitk) {
  switch (mode) {
    case TC_BF16: return launch_epi<TC_BF16>(p, BN, epi, splitk, st);
    case TC_TF32: return launch_epi<TC_TF32>(p, BN, epi, splitk, st);
    case TC_TF32X3: return launch_epi<TC_TF32X3>(p, BN, epi, splitk, st);
    case TC_F16X2: return launch_epi<TC_F16X2>(p, BN, epi, splitk, st);
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
