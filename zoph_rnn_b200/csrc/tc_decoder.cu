// Persistent decoder kernel for sm_100a (see tc_decoder.cuh for what it replaces and why).
//
// Work split.  A time step is a fixed list of phases: the L cells, [local-p: the stacked [W_p ; W_a^T] GEMM], the
// attention proper (SIMT, one target column per CTA in turn), the tanh combiner GEMM - a strict chain, every phase
// needs the one before it.  What bounds such a chain is latency (hand-over, pipeline fill, exchange, epilogue), not
// bytes, so the batch is cut into `groups` column groups that run the chain independently of one another, each on
// its own share of the clusters with its own phase counter: while one group hands a phase over, the others keep the
// memory system and the tensor pipe busy.  (Each group streams the weights itself; HBM has the room.)
// Inside a group, cluster c owns the row tiles c, c + NC, ... of a GEMM phase (128 packed weight rows = 32 hidden
// units x 4 gates each) and its four CTAs each take a quarter of every source's k-blocks, accumulate in tensor
// memory, push the three quarters of the partial tile that they do not own into the owners' shared memory
// (st.shared::cluster), and finish their own 32 columns: gate math and state update, or bias + tanh + mask.
//
// CTA = 10 warps.  Warps 0-7 are the epilogue team, warp 8 lane 0 is the TMA producer, warp 9 lane 0 issues the MMAs
// and warp 9 owns the tensor-memory allocation.  Weights and activations have rings of their own:
//   * weight tiles depend on nothing, so the producer streams them as far ahead as the ring allows - across phase
//     boundaries, i.e. while the current phase's exchange, gate math and the grid-wide hand-over run;
//   * an activation k-block is requested as soon as the phase that wrote it is complete.  A source that was written a
//     whole step ago (the layer's own h of step t - 1) or before the kernel (the gathered inputs) comes first in every
//     CTA's k-block order, so its MMAs are issued before the phase's last input exists;
//   * the exchange slots have memory of their own (the attention scratch aliases them), so a CTA pushes its partial
//     tile as soon as its own accumulators are complete: a slot is only written for phase q after the phase's last
//     input exists, i.e. after phase q - 1 is complete everywhere, which includes its owner's reads of phase q - 1.
// Phases hand over through one monotonic counter in global memory: a CTA adds 1 when its part of a phase is stored;
// phase q is complete at (q + 1) * CTAs.  Every wait is bounded (about a second of SM clock); a wait that gives up
// records where in p.err and makes every role of every CTA leave, so the kernel always returns.
#include "tc_decoder.cuh"

#include <cstdint>
#include <cstdlib>
#include <cstring>

#include "att_device.cuh"
#include "kernels.cuh"
#include "tc_device.cuh"

namespace zrnn {
namespace {

constexpr int kBN = 128;     // packed weight rows per tile
constexpr int kSplit = 4;    // CTAs per cluster = K split
constexpr int kOwn = kBN / kSplit;  // tile columns finished by one CTA
constexpr int kTeam = 256;   // epilogue threads
constexpr int kThreads = 320;
constexpr long long kWaitCycles = 2000000000LL;  // about a second of SM clock
constexpr int kSlotBytes = kSplit * 128 * kOwn * 4;  // 64 KB: four partial tiles of 128 rows x 32 columns, or two sets for 64 rows
constexpr int kARingBytes = 64 * 1024;               // activation ring
constexpr int kMaxAStages = 8;

__host__ __device__ constexpr int dec_wstage(int mode) { return (mode_split(mode) ? 2 : 1) * kBN * 128; }
__host__ __device__ constexpr int dec_nw(int mode) { return 96 * 1024 / dec_wstage(mode); }  // 3 (split) or 6
// The MMAs always read 128 activation rows; when a group has fewer columns only that many rows are loaded and the
// rest of the 128-row operand window is whatever follows in shared memory (rows nobody looks at; the window of the
// last stage runs into the exchange slots, which lie behind the ring).
__host__ __device__ constexpr int dec_smem(int mode) {
  return dec_nw(mode) * dec_wstage(mode) + kARingBytes + kSlotBytes + 1024;
}

enum { PH_CELL = 0, PH_PGEMM = 1, PH_ATT = 2, PH_COMB = 3 };
// developer timeline: CTA `detail_cta` leaves 8 %globaltimer stamps per phase in p.detail[ph * 8 ..]
#define ZD_STAMP(k)                                                                                        \
  do {                                                                                                     \
    if (p.detail && tid == 0) {                                                                            \
      if (p.detail_cta < 0) p.detail[((size_t)cta_all * NP + ph) * 8 + (k)] = gtime();                     \
      else if (cta_all == p.detail_cta) p.detail[(size_t)ph * 8 + (k)] = gtime();                          \
    }                                                                                                      \
  } while (0)

// What one CTA does for one row tile of one phase.
struct Plan {
  int kind, layer, t;
  int n_tiles;   // GEMM phases: 128-row tiles of the weight matrix
  int nsrc;      // sources in the order their k-blocks are issued (oldest data first)
  int src[3];    // position of the source inside the weight matrix's K axis
  int need[3];   // phase that must be complete before the source may be read (-1: written before the kernel)
  int lo[3], cnt[3];  // this CTA's k-block slice of each source
  int nitems;    // k-blocks this CTA accumulates (0 for a tile beyond the phase's tiles and for the attention phase)
};

__device__ __forceinline__ void make_plan(const DecParams& p, int ph, int P, int rank, int tile, Plan& pl) {
  const int t = ph / P, j = ph - t * P, L = p.L;
  pl.t = t;
  pl.layer = 0;
  pl.nsrc = 0;
  pl.nitems = 0;
  pl.n_tiles = 0;
  if (j < L) {
    pl.kind = PH_CELL;
    pl.layer = j;
    pl.n_tiles = (4 * p.H + kBN - 1) / kBN;
    if (j == 0) {
      pl.src[0] = 0; pl.need[0] = -1;                                  // gathered inputs
      pl.src[1] = 1; pl.need[1] = t > 0 ? ph - P : -1;                 // own h of step t - 1
      pl.nsrc = 2;
      if (t > 0) { pl.src[2] = 2; pl.need[2] = ph - 1; pl.nsrc = 3; }  // attention output of step t - 1
    } else {
      pl.src[0] = 1; pl.need[0] = t > 0 ? ph - P : -1;
      pl.src[1] = 0; pl.need[1] = ph - 1;                              // h of the layer below, this step
      pl.nsrc = 2;
    }
  } else if (p.att_type == 1 && j == L) {
    pl.kind = PH_PGEMM;
    pl.n_tiles = (2 * p.H + kBN - 1) / kBN;
    pl.src[0] = 0; pl.need[0] = ph - 1;
    pl.nsrc = 1;
  } else if (j == P - 2) {
    pl.kind = PH_ATT;
  } else {
    pl.kind = PH_COMB;
    pl.n_tiles = (p.H + kBN - 1) / kBN;
    pl.src[0] = 1; pl.need[0] = t * P + L - 1;   // top-layer h of this step
    pl.src[1] = 0; pl.need[1] = ph - 1;          // context
    pl.nsrc = 2;
  }
  if (pl.kind == PH_ATT || tile >= pl.n_tiles) { pl.nsrc = 0; return; }
  for (int s = 0; s < pl.nsrc; ++s) {
    pl.lo[s] = (p.kb * rank) / kSplit;
    pl.cnt[s] = (p.kb * (rank + 1)) / kSplit - pl.lo[s];
    pl.nitems += pl.cnt[s];
  }
}

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* ptr) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_cta_shared(const int* ptr) {
  int v;
  asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32(ptr)) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_cta_shared(int* ptr, int v) {
  asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(smem_u32(ptr)), "r"(v) : "memory");
}
// Weight tiles are read once per phase and do not fit the L2 over a step: stream them with an evict-first policy so
// that they do not push out what is re-read (the activations of the last steps, the attention's source memory).
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      :
      : "r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// the non-blocking form: try_wait may suspend the thread for a while before it answers "not yet", which a loop that
// has other things to look at cannot afford
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// arrive on the same barrier in the shared memory of cluster rank `rank`; orders this thread's earlier remote stores
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t rank) {
  const uint32_t addr = cluster_map(smem_u32(bar), rank);
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_local(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void team_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
struct SyncTeam {
  __device__ __forceinline__ void operator()() const { team_sync(); }
};

// Bounded wait on any condition.  Gives up when another role of this CTA has (abort flag), when any CTA has (the
// device error word) or after kWaitCycles; `code` says where.
template <class Pred>
__device__ __forceinline__ bool bounded_wait(Pred ready, volatile int* abort_s, int* gerr, int code) {
  if (ready()) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (!ready()) {
    if ((++spins & 63) == 0) {
      if (*abort_s) return false;
      if ((spins & 1023) == 0 && *reinterpret_cast<volatile int*>(gerr) != 0) { *abort_s = 1; return false; }
      if (clock64() - t0 > kWaitCycles) {
        *abort_s = 1;
        atomicCAS(gerr, 0, code);
        return false;
      }
    }
  }
  return true;
}

// The same for a whole warp: lane 0 polls (32 lanes spinning on one barrier word compete with the remote stores that
// the wait is for), the other lanes join through the warp barrier, which also orders their later reads after the
// acquire.  Every lane returns whether the wait succeeded.
template <class Pred>
__device__ __forceinline__ bool warp_bounded_wait(Pred ready, int lane, volatile int* abort_s, int* gerr, int code) {
  int ok = 1;
  if (lane == 0) ok = bounded_wait(ready, abort_s, gerr, code) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}

struct OpOut {  // where an epilogue leaves the operand-form copy of a row (see store4_operand)
  __nv_bfloat16* op_b16;
  float* op_hi;
  float* op_lo;
  __half* op_h_hi;
  __half* op_h_lo;
};
template <int MODE>
__device__ __forceinline__ OpOut make_opout(void* hi, void* lo) {
  OpOut o;
  o.op_b16 = MODE == TC_BF16 ? (__nv_bfloat16*)hi : nullptr;
  o.op_h_hi = MODE == TC_F16X2 ? (__half*)hi : nullptr;
  o.op_h_lo = MODE == TC_F16X2 ? (__half*)lo : nullptr;
  o.op_hi = (MODE == TC_TF32 || MODE == TC_TF32X3) ? (float*)hi : nullptr;
  o.op_lo = MODE == TC_TF32X3 ? (float*)lo : nullptr;
  return o;
}

// The slice of the batch one column group works on, and the share of the clusters that works on it.
struct Group {
  int b0, nb;     // first column and number of columns
  int cl, NC;     // this cluster's index inside the group and the group's number of clusters
  int TPC;        // row tiles of the largest phase that one cluster takes in turn
  unsigned G;     // CTAs of the group (what one complete phase adds to the group's counter)
  unsigned* counter;
};

// One item = one 128-byte k-block of one source: which activation rows and which weight rows feed it.
struct Item {
  const CUtensorMap *a_hi, *a_lo, *w_hi, *w_lo;
  int ax, ay, wx, wy;
  int need;
};
__device__ __forceinline__ void make_item(const DecParams& p, const Plan& pl, int s, int kbi, int tile, int b0, int epk,
                                          Item& it) {
  const int sid = pl.src[s], t = pl.t, Bs = p.B;
  it.need = pl.need[s];
  it.ax = kbi * epk;
  if (pl.kind == PH_CELL) {
    const int l = pl.layer;
    if (sid == 0) {
      if (l == 0) { it.a_hi = &p.x_hi; it.a_lo = &p.x_lo; }
      else { it.a_hi = &p.h_hi[l - 1]; it.a_lo = &p.h_lo[l - 1]; }
      it.ay = t * Bs + b0;
    } else if (sid == 1) {
      if (t == 0) { it.a_hi = &p.h0_hi[l]; it.a_lo = &p.h0_lo[l]; it.ay = p.h0_row[l] + b0; }
      else { it.a_hi = &p.h_hi[l]; it.a_lo = &p.h_lo[l]; it.ay = (t - 1) * Bs + b0; }
    } else {
      it.a_hi = &p.ht_hi; it.a_lo = &p.ht_lo;
      it.ay = (t - 1) * Bs + b0;
    }
    it.w_hi = &p.w_hi[l]; it.w_lo = &p.w_lo[l];
    const int kbg = sid * p.kpb + kbi;
    if (p.w_tiled[l] > 0) { it.wx = 0; it.wy = (tile * p.w_tiled[l] + kbg) * kBN; }
    else { it.wx = kbg * epk; it.wy = tile * kBN; }
  } else if (pl.kind == PH_PGEMM) {
    it.a_hi = &p.h_hi[p.L - 1]; it.a_lo = &p.h_lo[p.L - 1];
    it.ay = t * Bs + b0;
    it.w_hi = &p.wp_hi; it.w_lo = &p.wp_lo;
    it.wx = kbi * epk; it.wy = tile * kBN;
  } else {  // PH_COMB
    if (sid == 0) { it.a_hi = &p.ctx_hi; it.a_lo = &p.ctx_lo; it.ay = b0; }
    else { it.a_hi = &p.h_hi[p.L - 1]; it.a_lo = &p.h_lo[p.L - 1]; it.ay = t * Bs + b0; }
    it.w_hi = &p.wc_hi; it.w_lo = &p.wc_lo;
    it.wx = (sid * p.kpb + kbi) * epk; it.wy = tile * kBN;
  }
}

// Walks over this CTA's items in issue order: phase after phase, inside a phase tile after tile.
struct Cursor {
  int ph, ti, s, k;  // phase, tile round, source (in issue order), k-block inside this CTA's slice of the source
  int tile;
  Plan pl;
  bool end;
  __device__ __forceinline__ void seek(const DecParams& p, int NP, int P, int rank, const Group& gr) {
    while (ph < NP) {
      for (; ti < gr.TPC; ++ti) {
        tile = gr.cl + ti * gr.NC;
        make_plan(p, ph, P, rank, tile, pl);
        s = 0;
        while (s < pl.nsrc && pl.cnt[s] == 0) ++s;
        if (s < pl.nsrc) { k = 0; end = false; return; }
      }
      ++ph;
      ti = 0;
    }
    end = true;
  }
  __device__ __forceinline__ void start(const DecParams& p, int NP, int P, int rank, const Group& gr) {
    ph = 0;
    ti = 0;
    seek(p, NP, P, rank, gr);
  }
  __device__ __forceinline__ void advance(const DecParams& p, int NP, int P, int rank, const Group& gr) {
    if (++k < pl.cnt[s]) return;
    k = 0;
    do { ++s; } while (s < pl.nsrc && pl.cnt[s] == 0);
    if (s < pl.nsrc) return;
    ++ti;
    seek(p, NP, P, rank, gr);
  }
};

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1) tc_decoder_kernel(const __grid_constant__ DecParams p) {
  constexpr int NW = dec_nw(MODE);
  constexpr int WSTAGE = dec_wstage(MODE);
  constexpr int HALF = 128 * 128;  // bytes of one operand part (hi or lo) of a weight stage
  constexpr int PARTS = mode_split(MODE) ? 2 : 1;
  constexpr int EPK = mode_epk(MODE);
  constexpr uint32_t IDESC = make_idesc(mode_fmt(MODE), kBN);
  constexpr int NACC = num_acc(kBN, MODE);
  constexpr int TMEM_COLS = tmem_cols(kBN, MODE);
  static_assert(kSlotBytes >= kAttGlobalScratchBytes && kSlotBytes >= kAttLocalScratchBytes, "attention scratch");
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t wfull[NW], wempty[NW], afull[kMaxAStages], aempty[kMaxAStages];
  __shared__ __align__(8) uint64_t accum_bar, tmem_free, xchg_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int in_exchange;  // the team is exchanging partial tiles: the producer holds back its loads meanwhile
  __shared__ int prod_done;    // phases the producer has seen complete (saves the team a look at the global counter)
  __shared__ float s_bias[kBN];
  __shared__ long long s_push[kTeam / 32];  // developer timeline: when each warp finished pushing

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int rank = (int)blockIdx.x;  // cluster dims (4,1,1): rank in cluster == blockIdx.x
  Group gr;
  {
    const int groups = (int)gridDim.z, gi = (int)blockIdx.z;
    const int Bv = (p.B + groups - 1) / groups;
    gr.b0 = gi * Bv;
    gr.nb = p.B - gr.b0 < Bv ? p.B - gr.b0 : Bv;
    if (gr.nb < 0) gr.nb = 0;
    gr.cl = (int)blockIdx.y;
    gr.NC = (int)gridDim.y;
    gr.TPC = ((4 * p.H + kBN - 1) / kBN + gr.NC - 1) / gr.NC;
    gr.G = gridDim.x * gridDim.y;
    gr.counter = p.counter + 32 * gi;  // 128 bytes apart
  }
  const unsigned G = gr.G;
  const int cta_id = (int)(blockIdx.y * gridDim.x + blockIdx.x);       // inside the group
  const int cta_all = (int)blockIdx.z * (int)G + cta_id;               // inside the grid
  const int P = p.L + (p.att_type == 1 ? 3 : 2), NP = p.T * P;
  // activation stages hold a_rows rows per part; the ring has as many of them as fit (at most kMaxAStages)
  const int a_rows = p.a_rows;
  const int APART = a_rows * 128, ASTAGE = PARTS * APART;
  const int NA = kARingBytes / ASTAGE < kMaxAStages ? kARingBytes / ASTAGE : kMaxAStages;
  // exchange slots: [set][rank][8 column quads][SR rows] float4; two sets when 64 rows are enough, used in turn by
  // consecutive tiles (a peer may push the next tile while this CTA still reads the previous one)
  const int SR = a_rows <= 64 ? 64 : 128;
  const int slot_sets = SR == 64 ? 2 : 1;
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  uint8_t* wring = base;
  uint8_t* aring = base + (size_t)NW * WSTAGE;
  float4* slots_all = reinterpret_cast<float4*>(aring + kARingBytes);
  unsigned char* scratch = reinterpret_cast<unsigned char*>(slots_all);  // attention phases: nobody exchanges then

  if (tid == 0) {
    for (int s = 0; s < NW; ++s) { mbar_init(&wfull[s], 1); mbar_init(&wempty[s], 1); }
    for (int s = 0; s < kMaxAStages; ++s) { mbar_init(&afull[s], 1); mbar_init(&aempty[s], 1); }
    mbar_init(&accum_bar, 1);
    mbar_init(&tmem_free, kTeam / 32);
    mbar_init(&xchg_bar, kSplit * (kTeam / 32));
    abort_s = 0;
    in_exchange = 0;
    prod_done = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (p.stamps && cta_all == 0) p.stamps[0] = gtime();
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // every CTA's barriers exist before a peer arrives on them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* ab = &abort_s;

  if (gr.nb <= 0) {
    // a group without columns (more groups than the batch can fill): nothing to do, nobody waits for it
  } else if (warp == 8) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t w_policy = p.w_evict_first ? policy_evict_first() : 0;
      Cursor wc, ac;  // weights, activations
      wc.start(p, NP, P, rank, gr);
      ac.start(p, NP, P, rank, gr);
      int w_it = 0, a_it = 0;
      unsigned done_phases = 0;  // phases known to be complete
      long long t_progress = clock64();
      int idle = 0;
      bool ok = true;
      while (!ac.end) {
        bool progressed = false;
        const bool hold = p.hold_loads && *reinterpret_cast<volatile int*>(&in_exchange) != 0;
        // weights: as far ahead as the ring allows
        if (!hold && !wc.end && w_it < a_it + NW) {
          const int st = w_it % NW;
          if (mbar_test_wait(&wempty[st], (uint32_t)(((w_it / NW) & 1) ^ 1))) {
            Item it;
            make_item(p, wc.pl, wc.s, wc.pl.lo[wc.s] + wc.k, wc.tile, gr.b0, EPK, it);
            uint8_t* dst = wring + (size_t)st * WSTAGE;
            mbar_expect_tx(&wfull[st], (uint32_t)WSTAGE);
            if (w_policy) {
              tma_load_2d_hint(dst, it.w_hi, &wfull[st], it.wx, it.wy, w_policy);
              if (mode_split(MODE)) tma_load_2d_hint(dst + HALF, it.w_lo, &wfull[st], it.wx, it.wy, w_policy);
            } else {
              tma_load_2d(dst, it.w_hi, &wfull[st], it.wx, it.wy);
              if (mode_split(MODE)) tma_load_2d(dst + HALF, it.w_lo, &wfull[st], it.wx, it.wy);
            }
            ++w_it;
            wc.advance(p, NP, P, rank, gr);
            progressed = true;
          }
        }
        // activations: the next k-block, once its data exists and its stage is free
        {
          bool can = !hold;
          Item it;
          make_item(p, ac.pl, ac.s, ac.pl.lo[ac.s] + ac.k, ac.tile, gr.b0, EPK, it);
          if (it.need >= 0 && (unsigned)(it.need + 1) > done_phases) {
            const unsigned c = ld_acquire_gpu(gr.counter);
            if (c / G != done_phases) {
              done_phases = c / G;
              st_release_cta_shared(&prod_done, (int)done_phases);
            }
            if ((unsigned)(it.need + 1) > done_phases) can = false;
            else fence_proxy_async();  // the rows were written with ordinary stores; TMA reads them
          }
          const int st = a_it % NA;
          if (can && !mbar_test_wait(&aempty[st], (uint32_t)(((a_it / NA) & 1) ^ 1))) can = false;
          if (can) {
            uint8_t* dst = aring + (size_t)st * ASTAGE;
            mbar_expect_tx(&afull[st], (uint32_t)ASTAGE);
            tma_load_2d(dst, it.a_hi, &afull[st], it.ax, it.ay);
            if (mode_split(MODE)) tma_load_2d(dst + APART, it.a_lo, &afull[st], it.ax, it.ay);
            ++a_it;
            ac.advance(p, NP, P, rank, gr);
            progressed = true;
          }
        }
        if (progressed) {
          t_progress = clock64();
          idle = 0;
        } else if ((++idle & 63) == 0) {
          if (*ab) { ok = false; break; }
          if ((idle & 1023) == 0 && *reinterpret_cast<volatile int*>(p.err) != 0) { *ab = 1; ok = false; break; }
          if (clock64() - t_progress > kWaitCycles) {
            *ab = 1;
            atomicCAS(p.err, 0, 100000 + ac.ph);
            ok = false;
            break;
          }
        }
      }
      if (!ok) {  // give copies already in flight time to land before the CTA may retire
        const long long t0 = clock64();
        while (clock64() - t0 < 20000000LL) {}
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int it = 0, g = 0;
      bool ok = true;
      Plan pl;
      for (int ph = 0; ph < NP && ok; ++ph) {
        for (int ti = 0; ti < gr.TPC && ok; ++ti) {
          const int tile = gr.cl + ti * gr.NC;
          make_plan(p, ph, P, rank, tile, pl);
          if (pl.kind == PH_ATT || tile >= pl.n_tiles) continue;
          if (g > 0) {  // the team has read the previous tile's accumulators
            ok = bounded_wait([&] { return mbar_try_wait(&tmem_free, (uint32_t)((g - 1) & 1)); }, ab, p.err, 200000 + ph);
            if (!ok) break;
          }
          tc_fence_after();
          for (int i = 0; i < pl.nitems; ++i, ++it) {
            const int ws = it % NW, as = it % NA;
            ok = bounded_wait([&] { return mbar_try_wait(&wfull[ws], (uint32_t)((it / NW) & 1)); }, ab, p.err, 300000 + ph) &&
                 bounded_wait([&] { return mbar_try_wait(&afull[as], (uint32_t)((it / NA) & 1)); }, ab, p.err, 400000 + ph);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_addr = smem_u32(aring + (size_t)as * ASTAGE), b_addr = smem_u32(wring + (size_t)ws * WSTAGE);
            const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(b_addr);
            const uint32_t d_main = tmem_base + (uint32_t)((i % NACC) * kBN);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              umma<mode_kind_tf32(MODE)>(d_main, da + 2 * k, db + 2 * k, IDESC, (i >= NACC || k > 0) ? 1u : 0u);
              if (mode_split(MODE)) {
                const uint64_t dal = make_smem_desc(a_addr + (uint32_t)APART), dbl = make_smem_desc(b_addr + HALF);
                const uint32_t d_cross = tmem_base + (uint32_t)(NACC * kBN);
                umma<mode_kind_tf32(MODE)>(d_cross, dal + 2 * k, db + 2 * k, IDESC, (i > 0 || k > 0) ? 1u : 0u);
                umma<mode_kind_tf32(MODE)>(d_cross, da + 2 * k, dbl + 2 * k, IDESC, 1u);
              }
            }
            umma_commit(&wempty[ws]);
            umma_commit(&aempty[as]);
          }
          if (ok) {
            if (pl.nitems > 0) umma_commit(&accum_bar);
            else mbar_arrive_local(&accum_bar);  // nothing to accumulate (fewer k-blocks than CTAs): the team reads zeros
          }
          ++g;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue team (warps 0-7)
    const int q = warp & 3, chalf = warp >> 2;     // TMEM lane quadrant and column half read by this warp
    const int lrow = q * 32 + lane;                // tile row (= batch column) behind this thread's TMEM lane
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
    const int r = tid & 127, whalf = tid >> 7;     // after the exchange: row r, half whalf of this CTA's columns
    const int H = p.H, Bs = p.B, b0 = gr.b0, nb = gr.nb;
    const bool my_rows = q * 32 < SR;              // this warp's accumulator rows can hold columns of the group
    int g = 0;
    unsigned done_phases = 0;
    Plan pl;
    for (int ph = 0; ph < NP; ++ph) {
      make_plan(p, ph, P, rank, gr.cl, pl);
      const int t = pl.t;
      const int* mask = p.mask + (size_t)t * Bs + b0;
      ZD_STAMP(0);
      if (pl.kind == PH_ATT) {
        // ---- attention proper: scores, softmax, context; one column per CTA in turn
        if (tid == 0) {
          const unsigned want = (unsigned)ph * G;  // phases 0 .. ph-1 complete
          bounded_wait([&] { return ld_acquire_gpu(gr.counter) >= want; }, ab, p.err, 500000 + ph);
        }
        ZD_STAMP(1);
        team_sync();
        if (!*ab) {
          AttArgs a;
          a.H = H; a.B = Bs; a.D = p.D; a.S_max = p.S_max; a.B_src = Bs; a.cols_per_sent = 1;
          a.hs = p.hs; a.len = p.len; a.offset = p.off; a.mask = p.mask + (size_t)t * Bs;
          a.h_t = p.h_f32[p.L - 1] + (size_t)t * Bs * H;
          a.tanh1 = p.tq; a.q = p.tq ? p.tq + H : nullptr; a.ld_tq = 2 * H; a.v_p = p.v_p;
          a.c_t = p.ctx_f32; a.align_out = nullptr; a.align_by_pos = 0; a.viterbi_out = nullptr; a.viterbi_init = -1.f;
          a.op_b16 = MODE == TC_BF16 ? p.ctx_op_hi : nullptr;
          a.op_h_hi = MODE == TC_F16X2 ? p.ctx_op_hi : nullptr;
          a.op_h_lo = MODE == TC_F16X2 ? p.ctx_op_lo : nullptr;
          a.op_hi = (MODE == TC_TF32 || MODE == TC_TF32X3) ? (float*)p.ctx_op_hi : nullptr;
          a.op_lo = MODE == TC_TF32X3 ? (float*)p.ctx_op_lo : nullptr;
          a.ld_op = p.Kpad;
          for (int b = b0 + cta_id; b < b0 + nb; b += (int)G) {
            if (p.att_type == 1) att_local_fast_body(a, b, tid, scratch, SyncTeam());
            else att_global_fast_body(a, b, tid, scratch, SyncTeam());
            team_sync();  // the scratch is free for the next column
          }
        }
      } else {
        for (int ti = 0; ti < gr.TPC; ++ti) {
          const int tile = gr.cl + ti * gr.NC;
          if (tile >= pl.n_tiles) break;
          if (ti > 0) make_plan(p, ph, P, rank, tile, pl);
          // ---- one row tile of a GEMM phase: exchange the partial tiles, finish this CTA's 32 columns
          float4* slots = slots_all + (size_t)((slot_sets == 2) ? (g & 1) : 0) * (kSplit * (kOwn / 4) * 64);
          const int n_main = pl.nitems < NACC ? pl.nitems : NACC;
          // bias of the tile (a weight: no dependency on the phase's inputs)
          if (tid < kBN) {
            float bv = 0.f;
            if (pl.kind == PH_CELL) {
              const int hid = tile * (kBN / 4) + (tid % (kBN / 4));
              if (hid < H) bv = __ldg(p.bias[pl.layer] + (size_t)(tid / (kBN / 4)) * H + hid);
            } else if (pl.kind == PH_COMB) {
              const int n = tile * kBN + tid;
              if (n < H) bv = __ldg(p.att_bias + n);
            }
            s_bias[tid] = bv;
          }
          float pre_c[4] = {0.f, 0.f, 0.f, 0.f};
          const float mk = ((pl.kind == PH_CELL || pl.kind == PH_COMB) && r < nb) ? (float)mask[r] : 1.0f;
          if (pl.kind == PH_CELL && r < nb) {  // this thread's old cell state: it wrote it itself one step ago
            const float* cp = p.c_buf[pl.layer][t & 1];
            const int hb = tile * (kBN / 4) + rank * 8 + whalf * 4;
#pragma unroll
            for (int u = 0; u < 4; ++u) pre_c[u] = (hb + u < H) ? cp[(size_t)(b0 + r) * H + hb + u] : 0.f;
          }
          warp_bounded_wait([&] { return mbar_try_wait(&accum_bar, (uint32_t)(g & 1)); }, lane, ab, p.err, 600000 + ph);
          tc_fence_after();
          ZD_STAMP(1);
          if (tid == 0) *reinterpret_cast<volatile int*>(&in_exchange) = 1;
          if (pl.nitems == 0 && tid == 0 && ph > 0) {
            // A CTA without k-blocks (fewer k-blocks than CTAs) has nothing that ties it to the phase's inputs: it must
            // not push its zeros before the owners have finished with the previous phase's slots.
            const unsigned want = (unsigned)ph * G;
            bounded_wait([&] { return ld_acquire_gpu(gr.counter) >= want; }, ab, p.err, 700000 + ph);
          }
          team_sync();  // (and the tile's bias values are in place)
          if (my_rows) {
            const uint32_t my_slot = smem_u32(slots + (size_t)rank * (kOwn / 4) * SR + lrow);
            for (int c0 = chalf * 64; c0 < chalf * 64 + 64; c0 += 32) {
              float v[32];
              if (pl.nitems == 0) {
#pragma unroll
                for (int u = 0; u < 32; ++u) v[u] = 0.f;
              } else {
                tmem_ld32(taddr + c0, v);
                if (mode_split(MODE)) {
                  float tv[32];
                  for (int a = 1; a < n_main; ++a) {
                    tmem_ld32(taddr + a * kBN + c0, tv);
                    tmem_wait_ld();
#pragma unroll
                    for (int u = 0; u < 32; ++u) v[u] += tv[u];
                  }
                  tmem_ld32(taddr + NACC * kBN + c0, tv);
                  tmem_wait_ld();
#pragma unroll
                  for (int u = 0; u < 32; ++u) v[u] = fmaf(tv[u], mode_cross_scale(MODE), v[u]);
                }
                tmem_wait_ld();
              }
#pragma unroll
              for (int u = 0; u < 32; u += 4) {
                const int c = c0 + u;
                int owner, lcol;
                if (pl.kind == PH_CELL) {  // tile column = gate * 32 + hidden unit; a CTA owns 8 hidden units, all gates
                  const int gate = c / 32, j = c % 32;
                  owner = j / 8;
                  lcol = gate * 8 + (j % 8);
                } else {
                  owner = c / kOwn;
                  lcol = c % kOwn;
                }
                if (owner == rank) {
                  slots[((size_t)rank * (kOwn / 4) + lcol / 4) * SR + lrow] = make_float4(v[u], v[u + 1], v[u + 2], v[u + 3]);
                } else {
                  const uint32_t local = my_slot + (uint32_t)((lcol / 4) * SR * 16);
                  st_cluster_v4(cluster_map(local, (uint32_t)owner), v[u], v[u + 1], v[u + 2], v[u + 3]);
                }
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          ZD_STAMP(3);
          if (p.detail && lane == 0) s_push[warp] = gtime();
          if (lane == 0) {
            mbar_arrive_local(&tmem_free);  // this warp's accumulator reads are complete
            for (int c = 0; c < kSplit; ++c) mbar_arrive_remote(&xchg_bar, (uint32_t)c);
          }
          warp_bounded_wait([&] { return mbar_try_wait_cluster(&xchg_bar, (uint32_t)(g & 1)); }, lane, ab, p.err, 800000 + ph);
          ZD_STAMP(4);
          if (tid == 0) *reinterpret_cast<volatile int*>(&in_exchange) = 0;
          if (p.detail && tid == 0) {  // slot 2 of the timeline: the last warp of this CTA to finish pushing
            long long mx = 0;
            for (int i = 0; i < kTeam / 32; ++i) mx = s_push[i] > mx ? s_push[i] : mx;
            if (p.detail_cta < 0) p.detail[((size_t)cta_all * NP + ph) * 8 + 2] = mx;
            else if (cta_all == p.detail_cta) p.detail[(size_t)ph * 8 + 2] = mx;
          }
          ++g;
          if (pl.kind == PH_CELL) {
            const int l = pl.layer;
            if (r < nb) {
              float gsum[4][4];
#pragma unroll
              for (int gq = 0; gq < 4; ++gq) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int rk = 0; rk < kSplit; ++rk) {  // fixed order: deterministic sums
                  const float4 tv = slots[((size_t)rk * (kOwn / 4) + gq * 2 + whalf) * SR + r];
                  acc.x += tv.x; acc.y += tv.y; acc.z += tv.z; acc.w += tv.w;
                }
                gsum[gq][0] = acc.x; gsum[gq][1] = acc.y; gsum[gq][2] = acc.z; gsum[gq][3] = acc.w;
              }
              const int jb = rank * 8 + whalf * 4;  // first hidden unit inside the tile
              const int hb = tile * 32 + jb;
              const int nvalid = H - hb >= 4 ? 4 : (H - hb > 0 ? H - hb : 0);
              float hv[4], cv[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float gi = act_sigmoid<MODE>(gsum[0][u] + s_bias[jb + u]);
                const float gf = act_sigmoid<MODE>(gsum[1][u] + s_bias[32 + jb + u]);
                const float gg = act_tanh<MODE>(gsum[2][u] + s_bias[64 + jb + u]);
                const float go = act_sigmoid<MODE>(gsum[3][u] + s_bias[96 + jb + u]);
                const float c = gf * pre_c[u] + gi * gg;
                hv[u] = go * act_tanh<MODE>(c) * mk;
                cv[u] = c * mk;
              }
              if (nvalid > 0) {
                const size_t row = (size_t)t * Bs + b0 + r;
                store4_f32(p.c_buf[l][(t + 1) & 1], (size_t)(b0 + r) * H + hb, cv, nvalid);
                store4_f32(p.h_f32[l], row * H + hb, hv, nvalid);
                store4_operand(make_opout<MODE>(p.h_op_hi[l], p.h_op_lo[l]), row * p.Kpad + hb, hv, nvalid);
              }
            }
          } else if (r < nb) {
            // store epilogue: this CTA's 32 tile columns, thread = (row r, columns 16 * whalf .. + 16)
            const int N = pl.kind == PH_PGEMM ? 2 * H : H;
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              const int lc = whalf * 16 + c4 * 4;  // column inside this CTA's 32
              float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
              for (int rk = 0; rk < kSplit; ++rk) {
                const float4 tv = slots[((size_t)rk * (kOwn / 4) + lc / 4) * SR + r];
                acc.x += tv.x; acc.y += tv.y; acc.z += tv.z; acc.w += tv.w;
              }
              const int n0 = tile * kBN + rank * kOwn + lc;
              const int nvalid = N - n0 >= 4 ? 4 : (N - n0 > 0 ? N - n0 : 0);
              float x[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                float v = x[u] + s_bias[rank * kOwn + lc + u];
                if (pl.kind == PH_COMB || n0 + u < H) v = act_tanh<MODE>(v);
                x[u] = v * mk;
              }
              if (nvalid > 0) {
                if (pl.kind == PH_PGEMM) {
                  store4_f32(p.tq, (size_t)(b0 + r) * (2 * H) + n0, x, nvalid);
                } else {
                  const size_t row = (size_t)t * Bs + b0 + r;
                  store4_f32(p.ht_f32, row * H + n0, x, nvalid);
                  store4_operand(make_opout<MODE>(p.ht_op_hi, p.ht_op_lo), row * p.Kpad + n0, x, nvalid);
                }
              }
            }
          }
          if (ti + 1 < gr.TPC) team_sync();  // the bias values and (single slot set) the slots are free for the next tile
        }
      }
      // ---- hand the phase over: results visible to ordinary loads and to TMA, then count this CTA
      ZD_STAMP(5);
      fence_proxy_async();
      team_sync();
      if (*ab) break;
      if (tid == 0) {
        // a CTA only adds its count for phase ph once phases < ph are complete, so the counter has one meaning.  An
        // active CTA knows that already (its producer needed them for this phase's inputs); an idle one has to look.
        if (done_phases < (unsigned)ph) {
          if (ld_acquire_cta_shared(&prod_done) < ph) {
            // (with a pause between looks: dozens of idle CTAs reading one word back to back get in the way of the
            // working CTAs' additions to it)
            const unsigned want = (unsigned)ph * G;
            bounded_wait([&] {
              if (ld_acquire_gpu(gr.counter) >= want) return true;
              __nanosleep(300);
              return false;
            }, ab, p.err, 900000 + ph);
          }
          done_phases = (unsigned)ph;
        }
        ZD_STAMP(6);
        if (!*ab)  // release: cumulative over the team's stores, which the barrier above ordered before this thread
          asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(gr.counter) : "memory");
        ZD_STAMP(7);
        if (p.stamps && cta_all == 0) p.stamps[1 + ph] = gtime();
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody retires while a peer may still write into its shared memory
  if (warp == 9) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

constexpr int kMaxDev = 64;
int cur_dev() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDev) d = 0;
  return d;
}

template <int MODE>
cudaError_t configure(int* max_clusters) {
  static bool done[kMaxDev] = {false};
  static int clusters[kMaxDev] = {0};
  const int dev = cur_dev();
  if (!done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tc_decoder_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, dec_smem(MODE));
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(kSplit, 64, 1);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = dec_smem(MODE);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kSplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, tc_decoder_kernel<MODE>, &cfg);
    if (e != cudaSuccess) return e;
    clusters[dev] = n;
    done[dev] = true;
  }
  *max_clusters = clusters[dev];
  return cudaSuccess;
}

template <int MODE>
cudaError_t launch_mode(const DecParams& p, cudaStream_t st) {
  int max_clusters = 0;
  cudaError_t e = configure<MODE>(&max_clusters);
  if (e != cudaSuccess) return e;
  const int NT = (4 * p.H + kBN - 1) / kBN;
  const int groups = p.groups < 1 ? 1 : p.groups;
  int NC = max_clusters / groups;  // clusters per column group
  if (NC > NT) NC = NT;
  if (NC < 1 || p.a_rows < 8 || p.a_rows > 128 || (p.a_rows & 7) != 0) return cudaErrorInvalidConfiguration;
  // one set of exchange slots (more than 64 columns per group) serves one row tile per phase only
  if (p.a_rows > 64 && NC < NT) return cudaErrorInvalidConfiguration;
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(kSplit, NC, groups);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = dec_smem(MODE);
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kSplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // all CTAs wait on one another: ask the runtime to refuse the launch unless they can be resident together
  attr[1].id = cudaLaunchAttributeCooperative;
  attr[1].val.cooperative = 1;
  cfg.attrs = attr;
  static int coop_ok[kMaxDev] = {0};  // 0 unknown, 1 accepted, -1 refused (the occupancy check above still holds)
  const int dev = cur_dev();
  cfg.numAttrs = coop_ok[dev] >= 0 ? 2 : 1;
  e = cudaLaunchKernelEx(&cfg, tc_decoder_kernel<MODE>, p);
  if (e != cudaSuccess && cfg.numAttrs == 2 && coop_ok[dev] == 0) {
    (void)cudaGetLastError();
    coop_ok[dev] = -1;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, tc_decoder_kernel<MODE>, p);
  } else if (e == cudaSuccess && cfg.numAttrs == 2) {
    coop_ok[dev] = 1;
  }
  count_launch();
  return e;
}

}  // namespace

bool tc_decoder_supported(int mode, int H, int B, int L, int att_type) {
  if (B < 1 || B > 128 || L < 1 || L > DecParams::MAXL || (att_type != 1 && att_type != 2)) return false;
  if ((H & 3) != 0 || H > 1024 || H < 8) return false;  // the attention step's 16-byte loads and register budget
  int max_clusters = 0;
  cudaError_t e = cudaErrorInvalidValue;
  switch (mode) {
    case TC_BF16: e = configure<TC_BF16>(&max_clusters); break;
    case TC_TF32: e = configure<TC_TF32>(&max_clusters); break;
    case TC_TF32X3: e = configure<TC_TF32X3>(&max_clusters); break;
    case TC_F16X2: e = configure<TC_F16X2>(&max_clusters); break;
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return (4 * H + kBN - 1) / kBN <= max_clusters;
}

int tc_decoder_default_groups(int B) {
  static const int forced = [] {
    const char* e = std::getenv("ZRNN_DEC_GROUPS");
    return e ? std::atoi(e) : 0;
  }();
  int g = forced > 0 ? forced : (B >= 32 ? 2 : 1);
  if (g > 4) g = 4;
  while (g > 1 && (B + g - 1) / g > 64) g *= 2;  // not reachable for B <= 128; keeps the 64-column rule explicit
  while (g > 1 && B < 8 * g) g /= 2;
  return g;
}

cudaError_t launch_tc_decoder(const DecParams& p, int mode, cudaStream_t st) {
  switch (mode) {
    case TC_BF16: return launch_mode<TC_BF16>(p, st);
    case TC_TF32: return launch_mode<TC_TF32>(p, st);
    case TC_TF32X3: return launch_mode<TC_TF32X3>(p, st);
    case TC_F16X2: return launch_mode<TC_F16X2>(p, st);
  }
  return cudaErrorInvalidValue;
}

}  // namespace zrnn
