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
#include "tc_device.cuh"

namespace zrnn {
namespace {

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

// ------------------------------------------------------------------------------------------
// Exercise of the bounded wait: one warp waits on a barrier that nothing ever completes, with a short limit, and
// must come back with the error word set and the context intact.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32) wait_probe_kernel(int* err, long long limit_cycles, int code) {
  __shared__ uint64_t bar;
  __shared__ int abort_s;
  if (threadIdx.x == 0) {
    abort_s = 0;
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, &abort_s, err, code, limit_cycles);
}
cudaError_t launch_wait_probe(int* err, long long limit_cycles, int code, cudaStream_t st) {
  wait_probe_kernel<<<1, 32, 0, st>>>(err, limit_cycles, code);
  count_launch();
  return cudaGetLastError();
}

}  // namespace zrnn
