// The per-column attention step (scores, masked softmax, context) as device functions for a team of 256 threads, so
// that the same code runs as a kernel of its own (kernels.cu: one CTA per target column) and inside the persistent
// decoder kernel (tc_decoder.cu: the epilogue warps of every CTA take columns in turn).  `sync` is the team's
// barrier (__syncthreads in a kernel, a named barrier inside the persistent kernel); `scratch` is team-private
// shared memory of kAtt*ScratchBytes bytes, 16-byte aligned.  Both need H % 4 == 0 and H <= 1024.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels.cuh"

namespace zrnn {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float sigmoidf_acc(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ void att_store_op(const AttArgs& a, int b, int i, float v) {
  const size_t idx = (size_t)b * a.ld_op + i;
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

#define ZR_ATT_MAXW 64
struct SyncCta {  // the team is a whole CTA
  __device__ __forceinline__ void operator()() const { __syncthreads(); }
};
constexpr int kAttTeam = 256;                                         // threads per column team
constexpr int kAttLocalSmall = (32 + ZR_ATT_MAXW) * 4 + ZR_ATT_MAXW * 4 + 16;      // sums, weights, slots, p_t, window
constexpr int kAttLocalScratchBytes = 8 * 256 * 16 + ((kAttLocalSmall + 15) / 16) * 16;  // + 8 partial contexts
constexpr int kAttGlobalScratchBytes = 8 * 256 * 16 + 4 * 8 * 4;

// sum over the team; result valid in every thread.  `red` holds 32 floats.
template <class Sync>
__device__ __forceinline__ float team_sum(float v, float* red, int tid, Sync sync) {
  const int lane = tid & 31, w = tid >> 5;
  v = warp_sum(v);
  sync();
  if (lane == 0) red[w] = v;
  sync();
  float t = (tid < kAttTeam / 32) ? red[tid] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  sync();
  return red[0];
}

// Local-p attention of target column b (attention_node::forward_prop, src/attention_node.hpp:141-281, with the
// kernels of src/custom_kernels.h:1581-1813): p_t from tanh(W_p h) and v_p, the window [p_t - D, p_t + D] cut at the
// sentence, scores h_s . (W_a^T h), softmax over the valid window positions with the maximum started at 0, the
// un-renormalised Gaussian, the context.  16-byte loads, and no data-dependent branch inside the loops over the
// window.  An empty slot gets weight 0 and reads row 0 of the source memory.
// Windows of up to 24 slots (D <= 11; the reference's default D is 10) take the register path: warp w owns slots w,
// w + 8, w + 16, requests their rows in one go, keeps them in registers for the score AND the context (the source
// memory is read once), and the eight partial contexts meet in shared memory.  Wider windows walk the slots twice.
template <class Sync>
__device__ __forceinline__ void att_local_fast_body(const AttArgs& a, const int b, const int tid, unsigned char* scratch,
                                                    Sync sync) {
  float4(*s_ctx)[256] = reinterpret_cast<float4(*)[256]>(scratch);
  float* red = reinterpret_cast<float*>(scratch + 8 * 256 * 16);
  float* s_al = red + 32;
  int* s_slot = reinterpret_cast<int*>(s_al + ZR_ATT_MAXW);
  const int lane = tid & 31, w = tid >> 5;
  const int H = a.H, H4 = H >> 2, Wn = 2 * a.D + 1, sb = b / a.cols_per_sent;
  float* c = a.c_t + (size_t)b * H;
  if (a.mask && a.mask[b] != 1) {
    for (int i = tid; i < H; i += kAttTeam) { c[i] = 0.f; att_store_op(a, b, i, 0.f); }
    if (a.align_out) {
      const int n_out = a.align_by_pos ? a.S_max : Wn;
      for (int j = tid; j < n_out; j += kAttTeam) a.align_out[(size_t)j * a.B + b] = 0.f;
    }
    if (a.viterbi_out && tid == 0) a.viterbi_out[b] = -1;
    return;
  }
  float part = 0.f;
  if (tid < H4) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(a.v_p) + tid);
    const float4 t = reinterpret_cast<const float4*>(a.tanh1 + (size_t)b * a.ld_tq)[tid];
    part = v.x * t.x + v.y * t.y + v.z * t.z + v.w * t.w;
  }
  // q = W_a^T h does not depend on the window: request it before the reduction
  const float4* q4 = reinterpret_cast<const float4*>(a.q + (size_t)b * a.ld_tq);
  float4 qv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int j4 = lane + 32 * i;
    qv[i] = j4 < H4 ? q4[j4] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float tot = team_sum(part, red, tid, sync);
  const int len = a.len[sb], off = a.offset[sb];
  // every thread derives the window itself (the same arithmetic on the same value: no barrier needed for it)
  const float sg = (float)(1.0 / (1.0 + exp(-1.0 * (double)tot)));
  const float pt = len * sg;
  const int ip = (int)pt;
  const int lo = (0 > ip - a.D) ? 0 : (ip - a.D);
  const int hi = ((len - 1) < ip + a.D) ? (len - 1) : (ip + a.D);
  const bool reg_path = Wn <= 24;
  float4 rows[3][8];
  if (reg_path) {
#pragma unroll
    for (int u = 0; u < 3; ++u) {
      const int j = w + 8 * u, pos = lo + j;
      const bool valid = j < Wn && pos <= hi;
      const int slot = valid ? len - 1 - pos + off : 0;
      const float4* r4 = reinterpret_cast<const float4*>(a.hs + ((size_t)slot * a.B_src + sb) * H);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int j4 = lane + 32 * i;
        rows[u][i] = j4 < H4 ? __ldg(r4 + j4) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int u = 0; u < 3; ++u) {
      const int j = w + 8 * u, pos = lo + j;
      const bool valid = j < Wn && pos <= hi;
      float sc = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        sc += rows[u][i].x * qv[i].x + rows[u][i].y * qv[i].y + rows[u][i].z * qv[i].z + rows[u][i].w * qv[i].w;
      sc = warp_sum(sc);
      if (lane == 0 && j < Wn) { s_al[j] = valid ? sc : 0.f; s_slot[j] = valid ? len - 1 - pos + off : -1; }
    }
  } else {
    for (int j = w; j < Wn; j += 8) {
      const int pos = lo + j;
      const bool valid = pos <= hi;
      const int slot = valid ? len - 1 - pos + off : 0;  // an empty slot reads row 0 and is discarded
      const float4* r4 = reinterpret_cast<const float4*>(a.hs + ((size_t)slot * a.B_src + sb) * H);
      float sc = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int j4 = lane + 32 * i;
        if (j4 < H4) {
          const float4 r = __ldg(r4 + j4);
          sc += r.x * qv[i].x + r.y * qv[i].y + r.z * qv[i].z + r.w * qv[i].w;
        }
      }
      sc = warp_sum(sc);
      if (lane == 0) { s_al[j] = valid ? sc : 0.f; s_slot[j] = valid ? slot : -1; }
    }
  }
  sync();
  // softmax over the window by the first warps, one slot per lane (the sums are warp reductions)
  {
    if (w == 0) {
      float mx = 0.f;  // the reference starts the max at 0
      for (int j = lane; j < Wn; j += 32)
        if (s_slot[j] != -1) mx = fmaxf(mx, s_al[j]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float e[2] = {0.f, 0.f};
      float sum = 0.f;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int j = lane + 32 * u;
        if (j < Wn && s_slot[j] != -1) e[u] = expf(s_al[j] - mx);
        sum += e[u];
      }
      sum = warp_sum(sum);
      const float sigma_sq = (float)((a.D * a.D) / 4.0);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int j = lane + 32 * u;
        if (j < Wn) {
          float v = e[u];
          if (s_slot[j] != -1) {
            const float d = pt - (float)(lo + j);
            const float gs = expf((-1.f * d * d) / (2.f * sigma_sq));
            if (sum != 0.f) v = (v / sum) * gs;
          }
          s_al[j] = v;
        }
      }
      __syncwarp();
      if (a.viterbi_out && lane == 0) {
        float best = a.viterbi_init;
        int best_pos = -1;
        for (int j = 0; j < Wn; ++j)
          if (best < s_al[j]) { best = s_al[j]; best_pos = (s_slot[j] != -1) ? lo + j : -1; }
        a.viterbi_out[b] = best_pos;
      }
    }
  }
  sync();
  if (a.align_out) {
    if (a.align_by_pos) {
      for (int s = tid; s < a.S_max; s += kAttTeam) {
        const int j = s - lo;
        a.align_out[(size_t)s * a.B + b] = (j >= 0 && j < Wn && s <= hi) ? s_al[j] : 0.f;
      }
    } else {
      for (int j = tid; j < Wn; j += kAttTeam) a.align_out[(size_t)j * a.B + b] = s_al[j];
    }
  }
  if (reg_path) {
    // each warp's share of the context from the rows it still holds, then the eight shares in a fixed order
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 3; ++u) {
        const int j = w + 8 * u;
        const float wj = (j < Wn) ? s_al[j] : 0.f;
        acc.x += wj * rows[u][i].x; acc.y += wj * rows[u][i].y; acc.z += wj * rows[u][i].z; acc.w += wj * rows[u][i].w;
      }
      s_ctx[w][lane + 32 * i] = acc;
    }
    sync();
    if (tid < H4) {
      float4 acc = s_ctx[0][tid];
#pragma unroll
      for (int q = 1; q < 8; ++q) {
        const float4 r = s_ctx[q][tid];
        acc.x += r.x; acc.y += r.y; acc.z += r.z; acc.w += r.w;
      }
      reinterpret_cast<float4*>(c)[tid] = acc;
      att_store_op(a, b, 4 * tid + 0, acc.x);
      att_store_op(a, b, 4 * tid + 1, acc.y);
      att_store_op(a, b, 4 * tid + 2, acc.z);
      att_store_op(a, b, 4 * tid + 3, acc.w);
    }
  } else if (tid < H4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const size_t colb = (size_t)sb * H;
#pragma unroll 7
    for (int j = 0; j < Wn; ++j) {
      const float wj = s_al[j];
      const int slot = s_slot[j] == -1 ? 0 : s_slot[j];  // weight 0, any readable row
      const float4 r = __ldg(reinterpret_cast<const float4*>(a.hs + (size_t)slot * a.B_src * H + colb) + tid);
      acc.x += wj * r.x; acc.y += wj * r.y; acc.z += wj * r.z; acc.w += wj * r.w;
    }
    reinterpret_cast<float4*>(c)[tid] = acc;
    att_store_op(a, b, 4 * tid + 0, acc.x);
    att_store_op(a, b, 4 * tid + 1, acc.y);
    att_store_op(a, b, 4 * tid + 2, acc.z);
    att_store_op(a, b, 4 * tid + 3, acc.w);
  }
}

// Global dot-product attention of target column b in a single pass: each of the team's 8 warps walks over every 8th
// source position, keeps the position's vector in registers for both the score and the context (so the source memory
// is read once, with 16-byte loads), and carries a running (max, sum, context); the 8 partial results are merged through
// shared memory at the end.
template <class Sync>
__device__ __forceinline__ void att_global_fast_body(const AttArgs& a, const int b, const int tid, unsigned char* scratch,
                                                     Sync sync) {
  float4(*s_ctx)[256] = reinterpret_cast<float4(*)[256]>(scratch);
  float* s_m = reinterpret_cast<float*>(scratch + 8 * 256 * 16);
  float* s_l = s_m + 8;
  float* s_bsc = s_l + 8;
  int* s_bpos = reinterpret_cast<int*>(s_bsc + 8);
  const int lane = tid & 31, w = tid >> 5;
  const int H = a.H, H4 = H >> 2, sb = b / a.cols_per_sent;
  float* c = a.c_t + (size_t)b * H;
  if (a.mask && a.mask[b] != 1) {
    for (int i = tid; i < H; i += kAttTeam) { c[i] = 0.f; att_store_op(a, b, i, 0.f); }
    if (a.align_out)
      for (int s = tid; s < a.S_max; s += kAttTeam) a.align_out[(size_t)s * a.B + b] = 0.f;
    if (a.viterbi_out && tid == 0) a.viterbi_out[b] = -1;
    return;
  }
  const int len = a.len[sb], off = a.offset[sb];
  const float4* h4 = reinterpret_cast<const float4*>(a.h_t + (size_t)b * H);
  float4 hv[8], ctx[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int j = lane + 32 * i;
    hv[i] = j < H4 ? h4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    ctx[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float m = -INFINITY, l = 0.f, bsc = -INFINITY;
  int bpos = -1;
  // two source positions per round: the 16 loads of a lane are in flight together, which halves the number of L2
  // round trips a warp waits for
  for (int pos = w; pos < len; pos += 16) {
    const int pos2 = pos + 8;
    const bool two = pos2 < len;
    const float4* r4 = reinterpret_cast<const float4*>(a.hs + ((size_t)(len - 1 - pos + off) * a.B_src + sb) * H);
    const float4* s4 = reinterpret_cast<const float4*>(a.hs + ((size_t)(len - 1 - (two ? pos2 : pos) + off) * a.B_src + sb) * H);
    float4 rv[8], sv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int j = lane + 32 * i;
      rv[i] = j < H4 ? __ldg(r4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
      sv[i] = j < H4 ? __ldg(s4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float sc = 0.f, sc2 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sc += rv[i].x * hv[i].x + rv[i].y * hv[i].y + rv[i].z * hv[i].z + rv[i].w * hv[i].w;
      sc2 += sv[i].x * hv[i].x + sv[i].y * hv[i].y + sv[i].z * hv[i].z + sv[i].w * hv[i].w;
    }
    sc = warp_sum(sc);
    sc2 = warp_sum(sc2);
    {
      if (a.align_out && lane == 0) a.align_out[(size_t)pos * a.B + b] = sc;  // raw score, normalised below
      if (sc > bsc) { bsc = sc; bpos = pos; }
      const float mn = fmaxf(m, sc);
      const float scale = expf(m - mn), e = expf(sc - mn);
      l = l * scale + e;
      m = mn;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        ctx[i].x = ctx[i].x * scale + e * rv[i].x;
        ctx[i].y = ctx[i].y * scale + e * rv[i].y;
        ctx[i].z = ctx[i].z * scale + e * rv[i].z;
        ctx[i].w = ctx[i].w * scale + e * rv[i].w;
      }
    }
    if (two) {
      if (a.align_out && lane == 0) a.align_out[(size_t)pos2 * a.B + b] = sc2;
      if (sc2 > bsc) { bsc = sc2; bpos = pos2; }
      const float mn = fmaxf(m, sc2);
      const float scale = expf(m - mn), e = expf(sc2 - mn);
      l = l * scale + e;
      m = mn;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        ctx[i].x = ctx[i].x * scale + e * sv[i].x;
        ctx[i].y = ctx[i].y * scale + e * sv[i].y;
        ctx[i].z = ctx[i].z * scale + e * sv[i].z;
        ctx[i].w = ctx[i].w * scale + e * sv[i].w;
      }
    }
  }
  if (lane == 0) { s_m[w] = m; s_l[w] = l; s_bsc[w] = bsc; s_bpos[w] = bpos; }
#pragma unroll
  for (int i = 0; i < 8; ++i) s_ctx[w][lane + 32 * i] = ctx[i];
  sync();
  if (a.viterbi_out && tid == 0) {  // largest score = largest weight; the lowest position wins a tie
    float best = -INFINITY;
    int best_pos = -1;
    for (int q = 0; q < 8; ++q)
      if (s_bpos[q] >= 0 && (s_bsc[q] > best || (s_bsc[q] == best && s_bpos[q] < best_pos))) { best = s_bsc[q]; best_pos = s_bpos[q]; }
    a.viterbi_out[b] = best_pos;
  }
  float M = -INFINITY;
#pragma unroll
  for (int q = 0; q < 8; ++q) M = fmaxf(M, s_m[q]);
  float Lsum = 0.f, wq[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    wq[q] = (s_m[q] == -INFINITY) ? 0.f : expf(s_m[q] - M);
    Lsum += s_l[q] * wq[q];
  }
  const float inv = 1.0f / Lsum;
  if (tid < H4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 v = s_ctx[q][tid];
      acc.x += wq[q] * v.x; acc.y += wq[q] * v.y; acc.z += wq[q] * v.z; acc.w += wq[q] * v.w;
    }
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    reinterpret_cast<float4*>(c)[tid] = acc;
    att_store_op(a, b, 4 * tid + 0, acc.x);
    att_store_op(a, b, 4 * tid + 1, acc.y);
    att_store_op(a, b, 4 * tid + 2, acc.z);
    att_store_op(a, b, 4 * tid + 3, acc.w);
  }
  if (a.align_out) {
    sync();
    for (int pos = tid; pos < a.S_max; pos += kAttTeam) {
      const size_t idx = (size_t)pos * a.B + b;
      a.align_out[idx] = pos < len ? expf(a.align_out[idx] - M) * inv : 0.f;
    }
  }
}

}  // namespace zrnn
