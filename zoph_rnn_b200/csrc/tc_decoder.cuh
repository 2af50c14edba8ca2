// Persistent decoder kernel: the whole target side of a feed-input model (every time step's LSTM cells, attention and
// tanh combiner) in ONE launch.  With feed-input the steps form a strict chain (layer 0 of step t reads the attention
// output of step t - 1), so a launch per cell leaves the machine idle across every launch boundary and requests no
// weight byte of the next cell before the current one has retired.  Here clusters of four CTAs stay resident, keep
// their barriers, tensor memory and exchange slots alive, stream the next phase's weight tiles while the current
// phase's exchange and gate math run, and hand activations from phase to phase through a grid-wide counter.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace zrnn {

struct DecParams {
  enum { MAXL = 4 };
  int H, Kpad, B, T, L;      // B <= 128 columns, L <= MAXL layers
  int groups;                // column groups that run the chain of phases independently (1, 2 or 4)
  int a_rows;                // rows per activation box = columns of a group rounded up to 8 (the tensor maps' box height)
  int att_type;              // 1 = local-p, 2 = global dot
  int D;                     // local-p half window
  int kb;                    // 128-byte k-blocks that cover H elements
  int kpb;                   // k-blocks per Kpad (stride of a source inside a weight matrix's K axis)
  int w_tiled[MAXL];         // > 0: layer's weights are stored tile-contiguously with this many k-blocks per row tile
  // activations in operand form (K-major rows of Kpad elements), one tensor map per buffer (hi, lo parts)
  CUtensorMap x_hi, x_lo;                  // gathered layer-0 inputs, T*B rows
  CUtensorMap h_hi[MAXL], h_lo[MAXL];      // h sequence of every layer, T*B rows (row t*B + b)
  CUtensorMap h0_hi[MAXL], h0_lo[MAXL];    // the buffer holding every layer's state before step 0
  int h0_row[MAXL];                        // ... and its first row there
  CUtensorMap ht_hi, ht_lo;                // attention output sequence, T*B rows
  CUtensorMap ctx_hi, ctx_lo;              // context vectors of the current step, B rows
  // weights
  CUtensorMap w_hi[MAXL], w_lo[MAXL];      // packed LSTM weights, K axis = x | h | htild
  CUtensorMap wc_hi, wc_lo;                // [W_c1 | W_c2], H rows x 2 Kpad
  CUtensorMap wp_hi, wp_lo;                // [W_p ; W_a^T], 2H rows x Kpad (local-p)
  // epilogue operands and outputs
  const float* bias[MAXL];   // [4][H] gate-major
  float* c_buf[MAXL][2];     // cell state ping-pong: step t reads [t & 1], writes [(t + 1) & 1]
  float* h_f32[MAXL];        // fp32 h sequence, H x (T*B)
  void* h_op_hi[MAXL];       // operand-form h sequence
  void* h_op_lo[MAXL];
  float* ht_f32;             // attention output sequence (what the softmax reads)
  void* ht_op_hi;
  void* ht_op_lo;
  float* ctx_f32;            // H x B
  void* ctx_op_hi;
  void* ctx_op_lo;
  float* tq;                 // local-p: 2H x B, rows [0,H) tanh(W_p h), rows [H,2H) W_a^T h
  const float* att_bias;     // H
  const float* v_p;          // H (local-p)
  const int* mask;           // T*B, 0/1
  const float* hs;           // source memory: S_max slots of H x B
  int S_max;
  const int* len;
  const int* off;
  unsigned int* counter;     // grid-wide phase counter, zero at launch
  int* err;                  // device error word
  long long* stamps;         // optional: [1 + phases] globaltimer values (kernel start, end of every phase)
  long long* detail;         // optional developer timeline: 8 stamps per phase written by CTA detail_cta
  int detail_cta;
  int w_evict_first;         // stream the weight tiles with the L2 evict-first policy
  int hold_loads;            // experiment: no TMA loads are issued while the CTA exchanges partial tiles
};

// number of phases of one time step: L cells, [the stacked local-p GEMM], the attention proper, the combiner
inline int dec_phases_per_step(const DecParams& p) { return p.L + (p.att_type == 1 ? 3 : 2); }

// Can the kernel run this shape on the current device?  (tile count against the clusters that fit at once)
bool tc_decoder_supported(int mode, int H, int B, int L, int att_type);
// Column groups to cut a batch of B columns into (every group needs 64 columns or fewer to take more than one row
// tile per phase, which it must when the clusters are shared among groups).
int tc_decoder_default_groups(int B);
// mode: TC_BF16 / TC_TF32 / TC_TF32X3 / TC_F16X2.  The counter must be zero when the kernel starts.
cudaError_t launch_tc_decoder(const DecParams& p, int mode, cudaStream_t st);

}  // namespace zrnn
