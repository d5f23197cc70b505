// Host-visible launchers of the memory-bound kernels (elementwise.cu, loss_optim.cu, comm.cu).
// Every launcher returns nullptr on success or a static message naming what was wrong; none
// of them allocates memory or synchronises.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "quant_out.h"

namespace gd {

struct Status;

// ---- causal depthwise conv ------------------------------------------------------------------
// Sequence-parallel neighbour exchange done by the conv kernels themselves (slots == nullptr: off). Forward:
// the warps that own the last k-1 rows of a sequence store them into the next rank's slot and the last of
// them raises that rank's flag; the warps that own the first rows wait (bounded) for this rank's own flag and
// read the previous rank's rows from this rank's slot. Backward runs the other way: the halo gradient goes to
// the previous rank, and the next rank's halo gradient is added to the last k-1 rows of dx before they are
// stored. Blocks are ordered so that the stores come first and the waits last.
struct ConvSp {
  uint8_t* const* slots;    // [world] base of every rank's slot area (peer-mapped)
  uint32_t* const* flags;   // [world] base of every rank's flag area
  int64_t slot_offset;      // byte offset of this exchange's slot
  int flag_index;
  int rank, world;
  uint32_t seq;             // sequence number of this exchange (grows with every use of the slot)
  uint32_t* counter;        // local word, zero between launches: warps that have stored their rows
  uint64_t budget_ns;       // time limit of the wait; 0 = the library default
  __nv_bfloat16* halo_out;  // forward: the rows received (zeros on the first rank), (B, k-1, d), kept for backward
  Status* status;
};

struct ConvArgs {
  const __nv_bfloat16* x;     // (B, T, d), row pitch x_ld
  const __nv_bfloat16* halo;  // (B, k-1, d) or null (zeros)
  const float* w;             // taps transposed: (k, d)
  __nv_bfloat16* out;         // (B, T, d), row pitch out_ld
  int B, T, d, k;
  int64_t x_ld, out_ld;
  RowQuantOut quant;          // optional 1x128-quantised copy of out (d % 128 == 0)
  ConvSp sp;                  // in-kernel halo exchange (k == 4 and T % 8 == 0 only)
};

struct ConvBwdArgs {
  const __nv_bfloat16* dc;    // (B, T, d), row pitch dc_ld
  const __nv_bfloat16* x;     // (B, T, d), row pitch x_ld
  const __nv_bfloat16* halo;  // (B, k-1, d) or null
  const float* w;             // taps transposed: (k, d)
  const __nv_bfloat16* dx_tail_add;  // (B, k-1, d) or null: halo gradient from the next shard
  __nv_bfloat16* dx;          // (B, T, d) contiguous
  __nv_bfloat16* dhalo;       // (B, k-1, d) or null
  float* dw;                  // (d, k), accumulated with atomics
  int B, T, d, k;
  int64_t dc_ld, x_ld;
  ConvSp sp;                  // in-kernel halo-gradient exchange (k == 4 and T % 8 == 0 only)
};

const char* launch_dwconv_fwd(const ConvArgs& a, cudaStream_t st);
const char* launch_dwconv_bwd(const ConvBwdArgs& a, cudaStream_t st);

// ---- gate / stream update ---------------------------------------------------------------------
struct GateFwdArgs {
  const __nv_bfloat16* g_pre;  // (rows, d)
  const __nv_bfloat16* z;      // (rows, d) recovery pre-norm
  const __nv_bfloat16* c;      // (rows, d) pitch c_ld
  const __nv_bfloat16* s;      // (rows, d) pitch s_ld
  const float* w_r;            // (d) recovery RMSNorm weight
  __nv_bfloat16* fwd_out;      // (rows, d)
  __nv_bfloat16* side_out;     // (rows, d)
  __nv_bfloat16* gate_out;     // (rows, d) or null
  float* rstd_out;             // (rows) or null
  float* gate_sum;             // scalar accumulator or null
  int64_t rows;
  int d;
  int64_t c_ld, s_ld;
  float eps_r;
  RowQuantOut quant;           // optional 1x128-quantised copy of side_out (d % 128 == 0)
};

struct GateBwdArgs {
  const __nv_bfloat16* dF;   // (rows, d) pitch dF_ld
  const __nv_bfloat16* dS;   // (rows, d) pitch dS_ld
  const __nv_bfloat16* g_pre;
  const __nv_bfloat16* z;
  const __nv_bfloat16* c;    // pitch c_ld
  const __nv_bfloat16* s;    // pitch s_ld
  const float* w_r;
  const float* b2g;          // (d) gate W2 bias, fp32
  int b2g_f32;
  const float* rstd_z;       // (rows)
  const float* ssq_g;        // (rows, ssq_parts) partial sums of squares of silu(W1 c + b1)
  int ssq_parts;
  float eps_g;
  const float* dgate_mean;   // scalar d(loss)/d(mean gate) or null
  __nv_bfloat16* dq;         // (rows, d)
  __nv_bfloat16* dz;         // (rows, d)
  __nv_bfloat16* dsc;        // (rows, 2d): [ds_dir | dc_dir]
  float* rowcoef;            // (rows)
  float* row_dotz;           // unused (the row statistics stay in registers between the two passes of the kernel)
  float* row_rstdg;          // unused
  float* db2g;               // (d) accumulated
  float* dw_r;               // (d) accumulated
  float* db2r;               // (d) accumulated
  int64_t rows;
  int d;
  int64_t dF_ld, dS_ld, c_ld, s_ld;
  RowQuantOut quant_dz;      // optional 1x128-quantised copy of dz (d % 128 == 0): A operand of the next data-gradient GEMM
};

const char* launch_gate_update_fwd(const GateFwdArgs& a, cudaStream_t st);

// The stream update of a step whose side stream is identically zero (the first forward step of every layer):
// fwd' = c g, side' = c (1 - g); the recovery gate multiplies zero and is not evaluated. d = 256 n, n <= 8.
struct GateOnlyFwdArgs {
  const __nv_bfloat16* g_pre;  // (rows, d)
  const __nv_bfloat16* c;      // (rows, d) pitch c_ld
  __nv_bfloat16* fwd_out;      // (rows, d)
  __nv_bfloat16* side_out;     // (rows, d)
  float* gate_sum;             // scalar accumulator or null
  int64_t rows;
  int d;
  int64_t c_ld;
  RowQuantOut quant;           // optional 1x128-quantised copy of side_out
};
const char* launch_gate_only_fwd(const GateOnlyFwdArgs& a, cudaStream_t st);

// Its backward: dg_pre = ((dF - dS) c + dgm) g (1 - g), dq = dg_pre rstd_g, dc = dS + (dF - dS) g,
// rowcoef = rstd_g^2 / d * sum_n dg_pre (g_pre - b2g), db2g += column sums of dg_pre.
struct GateOnlyBwdArgs {
  const __nv_bfloat16* dF;     // (rows, d) pitch dF_ld
  const __nv_bfloat16* dS;     // (rows, d) pitch dS_ld
  const __nv_bfloat16* g_pre;  // (rows, d)
  const __nv_bfloat16* c;      // (rows, d) pitch c_ld
  const float* b2g;            // (d)
  const float* ssq_g;          // (rows, ssq_parts)
  int ssq_parts;
  float eps_g;
  const float* dgate_mean;     // scalar or null
  __nv_bfloat16* dq;           // (rows, d)
  __nv_bfloat16* dc;           // (rows, d)
  float* rowcoef;              // (rows)
  float* db2g;                 // (d) accumulated
  int64_t rows;
  int d;
  int64_t dF_ld, dS_ld, c_ld;
};
const char* launch_gate_only_bwd(const GateOnlyBwdArgs& a, cudaStream_t st);
const char* launch_gate_update_bwd(const GateBwdArgs& a, cudaStream_t st);

// Stream update with both gates given (the stand-alone form of the reference's K4 / K5 kernels,
// gdnet/kernel/gated_causal_depthwise_conv/gate_norm.py:34-102): g = sigmoid(g_pre),
//   fwd' = c g + s R,  side' = c (1 - g) + s (1 - R).
// Backward also prepares the gate MLP's backward: dgp = (dF - dS) c g (1 - g); with r = rstd of the row of the
// normalised hidden layer (from the ssq partials, r = rsqrt(sum / d + eps)): dq = r dgp and
// rowcoef = r^2 / d * sum_n dgp (g_pre - b2).
struct GateMixArgs {
  const __nv_bfloat16* g_pre;  // (rows, d) contiguous
  const __nv_bfloat16* c;      // (rows, d), pitch c_ld
  const __nv_bfloat16* s;      // (rows, d), pitch s_ld
  const __nv_bfloat16* R;      // (rows, d), pitch r_ld
  int64_t rows;
  int d;
  int64_t c_ld, s_ld, r_ld;
  // forward
  __nv_bfloat16* fwd_out;      // (rows, d) contiguous
  __nv_bfloat16* side_out;
  // backward
  const __nv_bfloat16* dF;     // (rows, d) contiguous
  const __nv_bfloat16* dS;
  const float* ssq;            // (rows, parts) or null (then dq = dgp and rowcoef is not written)
  int ssq_parts;
  const float* b2;             // (d) or null
  float eps;
  __nv_bfloat16* dgp;          // (rows, d)
  __nv_bfloat16* dq;           // (rows, d) or null
  __nv_bfloat16* dc;           // (rows, d)
  __nv_bfloat16* ds;
  __nv_bfloat16* dR;
  float* rowcoef;              // (rows) or null
};
const char* launch_gate_mix_fwd(const GateMixArgs& a, cudaStream_t st);
const char* launch_gate_mix_bwd(const GateMixArgs& a, cudaStream_t st);

// Read-out blend of the content-addressed memory (reference: gdnet/memory.py:127-139, after the two linears):
//   R = sigmoid(RMSNorm(z; w, eps)),  out[b, t] = fwd[b, t] (1 - R) + retrieved[b] R
// with z, fwd, out (rows = B * T, d) and retrieved (B, d) constant along T. Backward gives dz (through the sigmoid
// and the norm), dfwd, dretrieved (B, d; summed over T) and dw (d), the last two accumulated with atomics.
struct CamBlendArgs {
  const __nv_bfloat16* z;      // (rows, d) contiguous
  const __nv_bfloat16* fwd;    // (rows, d) contiguous
  const __nv_bfloat16* retr;   // (B, d) contiguous
  const float* w;              // (d)
  int64_t rows;
  int T, d;
  float eps;
  __nv_bfloat16* out;          // forward: (rows, d)
  float* rstd;                 // forward: written; backward: read. (rows)
  const __nv_bfloat16* dout;   // backward
  __nv_bfloat16* dz;
  __nv_bfloat16* dfwd;
  float* dretr;                // (B, d) fp32, accumulated
  float* dw;                   // (d) fp32, accumulated
};
const char* launch_cam_blend_fwd(const CamBlendArgs& a, cudaStream_t st);
const char* launch_cam_blend_bwd(const CamBlendArgs& a, cudaStream_t st);

const char* launch_rmsnorm_fwd(const __nv_bfloat16* x, const float* w, __nv_bfloat16* y, float* rstd, int64_t rows,
                               int d, float eps, cudaStream_t st);
const char* launch_rmsnorm_bwd(const __nv_bfloat16* dy, const __nv_bfloat16* x, const float* w, const float* rstd,
                               __nv_bfloat16* dx, float* dw, int64_t rows, int d, cudaStream_t st);

// ---- FP8 quantisation -------------------------------------------------------------------------
enum QuantMode : int { QUANT_ROWS = 0, QUANT_COLS = 1, QUANT_BLOCK = 2 };

struct QuantArgs {
  const __nv_bfloat16* x;  // (rows, cols) pitch x_ld
  int64_t rows;
  int cols;
  int64_t x_ld;
  int pre_silu;            // quantise silu(x) instead of x
  uint8_t* q_row;          // (rows, cols) pitch q_row_ld, or null
  int64_t q_row_ld;
  float* s_row;
  int64_t s_row_ld;
  int row_mode;            // QUANT_ROWS or QUANT_BLOCK
  uint8_t* q_col;          // (cols, rows) pitch q_col_ld, or null
  int64_t q_col_ld;
  float* s_col;
  int64_t s_col_ld;
  int col_mode;            // QUANT_COLS or QUANT_BLOCK
  int pow2;                // scales rounded up to powers of two (needed by the hardware block-scaled GEMM)
  uint8_t* p_row;          // packed UE8M0 chunks for q_row, (rows/128, cols/128, 512) bytes, or null
  int64_t p_row_stride;    // chunks between consecutive row blocks of p_row (cols/128 when dense)
  uint8_t* p_col;          // packed UE8M0 chunks for q_col, (cols/128, rows/128, 512) bytes, or null
  // Every store of an output is repeated at the same offset in n_peer other copies of the output buffers
  // (other ranks' symmetric weight caches): address + peer_delta[r] bytes. Used by the owner of a weight to
  // hand its e4m3 copies to all ranks from inside the quantisation kernel.
  const int64_t* peer_delta;
  int n_peer;
};

const char* launch_quant_tile(const QuantArgs& a, cudaStream_t st);
const char* launch_quant_tensor(const __nv_bfloat16* x, const float* scale, uint8_t* q_row, uint8_t* q_col,
                                float* amax_out, int64_t rows, int cols, cudaStream_t st);

// ---- reductions and small helpers -------------------------------------------------------------
const char* launch_colsum(const __nv_bfloat16* x, float* out, int64_t rows, int cols, int64_t ld, cudaStream_t st);
// dst_s[j] += src[seg_off[s] + j]; dst_addr holds absolute device addresses (fp32), seg_off is ascending from 0
const char* launch_segment_add(const float* src, const int64_t* dst_addr, const int* seg_off, int n_seg, int total,
                               cudaStream_t st);
const char* launch_scale_cols(const __nv_bfloat16* w, const float* colw, __nv_bfloat16* out, int64_t rows, int cols,
                              cudaStream_t st);
const char* launch_unscale_cols_bwd(const float* dW2w, const __nv_bfloat16* W2, const float* colw, float* dW2,
                                    float* dcolw, int rows, int cols, cudaStream_t st);

// ---- loss, memory read, optimiser (loss_optim.cu) ------------------------------------------------
// Cross-entropy over logits (rows, vocab_padded) bf16; only the first `vocab` columns take part.
// Writes per-row loss (0 for ignored rows) and overwrites logits with d(mean loss)/d(logits) * grad_scale.
// A target outside [0, vocab) other than ignore_index is treated as ignored and reported through `status`
// (STATUS_BAD_ARGUMENT, site 60, detail = row); it is never used as an index.
const char* launch_cross_entropy(__nv_bfloat16* logits, const int64_t* targets, float* row_loss,
                                 const float* inv_count, int64_t rows, int vocab, int64_t ld, int ignore_index,
                                 float grad_scale, int write_grad, Status* status, cudaStream_t st);

const char* launch_mem_read_fwd(const float* q, const float* gamma, const float* e, const float* tags,
                                const float* vals, const float* alpha, float* w, float* out, int B, int S, int dsig,
                                int dc, cudaStream_t st);
const char* launch_mem_read_bwd(const float* d_out, const float* q, const float* gamma, const float* e,
                                const float* tags, const float* vals, const float* w, const float* alpha, float* d_q,
                                float* d_gamma, float* d_e, float* d_tags, float* d_vals, float* d_alpha, int B, int S,
                                int dsig, int dc, cudaStream_t st);

// sums[0] += sum gt^2, sums[1] += sum gi*gt, sums[2] += sum gi^2 over n fp32 elements
const char* launch_grad_dots(const float* gt, const float* gi, float* sums, int64_t n, cudaStream_t st);

struct AdamWArgs {
  __nv_bfloat16* p_bf16;   // parameters stored as bf16 (or null)
  float* p_f32;            // parameters stored as fp32 (or null); exactly one of the two is set
  const float* gt;         // task gradient
  const float* gi;         // information gradient (may be null: plain AdamW on gt)
  float* m;
  float* v;
  const float* scalars;    // device: [coef, grad_scale] (projection coefficient, 1/world * clip factor)
  int64_t n;
  float beta_proj, lr, beta1, beta2, eps, weight_decay;
  float bc1, bc2;          // bias corrections 1-beta^t
};
const char* launch_projected_adamw(const AdamWArgs& a, cudaStream_t st);

// y_i = W_i v_i for a batch of bf16/fp32 matrices given by pointer tables (spectral estimates)
// One power iteration of torch's spectral norm (v <- normalize(W^T u), u <- normalize(W v)) and sigma = u^T W v for one
// row-major matrix, bf16 or fp32, any shape; u (rows), v (cols), t (rows, scratch) fp32. do_iter = 0: sigma only.
const char* launch_sn_power_iter(const void* W, int w_is_bf16, float* u, float* v, float* t, float* sigma_out, int rows,
                                 int cols, int do_iter, float eps, cudaStream_t st);

const char* launch_batched_gemv(const void* const* mats, const float* const* vecs, float* const* outs,
                                const int* rows, const int* cols, const int* is_bf16, int n_mats, int max_rows,
                                cudaStream_t st);

// dst_i (fp32, rows_i x cols_i) += coef[i] * y_i v_i^T for all i in one launch
const char* launch_batched_outer_add(float* const* dsts, const float* const* ys, const float* const* vecs,
                                     const float* coef, const int* rows, const int* cols, int n_mats, int max_rows,
                                     cudaStream_t st);

}  // namespace gd
