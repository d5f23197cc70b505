// Host-visible interface of the sm_100a tensor-core GEMMs (gemm_sm100.cu).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gd {

struct Status;

enum AuxMode : int {
  AUX_NONE = 0,
  AUX_ADD = 1,            // v += aux
  AUX_MUL_SILU_GRAD = 2,  // v *= silu'(aux)
  AUX_RMS_SILU_BWD = 3,   // v = (v - silu(aux) * rowcoef[m]) * silu'(aux)
};

enum Activation : int { ACT_NONE = 0, ACT_SILU = 1 };

struct GemmOperands {
  const void* a;  // K-major: [M][K] row-major. MN-major: [K][M] row-major.
  const void* b;  // K-major: [N][K] row-major. MN-major: [K][N] row-major.
  int64_t a_ld;   // row pitch in elements
  int64_t b_ld;
};

struct GemmShape {
  int M, N, K;
  int a_mn, b_mn;   // bf16 only: operand is MN-major in memory
  const float* sa;  // fp8: scales of A, sa[kb * sa_ld + m]
  const float* sb;  // fp8: scales of B, sb[(n / 128) * ceil(K/128) + kb]
  int64_t sa_ld;
  int splits;       // split-K shares (set by the launcher)
  const uint8_t* sfa_packed;  // hardware-scaled fp8: UE8M0 chunks of A, (M/128, K/128, 512) bytes
  const uint8_t* sfb_packed;  // hardware-scaled fp8: UE8M0 chunks of B, (N/128, K/128, 512) bytes
  // Parameter all-gather carried by the GEMM (CTA-pair kernels; the launcher runs a plain copy kernel first when
  // another kernel form is chosen). `jobs`: n_jobs x 4 int64 words (src, dst, counter, 16-byte vectors), see
  // run_gather_jobs: the second CTA of every pair has an idle warp (only the leader issues the MMAs) that pulls
  // the listed ranges from their owners' memory into this GPU's staging area while the tensor cores work, and
  // adds one to each job's counter when its bytes have landed.
  const int64_t* jobs;
  int n_jobs;
  // Hardware-scaled fp8 pair kernel: when set, rows [128 nb, 128 nb + 128) of B and chunk row nb of its packed
  // scales are being gathered by this very launch; the producer warp waits (bounded) for the counters b_ready[nb]
  // and sfb_ready[nb] to reach b_target and sfb_target before the first bulk copy of a tile in column block nb.
  const uint32_t* b_ready;
  const uint32_t* sfb_ready;
  uint32_t b_target, sfb_target;
};

// Stand-alone form of the gather jobs (one warp per job slot), for launches that cannot carry them.
const char* launch_gather_jobs(const int64_t* jobs, int n_jobs, cudaStream_t stream);

// Applied in this order to the fp32 accumulator of element (m, n):
//   v = acc * row_scale(m) + bias[n];  aux;  pre_out = v;  v = act(v);  out (+)= v
struct GemmEpilogue {
  void* out;            // bf16 (default) or fp32 [M][out_ld]
  int64_t out_ld;
  int out_f32;
  int accumulate;       // out += v instead of out = v
  int atomic;           // fp32 out += v with atomics (set by the launcher for split-K)
  // Reduce-scatter from the epilogue: when peer_out is set, `out` is a view of this rank's flat fp32
  // gradient buffer at element offset flat_off, and every 32-column chunk is added (vector atomics over
  // NVLink) into the buffer of the rank that owns that part of the flat range: peer_out[idx / shard_elems] + idx.
  float* const* peer_out;
  int64_t flat_off;
  int64_t shard_elems;
  // Hardware-scaled fp8 kernel only: also leave silu(v) (q8_silu) or v as the e4m3 A operand of the next GEMM,
  // q8[m][n] with one power-of-two scale per 64 columns of a row, written as the two UE8M0 bytes of the packed
  // chunk (m / 128, n / 128) that belong to these columns. out may then be null (nothing but q8 is wanted).
  uint8_t* q8;
  int64_t q8_ld;
  uint8_t* q8_p;
  int64_t q8_p_stride;
  int q8_silu;
  const void* bias;     // [N] bf16 or fp32, may be null
  int bias_f32;
  const float* row_scale;   // [M], may be null
  const float* ssq_in;      // [M][ssq_parts]: row_scale = rsqrt(sum/norm_dim + norm_eps) when row_scale is null
  int ssq_parts;
  int norm_dim;
  float norm_eps;
  const __nv_bfloat16* aux; // [M][aux_ld], may be null
  int64_t aux_ld;
  int aux_mode;
  const float* rowcoef;     // [M], used by AUX_RMS_SILU_BWD
  __nv_bfloat16* pre_out;   // [M][pre_ld]: value before the activation, may be null
  int64_t pre_ld;
  int act;
  float* ssq_out;           // [M][ssq_parts]: per-row partial sums of squares of the stored values
  int tma_mask;             // set by the launcher: bit 0 out, bit 1 pre_out, bit 2 q8 leave through tiled bulk stores
};

const char* launch_gemm_bf16(const GemmOperands& op, const GemmShape& g, const GemmEpilogue& e, Status* status,
                             cudaStream_t stream);
const char* launch_gemm_fp8_mx(const GemmOperands& op, const GemmShape& g, const GemmEpilogue& e, Status* status,
                               cudaStream_t stream);
const char* launch_gemm_fp8(const GemmOperands& op, const GemmShape& g, const GemmEpilogue& e, Status* status,
                            cudaStream_t stream);

// CTA pairs (two-SM tensor-core tiles) that can be resident at once on the current device; 0 or less when the
// pair kernels cannot be launched and the single-CTA kernels are used instead.
int gemm_pair_capacity();

// Use (1) or bypass (0) the CTA-pair form of the hardware-scaled FP8 GEMM; default from GDNET_MX_PAIR (on unless it is 0).
void gemm_set_mx_pair(int on);

}  // namespace gd
