// Memory-bound sm_100a kernels of a GDLayer step: causal depthwise conv (forward and
// backward, with sequence-parallel halo rows), the fused gate/stream update (forward and
// backward, RMSNorm of the recovery path included), FP8 block quantisers and column sums.
//
// All of them move 16-byte vectors, keep running windows / row statistics in registers and
// read every input exactly once from HBM.
#include "kernels.h"

#include "common.cuh"

namespace gd {

// =======================================================================================
// causal depthwise convolution
// =======================================================================================
// Block = 8 warps. A lane owns CH consecutive channels (one vector), a warp owns 32*CH
// channels, and the 8 warps of a block take 8 consecutive row tiles of TT time steps, so a
// block covers 8*TT rows x 32*CH channels of one batch row. Taps are padded at the front
// to KMAX so the sliding window has a compile-time length.
constexpr int CONV_TT = 16;

template <int CH> struct VecOf;
template <> struct VecOf<8> { using type = uint4; };
template <> struct VecOf<4> { using type = uint2; };
template <> struct VecOf<2> { using type = uint32_t; };

template <int CH>
__device__ __forceinline__ void load_bf16_vec(const __nv_bfloat16* p, float (&out)[CH]) {
  using V = typename VecOf<CH>::type;
  const V raw = *reinterpret_cast<const V*>(p);
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
  for (int i = 0; i < CH / 2; ++i) {
    const float2 f = unpack_bf16x2(w[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

template <int CH>
__device__ __forceinline__ void store_bf16_vec(__nv_bfloat16* p, const float (&v)[CH]) {
  using V = typename VecOf<CH>::type;
  V raw;
  uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
  for (int i = 0; i < CH / 2; ++i) w[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<V*>(p) = raw;
}

// Row t of the padded input: t >= 0 from x, -(k-1) <= t < 0 from the halo (or zero), else zero.
template <int CH>
__device__ __forceinline__ void load_conv_row(const __nv_bfloat16* x, const __nv_bfloat16* halo, int64_t x_ld,
                                              int T, int k, int b, int t, int ch, int d, float (&out)[CH]) {
  if (t >= 0 && t < T) {
    load_bf16_vec<CH>(x + ((int64_t)b * T + t) * x_ld + ch, out);
  } else if (t < 0 && t >= -(k - 1) && halo != nullptr) {
    load_bf16_vec<CH>(halo + ((int64_t)b * (k - 1) + (t + k - 1)) * d + ch, out);
  } else {
#pragma unroll
    for (int i = 0; i < CH; ++i) out[i] = 0.0f;
  }
}

template <int KMAX, int CH>
__global__ void __launch_bounds__(256)
dwconv_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ halo,
                  const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int B, int T, int d, int k,
                  int64_t x_ld, int64_t out_ld) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = (blockIdx.y * 32 + lane) * CH;
  const int tiles_per_b = (T + 8 * CONV_TT - 1) / (8 * CONV_TT);
  const int b = blockIdx.x / tiles_per_b;
  const int t0 = ((blockIdx.x % tiles_per_b) * 8 + warp) * CONV_TT;
  if (ch >= d || t0 >= T) return;

  float taps[KMAX][CH];
#pragma unroll
  for (int i = 0; i < KMAX; ++i)
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int src = i - (KMAX - k);
      taps[i][c] = src >= 0 ? w[(ch + c) * k + src] : 0.0f;
    }

  float win[KMAX][CH];  // win[i] = input at t - (KMAX-1) + i
#pragma unroll
  for (int i = 0; i < KMAX - 1; ++i) load_conv_row<CH>(x, halo, x_ld, T, k, b, t0 - (KMAX - 1) + i, ch, d, win[i + 1]);

  const int t_end = min(t0 + CONV_TT, T);
#pragma unroll 4
  for (int t = t0; t < t_end; ++t) {
#pragma unroll
    for (int i = 0; i < KMAX - 1; ++i)
#pragma unroll
      for (int c = 0; c < CH; ++c) win[i][c] = win[i + 1][c];
    load_bf16_vec<CH>(x + ((int64_t)b * T + t) * x_ld + ch, win[KMAX - 1]);
    float acc[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) acc[c] = 0.0f;
#pragma unroll
    for (int i = 0; i < KMAX; ++i)
#pragma unroll
      for (int c = 0; c < CH; ++c) acc[c] = fmaf(taps[i][c], win[i][c], acc[c]);
    store_bf16_vec<CH>(out + ((int64_t)b * T + t) * out_ld + ch, acc);
  }
}

// Backward. For every position t in [-(k-1), T): dx[t] = sum_j w[k-1-j] * dc[t+j] (dc outside
// [0,T) is zero); positions t < 0 are the gradient of the halo rows. dw[ch][i] += sum_t dc[t] *
// xpad[t-(k-1)+i]. `dx_tail_add` (B, k-1, d) holds the halo gradient received from the next
// sequence shard; it is added to the last k-1 rows of dx here, before dx leaves the kernel.
template <int KMAX, int CH>
__global__ void __launch_bounds__(256)
dwconv_bwd_kernel(const __nv_bfloat16* __restrict__ dc, const __nv_bfloat16* __restrict__ x,
                  const __nv_bfloat16* __restrict__ halo, const float* __restrict__ w,
                  const __nv_bfloat16* __restrict__ dx_tail_add, __nv_bfloat16* __restrict__ dx,
                  __nv_bfloat16* __restrict__ dhalo, float* __restrict__ dw, int B, int T, int d, int k,
                  int64_t dc_ld, int64_t x_ld) {
  __shared__ float dw_part[8][KMAX][32 * CH + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = (blockIdx.y * 32 + lane) * CH;
  const int tiles_per_b = (T + (k - 1) + 8 * CONV_TT - 1) / (8 * CONV_TT);
  const int b = blockIdx.x / tiles_per_b;
  const int t0 = ((blockIdx.x % tiles_per_b) * 8 + warp) * CONV_TT - (k - 1);  // first tile starts in the halo
  const bool active = ch < d && t0 < T;

  float dwacc[KMAX][CH];
#pragma unroll
  for (int i = 0; i < KMAX; ++i)
#pragma unroll
    for (int c = 0; c < CH; ++c) dwacc[i][c] = 0.0f;

  if (active) {
    float taps[KMAX][CH];  // taps[j] multiplies dc[t+j]: w[k-1-j], zero for j >= k
#pragma unroll
    for (int j = 0; j < KMAX; ++j)
#pragma unroll
      for (int c = 0; c < CH; ++c) taps[j][c] = j < k ? w[(ch + c) * k + (k - 1 - j)] : 0.0f;

    float gwin[KMAX][CH];  // gwin[j] = dc[t + j]
    float xwin[KMAX][CH];  // xwin[i] = xpad[t - (KMAX-1) + i]
    auto load_dc = [&](int t, float (&o)[CH]) {
      if (t >= 0 && t < T) load_bf16_vec<CH>(dc + ((int64_t)b * T + t) * dc_ld + ch, o);
      else {
#pragma unroll
        for (int c = 0; c < CH; ++c) o[c] = 0.0f;
      }
    };
#pragma unroll
    for (int j = 0; j < KMAX - 1; ++j) load_dc(t0 + j, gwin[j + 1]);
#pragma unroll
    for (int i = 0; i < KMAX - 1; ++i) load_conv_row<CH>(x, halo, x_ld, T, k, b, t0 - (KMAX - 1) + i, ch, d, xwin[i + 1]);

    const int t_end = min(t0 + CONV_TT, T);
#pragma unroll 2
    for (int t = t0; t < t_end; ++t) {
#pragma unroll
      for (int j = 0; j < KMAX - 1; ++j)
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          gwin[j][c] = gwin[j + 1][c];
          xwin[j][c] = xwin[j + 1][c];
        }
      load_dc(t + KMAX - 1, gwin[KMAX - 1]);
      load_conv_row<CH>(x, halo, x_ld, T, k, b, t, ch, d, xwin[KMAX - 1]);

      float acc[CH];
#pragma unroll
      for (int c = 0; c < CH; ++c) acc[c] = 0.0f;
#pragma unroll
      for (int j = 0; j < KMAX; ++j)
#pragma unroll
        for (int c = 0; c < CH; ++c) acc[c] = fmaf(taps[j][c], gwin[j][c], acc[c]);

      if (t >= 0) {
        if (dx_tail_add != nullptr && t >= T - (k - 1)) {
          float extra[CH];
          load_bf16_vec<CH>(dx_tail_add + ((int64_t)b * (k - 1) + (t - (T - (k - 1)))) * d + ch, extra);
#pragma unroll
          for (int c = 0; c < CH; ++c) acc[c] += extra[c];
        }
        store_bf16_vec<CH>(dx + ((int64_t)b * T + t) * d + ch, acc);
        // dw: dc[t] (= gwin[0]) times the window that produced out[t]
#pragma unroll
        for (int i = 0; i < KMAX; ++i)
#pragma unroll
          for (int c = 0; c < CH; ++c) dwacc[i][c] = fmaf(gwin[0][c], xwin[i][c], dwacc[i][c]);
      } else if (dhalo != nullptr) {
        store_bf16_vec<CH>(dhalo + ((int64_t)b * (k - 1) + (t + k - 1)) * d + ch, acc);
      }
    }
  }

  // reduce dw over the 8 warps (same channels, different row tiles), then one atomic per (ch, tap)
#pragma unroll
  for (int i = 0; i < KMAX; ++i)
#pragma unroll
    for (int c = 0; c < CH; ++c) dw_part[warp][i][lane * CH + c] = dwacc[i][c];
  __syncthreads();
  for (int idx = threadIdx.x; idx < KMAX * 32 * CH; idx += blockDim.x) {
    const int i = idx / (32 * CH), cc = idx % (32 * CH);
    const int src = i - (KMAX - k);
    const int chan = blockIdx.y * 32 * CH + cc;
    if (src < 0 || chan >= d) continue;
    float s = 0.0f;
#pragma unroll
    for (int wq = 0; wq < 8; ++wq) s += dw_part[wq][i][cc];
    if (s != 0.0f) atomicAdd(dw + (int64_t)chan * k + src, s);
  }
}

template <int KMAX, int CH>
static const char* conv_fwd_launch(const ConvArgs& a, cudaStream_t st) {
  dim3 grid(a.B * ((a.T + 8 * CONV_TT - 1) / (8 * CONV_TT)), (a.d + 32 * CH - 1) / (32 * CH));
  dwconv_fwd_kernel<KMAX, CH><<<grid, 256, 0, st>>>(a.x, a.halo, a.w, a.out, a.B, a.T, a.d, a.k, a.x_ld, a.out_ld);
  return cudaGetLastError() == cudaSuccess ? nullptr : "dwconv_fwd launch failed";
}

template <int KMAX, int CH>
static const char* conv_bwd_launch(const ConvBwdArgs& a, cudaStream_t st) {
  dim3 grid(a.B * ((a.T + a.k - 1 + 8 * CONV_TT - 1) / (8 * CONV_TT)), (a.d + 32 * CH - 1) / (32 * CH));
  dwconv_bwd_kernel<KMAX, CH><<<grid, 256, 0, st>>>(a.dc, a.x, a.halo, a.w, a.dx_tail_add, a.dx, a.dhalo, a.dw,
                                                    a.B, a.T, a.d, a.k, a.dc_ld, a.x_ld);
  return cudaGetLastError() == cudaSuccess ? nullptr : "dwconv_bwd launch failed";
}

const char* launch_dwconv_fwd(const ConvArgs& a, cudaStream_t st) {
  if (a.k < 1 || a.k > 16) return "dwconv: kernel width must be in [1, 16]";
  if (a.d % 8 != 0) return "dwconv: d must be a multiple of 8";
  if (a.k <= 4) return conv_fwd_launch<4, 8>(a, st);
  if (a.k <= 8) return conv_fwd_launch<8, 4>(a, st);
  return conv_fwd_launch<16, 2>(a, st);
}

const char* launch_dwconv_bwd(const ConvBwdArgs& a, cudaStream_t st) {
  if (a.k < 1 || a.k > 16) return "dwconv: kernel width must be in [1, 16]";
  if (a.d % 8 != 0) return "dwconv: d must be a multiple of 8";
  if (a.k <= 4) return conv_bwd_launch<4, 4>(a, st);   // narrower vectors: two windows + dw accumulators per lane
  if (a.k <= 8) return conv_bwd_launch<8, 2>(a, st);
  return conv_bwd_launch<16, 2>(a, st);
}

// =======================================================================================
// gate / stream update: one warp per row, 8 columns per lane per step
// =======================================================================================
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&o)[8]) { load_bf16_vec<8>(p, o); }
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&v)[8]) { store_bf16_vec<8>(p, v); }

// fwd' = c*g + s*R, side' = c*(1-g) + s*(1-R) with g = sigmoid(g_pre),
// R = sigmoid(z * rstd(z) * w_r). Also writes rstd(z) per row, optionally g, and adds the
// sum of g over the block's rows to gate_sum (for the mean forward-gate value).
__global__ void __launch_bounds__(256)
gate_update_fwd_kernel(const GateFwdArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wpb = blockDim.x >> 5;
  float gsum = 0.0f;
  for (int64_t row = (int64_t)blockIdx.x * wpb + warp; row < a.rows; row += (int64_t)gridDim.x * wpb) {
    const __nv_bfloat16* zr = a.z + row * a.d;
    float ssq = 0.0f;
    for (int col = lane * 8; col < a.d; col += 256) {
      float zv[8];
      ld8(zr + col, zv);
#pragma unroll
      for (int i = 0; i < 8; ++i) ssq = fmaf(zv[i], zv[i], ssq);
    }
    ssq = warp_sum(ssq);
    const float rstd = rsqrtf(ssq / (float)a.d + a.eps_r);
    if (lane == 0 && a.rstd_out != nullptr) a.rstd_out[row] = rstd;
    for (int col = lane * 8; col < a.d; col += 256) {
      float zv[8], gp[8], cv[8], sv[8], wr[8], fo[8], so[8], gv[8];
      ld8(zr + col, zv);
      ld8(a.g_pre + row * a.d + col, gp);
      ld8(a.c + row * a.c_ld + col, cv);
      ld8(a.s + row * a.s_ld + col, sv);
#pragma unroll
      for (int i = 0; i < 8; ++i) wr[i] = a.w_r[col + i];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float R = sigmoidf_(zv[i] * rstd * wr[i]);
        const float g = sigmoidf_(gp[i]);
        gv[i] = g;
        gsum += g;
        fo[i] = cv[i] * g + sv[i] * R;
        so[i] = cv[i] * (1.0f - g) + sv[i] * (1.0f - R);
      }
      st8(a.fwd_out + row * a.d + col, fo);
      st8(a.side_out + row * a.d + col, so);
      if (a.gate_out != nullptr) st8(a.gate_out + row * a.d + col, gv);
    }
  }
  if (a.gate_sum != nullptr) {
    gsum = warp_sum(gsum);
    __shared__ float part[8];
    if (lane == 0) part[warp] = gsum;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.0f;
      for (int i = 0; i < wpb; ++i) t += part[i];
      atomicAdd(a.gate_sum, t);
    }
  }
}

const char* launch_gate_update_fwd(const GateFwdArgs& a, cudaStream_t st) {
  if (a.d % 8 != 0) return "gate_update: d must be a multiple of 8";
  const int64_t blocks = (a.rows + 7) / 8;
  const int grid = (int)(blocks < 148 * 8 ? blocks : 148 * 8);
  gate_update_fwd_kernel<<<grid, 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "gate_update_fwd launch failed";
}

// Backward of the update and of both activations feeding it. Per row (one warp):
//   g = sigmoid(g_pre), zh = z*rstd, R = sigmoid(zh*w_r), D = dF - dS
//   dg_pre = (D*c + dgm) * g(1-g)            dgm = d(loss)/d(mean g) / (rows*d)
//   dq     = dg_pre * rstd_g                 (gradient of the un-normalised gate GEMM output)
//   T_row  = sum_n dg_pre * (g_pre - b2g)    (for the rstd term of the gate RMSNorm)
//   dc_dir = dF*g + dS*(1-g),  ds_dir = dF*R + dS*(1-R)
//   dy = D*s*R(1-R),  dzh = dy*w_r,  dz = rstd*(dzh - zh*mean_n(dzh*zh))
// Column sums: db2g += dg_pre, dw_r += dy*zh, db2r += dz (shared-memory partials, then atomics).
// Outputs: dq (bf16), dz (bf16), dsc[:, :d] = ds_dir, dsc[:, d:] = dc_dir (bf16, row pitch 2d),
// rowcoef[row] = rstd_g^2 / d * T_row.
__global__ void __launch_bounds__(256)
gate_update_bwd_kernel(const GateBwdArgs a) {
  extern __shared__ float colacc_all[];  // [warps][3][d]: db2g, dw_r, db2r; each warp owns a slab, no atomics
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wpb = blockDim.x >> 5;
  float* colacc = colacc_all + (size_t)warp * 3 * a.d;
  for (int i = lane; i < 3 * a.d; i += 32) colacc[i] = 0.0f;
  __syncwarp();
  const float dgm = (a.dgate_mean != nullptr) ? a.dgate_mean[0] / ((float)a.rows * (float)a.d) : 0.0f;

  for (int64_t row = (int64_t)blockIdx.x * wpb + warp; row < a.rows; row += (int64_t)gridDim.x * wpb) {
    const float rstd = a.rstd_z[row];
    float rstd_g;
    {
      float ssum = 0.0f;
      for (int p = 0; p < a.ssq_parts; ++p) ssum += a.ssq_g[row * a.ssq_parts + p];
      rstd_g = rsqrtf(ssum / (float)a.d + a.eps_g);
    }
    // pass 1: row reductions sum(dzh*zh) and T_row
    float dot_z = 0.0f, t_row = 0.0f;
    for (int col = lane * 8; col < a.d; col += 256) {
      float dF[8], dS[8], zv[8], sv[8], gp[8], cv[8];
      ld8(a.dF + row * a.dF_ld + col, dF);
      ld8(a.dS + row * a.dS_ld + col, dS);
      ld8(a.z + row * a.d + col, zv);
      ld8(a.s + row * a.s_ld + col, sv);
      ld8(a.g_pre + row * a.d + col, gp);
      ld8(a.c + row * a.c_ld + col, cv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float wr = a.w_r[col + i];
        const float zh = zv[i] * rstd;
        const float R = sigmoidf_(zh * wr);
        const float D = dF[i] - dS[i];
        const float dzh = D * sv[i] * R * (1.0f - R) * wr;
        dot_z = fmaf(dzh, zh, dot_z);
        const float g = sigmoidf_(gp[i]);
        const float dgp = (D * cv[i] + dgm) * g * (1.0f - g);
        const float b2 = a.b2g_f32 ? reinterpret_cast<const float*>(a.b2g)[col + i]
                                   : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.b2g)[col + i]);
        t_row = fmaf(dgp, gp[i] - b2, t_row);
      }
    }
    dot_z = warp_sum(dot_z) / (float)a.d;
    t_row = warp_sum(t_row);
    if (lane == 0) a.rowcoef[row] = rstd_g * rstd_g / (float)a.d * t_row;

    // pass 2: outputs (inputs come back from L1/L2)
    for (int col = lane * 8; col < a.d; col += 256) {
      float dF[8], dS[8], zv[8], sv[8], gp[8], cv[8], dq[8], dz[8], dcd[8], dsd[8];
      ld8(a.dF + row * a.dF_ld + col, dF);
      ld8(a.dS + row * a.dS_ld + col, dS);
      ld8(a.z + row * a.d + col, zv);
      ld8(a.s + row * a.s_ld + col, sv);
      ld8(a.g_pre + row * a.d + col, gp);
      ld8(a.c + row * a.c_ld + col, cv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float wr = a.w_r[col + i];
        const float zh = zv[i] * rstd;
        const float R = sigmoidf_(zh * wr);
        const float g = sigmoidf_(gp[i]);
        const float D = dF[i] - dS[i];
        const float dgp = (D * cv[i] + dgm) * g * (1.0f - g);
        const float dy = D * sv[i] * R * (1.0f - R);
        const float dzv = rstd * (dy * wr - zh * dot_z);
        dq[i] = dgp * rstd_g;
        dz[i] = dzv;
        dcd[i] = dF[i] * g + dS[i] * (1.0f - g);
        dsd[i] = dF[i] * R + dS[i] * (1.0f - R);
        colacc[col + i] += dgp;                 // this lane is the only writer of these columns
        colacc[a.d + col + i] += dy * zh;
        colacc[2 * a.d + col + i] += dzv;
      }
      st8(a.dq + row * a.d + col, dq);
      st8(a.dz + row * a.d + col, dz);
      st8(a.dsc + row * 2 * a.d + col, dsd);
      st8(a.dsc + row * 2 * a.d + a.d + col, dcd);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 3 * a.d; i += blockDim.x) {
    float t = 0.0f;
    for (int w = 0; w < wpb; ++w) t += colacc_all[(size_t)w * 3 * a.d + i];
    float* dst = i < a.d ? a.db2g + i : (i < 2 * a.d ? a.dw_r + (i - a.d) : a.db2r + (i - 2 * a.d));
    atomicAdd(dst, t);
  }
}

const char* launch_gate_update_bwd(const GateBwdArgs& a, cudaStream_t st) {
  if (a.d % 8 != 0) return "gate_update_bwd: d must be a multiple of 8";
  int warps = 8;
  while (warps > 1 && (size_t)warps * 3 * a.d * sizeof(float) > 100 * 1024) warps >>= 1;
  const size_t smem = (size_t)warps * 3 * a.d * sizeof(float);
  if (smem > 200 * 1024) return "gate_update_bwd: d too large for the column accumulators";
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gate_update_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    attr = true;
  }
  const int64_t blocks = (a.rows + warps - 1) / warps;
  const int grid = (int)(blocks < 148 * 2 ? blocks : 148 * 2);
  gate_update_bwd_kernel<<<grid, warps * 32, smem, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "gate_update_bwd launch failed";
}

// =======================================================================================
// RMSNorm forward / backward (generic rows x d, d multiple of 8)
// =======================================================================================
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   float* __restrict__ rstd_out, int64_t rows, int d, float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  for (int64_t row = (int64_t)blockIdx.x * wpb + warp; row < rows; row += (int64_t)gridDim.x * wpb) {
    float ssq = 0.0f;
    for (int col = lane * 8; col < d; col += 256) {
      float v[8];
      ld8(x + row * d + col, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) ssq = fmaf(v[i], v[i], ssq);
    }
    const float rstd = rsqrtf(warp_sum(ssq) / (float)d + eps);
    if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
    for (int col = lane * 8; col < d; col += 256) {
      float v[8], o[8];
      ld8(x + row * d + col, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = v[i] * rstd * w[col + i];
      st8(y + row * d + col, o);
    }
  }
}

// dx = rstd * (dy*w - xh * mean(dy*w*xh)), dw += sum_rows dy * xh
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const float* __restrict__ w, const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw, int64_t rows, int d) {
  extern __shared__ float colacc[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  for (int i = threadIdx.x; i < d; i += blockDim.x) colacc[i] = 0.0f;
  __syncthreads();
  for (int64_t row = (int64_t)blockIdx.x * wpb + warp; row < rows; row += (int64_t)gridDim.x * wpb) {
    const float rstd = rstd_in[row];
    float dot = 0.0f;
    for (int col = lane * 8; col < d; col += 256) {
      float g[8], v[8];
      ld8(dy + row * d + col, g);
      ld8(x + row * d + col, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) dot = fmaf(g[i] * w[col + i], v[i] * rstd, dot);
    }
    dot = warp_sum(dot) / (float)d;
    for (int col = lane * 8; col < d; col += 256) {
      float g[8], v[8], o[8];
      ld8(dy + row * d + col, g);
      ld8(x + row * d + col, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = v[i] * rstd;
        o[i] = rstd * (g[i] * w[col + i] - xh * dot);
        atomicAdd(&colacc[col + i], g[i] * xh);
      }
      st8(dx + row * d + col, o);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) atomicAdd(dw + i, colacc[i]);
}

const char* launch_rmsnorm_fwd(const __nv_bfloat16* x, const float* w, __nv_bfloat16* y, float* rstd, int64_t rows,
                               int d, float eps, cudaStream_t st) {
  if (d % 8 != 0) return "rmsnorm: d must be a multiple of 8";
  const int64_t blocks = (rows + 7) / 8;
  rmsnorm_fwd_kernel<<<(int)(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, st>>>(x, w, y, rstd, rows, d, eps);
  return cudaGetLastError() == cudaSuccess ? nullptr : "rmsnorm_fwd launch failed";
}

const char* launch_rmsnorm_bwd(const __nv_bfloat16* dy, const __nv_bfloat16* x, const float* w, const float* rstd,
                               __nv_bfloat16* dx, float* dw, int64_t rows, int d, cudaStream_t st) {
  if (d % 8 != 0 || d > 16384) return "rmsnorm_bwd: d must be a multiple of 8 and at most 16384";
  const int64_t blocks = (rows + 7) / 8;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    attr = true;
  }
  rmsnorm_bwd_kernel<<<(int)(blocks < 148 * 4 ? blocks : 148 * 4), 256, d * sizeof(float), st>>>(dy, x, w, rstd, dx,
                                                                                                dw, rows, d);
  return cudaGetLastError() == cudaSuccess ? nullptr : "rmsnorm_bwd launch failed";
}

// =======================================================================================
// FP8 (e4m3) block quantisation
// =======================================================================================
// One block quantises a 128 x 128 tile of a bf16 matrix x[rows][cols] (row pitch x_ld),
// optionally through silu. Two independent outputs, each optional:
//   row-major  q_row[r][c]  with scales per (row, 128-col block)   [ROWS]  or per tile [BLOCK]
//   transposed q_col[c][r]  with scales per (col, 128-row block)   [COLS]  or per tile [BLOCK]
// Scale layouts (all fp32, scale = amax/448, 1 for an all-zero block):
//   ROWS : s_row[cb * s_row_ld + r]            (GEMM A operand: sa[kb*ld + m])
//   COLS : s_col[rb * s_col_ld + c]            (A operand of the weight-gradient GEMM)
//   BLOCK (row-major) : s_row[rb * n_cb + cb]  (GEMM B operand: sb[nb*KB + kb])
//   BLOCK (transposed): s_col[cb * n_rb + rb]
__global__ void __launch_bounds__(256)
quant_tile_kernel(const QuantArgs a) {
  __shared__ float s_colmax[16][128];
  __shared__ float s_scale_col[128];
  __shared__ float s_tilemax;
  __shared__ __align__(16) __nv_bfloat16 s_tile[128][128 + 8];

  const int tid = threadIdx.x;
  const int tr = tid >> 4;          // 0..15: row within a pass
  const int tc = (tid & 15) * 8;    // first of 8 columns
  const int64_t r0 = (int64_t)blockIdx.y * 128;
  const int c0 = blockIdx.x * 128;
  const int n_cb = gridDim.x, n_rb = gridDim.y;

  float v[8][8];
  float colmax[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) colmax[i] = 0.0f;

#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const int64_t r = r0 + p * 16 + tr;
    const int c = c0 + tc;
    if (r < a.rows && c < a.cols) {
      load_bf16_vec<8>(a.x + r * a.x_ld + c, v[p]);
      if (a.pre_silu) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[p][i] = __bfloat162float(__float2bfloat16(siluf_(v[p][i])));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[p][i] = 0.0f;
    }
    float rmax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float av = fabsf(v[p][i]);
      rmax = fmaxf(rmax, av);
      colmax[i] = fmaxf(colmax[i], av);
    }
    // row amax across the 16 threads that share this row
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
    if (a.q_row != nullptr && a.row_mode == QUANT_ROWS) {
      const float sc = rmax > 0.0f ? rmax / 448.0f : 1.0f;
      const float inv = 1.0f / sc;
      if (r < a.rows && c < a.cols) {
        uint8_t q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = to_e4m3(v[p][i] * inv);
        *reinterpret_cast<uint2*>(a.q_row + r * a.q_row_ld + c) = *reinterpret_cast<uint2*>(q);
        if ((tid & 15) == 0) a.s_row[(int64_t)blockIdx.x * a.s_row_ld + r] = sc;
      }
    }
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) s_colmax[tr][tc + i] = colmax[i];
  __syncthreads();
  if (tid < 128) {
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j) m = fmaxf(m, s_colmax[j][tid]);
    s_scale_col[tid] = m;  // column amax for now
  }
  __syncthreads();
  if (tid < 32) {
    float m = fmaxf(fmaxf(s_scale_col[tid], s_scale_col[tid + 32]), fmaxf(s_scale_col[tid + 64], s_scale_col[tid + 96]));
    m = warp_max(m);
    if (tid == 0) s_tilemax = m;
  }
  __syncthreads();
  const float tile_scale = s_tilemax > 0.0f ? s_tilemax / 448.0f : 1.0f;

  if (a.q_row != nullptr && a.row_mode == QUANT_BLOCK) {
    const float inv = 1.0f / tile_scale;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      const int64_t r = r0 + p * 16 + tr;
      const int c = c0 + tc;
      if (r < a.rows && c < a.cols) {
        uint8_t q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = to_e4m3(v[p][i] * inv);
        *reinterpret_cast<uint2*>(a.q_row + r * a.q_row_ld + c) = *reinterpret_cast<uint2*>(q);
      }
    }
    if (tid == 0) a.s_row[(int64_t)blockIdx.y * n_cb + blockIdx.x] = tile_scale;
  }

  if (a.q_col != nullptr) {
    // stage the tile row-major as bf16 (16-byte stores, conflict free), then every thread walks half
    // of one column: 64 values -> 64 output bytes of one transposed row
#pragma unroll
    for (int p = 0; p < 8; ++p) store_bf16_vec<8>(&s_tile[p * 16 + tr][tc], v[p]);
    __syncthreads();
    const int oc = tid >> 1, half = tid & 1;
    const float cm = s_scale_col[oc];
    const float sc = a.col_mode == QUANT_COLS ? (cm > 0.0f ? cm / 448.0f : 1.0f) : tile_scale;
    const float inv = 1.0f / sc;
    const int c = c0 + oc;
    const int64_t rbase = r0 + half * 64;
    if (c < a.cols) {
#pragma unroll
      for (int seg = 0; seg < 4; ++seg) {
        uint8_t q[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) q[i] = to_e4m3(__bfloat162float(s_tile[half * 64 + seg * 16 + i][oc]) * inv);
        if (rbase + seg * 16 < a.rows)
          *reinterpret_cast<uint4*>(a.q_col + (int64_t)c * a.q_col_ld + rbase + seg * 16) = *reinterpret_cast<uint4*>(q);
      }
    }
    if (a.col_mode == QUANT_COLS) {
      if (tid < 128 && c0 + tid < a.cols) {
        const float cm = s_scale_col[tid];
        a.s_col[(int64_t)blockIdx.y * a.s_col_ld + c0 + tid] = cm > 0.0f ? cm / 448.0f : 1.0f;
      }
    } else if (tid == 0) {
      a.s_col[(int64_t)blockIdx.x * n_rb + blockIdx.y] = tile_scale;
    }
  }
}

// Row-only quantiser (1x128 blocks): 16 lanes own one block of one row (8 values each), the block
// amax is a 4-step shuffle; no shared memory, every byte moved once with 16-byte loads.
__global__ void __launch_bounds__(256)
quant_rows_kernel(const QuantArgs a) {
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int groups_per_row = a.cols / 8;            // cols is a multiple of 128 here
  const int c = (int)(gid % groups_per_row) * 8;
  const bool live = gid / groups_per_row < a.rows;   // dead lanes stay for the shuffles, store nothing
  const int64_t r = live ? gid / groups_per_row : a.rows - 1;
  float v[8];
  load_bf16_vec<8>(a.x + r * a.x_ld + c, v);
  if (a.pre_silu) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(__float2bfloat16(siluf_(v[i])));
  }
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const float sc = m > 0.0f ? m / 448.0f : 1.0f;
  const float inv = 1.0f / sc;
  uint8_t q[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) q[i] = to_e4m3(v[i] * inv);
  if (!live) return;
  *reinterpret_cast<uint2*>(a.q_row + r * a.q_row_ld + c) = *reinterpret_cast<uint2*>(q);
  if ((threadIdx.x & 15) == 0) a.s_row[(int64_t)(c >> 7) * a.s_row_ld + r] = sc;
}

const char* launch_quant_tile(const QuantArgs& a, cudaStream_t st) {
  if (a.cols % 8 != 0) return "quantise: cols must be a multiple of 8";
  if (a.q_col == nullptr && a.q_row != nullptr && a.row_mode == QUANT_ROWS && a.cols % 128 == 0) {
    const int64_t threads = a.rows * (a.cols / 8);
    quant_rows_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? nullptr : "quant_rows launch failed";
  }
  if (a.q_col != nullptr && a.rows % 16 != 0) return "quantise: transposed output needs rows % 16 == 0";
  dim3 grid((a.cols + 127) / 128, (unsigned)((a.rows + 127) / 128));
  quant_tile_kernel<<<grid, 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "quant_tile launch failed";
}

// Per-tensor quantisation with a given scale (the reference's delayed-scaling recipe): writes the
// row-major e4m3 tensor, optionally the transposed one, and folds the tensor's amax into amax_out.
__global__ void __launch_bounds__(256)
quant_tensor_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale, uint8_t* __restrict__ q_row,
                    uint8_t* __restrict__ q_col, float* __restrict__ amax_out, int64_t rows, int cols) {
  __shared__ uint8_t s_t[64][64 + 4];
  __shared__ float s_max[8];
  const int64_t r0 = (int64_t)blockIdx.y * 64;
  const int c0 = blockIdx.x * 64;
  const float sc = scale[0];
  float amax = 0.0f;
  for (int idx = threadIdx.x; idx < 64 * 64; idx += 256) {
    const int rr = idx >> 6, cc = idx & 63;
    const int64_t r = r0 + rr;
    const int c = c0 + cc;
    uint8_t q = 0;
    if (r < rows && c < cols) {
      const float v = __bfloat162float(x[r * cols + c]);
      amax = fmaxf(amax, fabsf(v));
      q = to_e4m3(fminf(fmaxf(v * sc, -448.0f), 448.0f));
      q_row[r * cols + c] = q;
    }
    s_t[cc][rr] = q;
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0 && amax_out != nullptr) {
    float m = 0.0f;
    for (int i = 0; i < 8; ++i) m = fmaxf(m, s_max[i]);
    atomicMax(reinterpret_cast<int*>(amax_out), __float_as_int(m));  // valid for non-negative floats
  }
  if (q_col != nullptr) {
    for (int idx = threadIdx.x; idx < 64 * 64; idx += 256) {
      const int cc = idx >> 6, rr = idx & 63;
      const int64_t r = r0 + rr;
      const int c = c0 + cc;
      if (r < rows && c < cols) q_col[(int64_t)c * rows + r] = s_t[cc][rr];
    }
  }
}

const char* launch_quant_tensor(const __nv_bfloat16* x, const float* scale, uint8_t* q_row, uint8_t* q_col,
                                float* amax_out, int64_t rows, int cols, cudaStream_t st) {
  dim3 grid((cols + 63) / 64, (unsigned)((rows + 63) / 64));
  quant_tensor_kernel<<<grid, 256, 0, st>>>(x, scale, q_row, q_col, amax_out, rows, cols);
  return cudaGetLastError() == cudaSuccess ? nullptr : "quant_tensor launch failed";
}

// =======================================================================================
// column sums: out[c] += sum_r x[r][c]
// =======================================================================================
__global__ void __launch_bounds__(256)
colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int64_t rows, int cols, int64_t ld,
              int rows_per_block) {
  __shared__ float part[8][256 + 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + lane * 8;
  const int64_t r_begin = (int64_t)blockIdx.y * rows_per_block;
  const int64_t r_end = r_begin + rows_per_block < rows ? r_begin + rows_per_block : rows;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  if (col < cols) {
    for (int64_t r = r_begin + warp; r < r_end; r += 8) {
      float v[8];
      ld8(x + r * ld + col, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) part[warp][lane * 8 + i] = acc[i];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < cols) {
    float s = 0.0f;
#pragma unroll
    for (int wq = 0; wq < 8; ++wq) s += part[wq][threadIdx.x];
    atomicAdd(out + c, s);
  }
}

const char* launch_colsum(const __nv_bfloat16* x, float* out, int64_t rows, int cols, int64_t ld, cudaStream_t st) {
  if (cols % 8 != 0) return "colsum: cols must be a multiple of 8";
  const int rpb = 256;
  dim3 grid((cols + 255) / 256, (unsigned)((rows + rpb - 1) / rpb));
  colsum_kernel<<<grid, 256, 0, st>>>(x, out, rows, cols, ld, rpb);
  return cudaGetLastError() == cudaSuccess ? nullptr : "colsum launch failed";
}

// W2w[i][j] = W2[i][j] * w_norm[j]  (folds the RMSNorm weight into the GEMM that follows it)
__global__ void scale_cols_kernel(const __nv_bfloat16* __restrict__ w, const float* __restrict__ colw,
                                  __nv_bfloat16* __restrict__ out, int64_t n, int cols) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  float v[8];
  ld8(w + i, v);
  const int c = (int)(i % cols);
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] *= colw[c + j];
  st8(out + i, v);
}

const char* launch_scale_cols(const __nv_bfloat16* w, const float* colw, __nv_bfloat16* out, int64_t rows, int cols,
                              cudaStream_t st) {
  if (cols % 8 != 0) return "scale_cols: cols must be a multiple of 8";
  const int64_t n = rows * cols;
  scale_cols_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, st>>>(w, colw, out, n, cols);
  return cudaGetLastError() == cudaSuccess ? nullptr : "scale_cols launch failed";
}

// Backward of the folding: given dW2w (fp32), dW2 += dW2w * w_norm[j], dw_norm[j] += sum_i dW2w[i][j] * W2[i][j]
__global__ void __launch_bounds__(256)
unscale_cols_bwd_kernel(const float* __restrict__ dW2w, const __nv_bfloat16* __restrict__ W2,
                        const float* __restrict__ colw, float* __restrict__ dW2, float* __restrict__ dcolw, int rows,
                        int cols) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= cols) return;
  const int r_begin = blockIdx.y * 64, r_end = min(r_begin + 64, rows);
  const float wn = colw[c];
  float acc = 0.0f;
  for (int r = r_begin; r < r_end; ++r) {
    const float g = dW2w[(int64_t)r * cols + c];
    dW2[(int64_t)r * cols + c] += g * wn;
    acc = fmaf(g, __bfloat162float(W2[(int64_t)r * cols + c]), acc);
  }
  atomicAdd(dcolw + c, acc);
}

const char* launch_unscale_cols_bwd(const float* dW2w, const __nv_bfloat16* W2, const float* colw, float* dW2,
                                    float* dcolw, int rows, int cols, cudaStream_t st) {
  dim3 grid((cols + 255) / 256, (rows + 63) / 64);
  unscale_cols_bwd_kernel<<<grid, 256, 0, st>>>(dW2w, W2, colw, dW2, dcolw, rows, cols);
  return cudaGetLastError() == cudaSuccess ? nullptr : "unscale_cols_bwd launch failed";
}

}  // namespace gd
