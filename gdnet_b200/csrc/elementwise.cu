// Memory-bound sm_100a kernels of a GDLayer step: causal depthwise conv (forward and
// backward, with sequence-parallel halo rows), the fused gate/stream update (forward and
// backward, RMSNorm of the recovery path included), FP8 block quantisers and column sums.
//
// All of them move 16-byte vectors, keep running windows / row statistics in registers and
// read every input exactly once from HBM.
#include <algorithm>
#include <cstdlib>
#include "kernels.h"

#include "common.cuh"
#include "launch.h"

namespace gd {

// =======================================================================================
// causal depthwise convolution
// =======================================================================================
// x is (B, T, d) with d contiguous; a lane always owns a vector of consecutive channels, so a warp
// reads and writes 512 contiguous bytes of one row.

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

// ---------------------------------------------------------------------------------------
// point-wise formulation: one thread per output vector (8 channels of one time step); the taps come
// from a transposed table wt[k][d], so a warp reads them as contiguous vectors. Every load
// is independent, so the kernels run at full occupancy with many loads in flight; the k-fold
// re-read of neighbouring rows is served by L1/L2 (blocks cover consecutive time steps).
// ---------------------------------------------------------------------------------------
template <int KT>
__global__ void __launch_bounds__(256)
dwconv_fwd_pt_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ halo,
                     const float* __restrict__ wt, __nv_bfloat16* __restrict__ out, int B, int T, int d, int k,
                     int64_t x_ld, int64_t out_ld, const RowQuantOut qo) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = (blockIdx.y * 32 + lane) * 8;
  const int row = blockIdx.x * 8 + warp;      // 8 consecutive time steps per block (B*T < 2^31, checked by the launcher)
  if (row >= B * T) return;                   // warp-uniform
  if (ch >= d) {                              // with a quantised output d is a multiple of 128: whole 16-lane groups leave
    return;
  }
  const int b = row / T, t = row - b * T;
  if (KT > 0) k = KT;
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = 0.0f;
#pragma unroll
  for (int i = 0; i < (KT > 0 ? KT : k); ++i) {
    float in[8];
    load_conv_row<8>(x, halo, x_ld, T, k, b, t - (k - 1) + i, ch, d, in);
    const float4 w0 = *reinterpret_cast<const float4*>(wt + (int64_t)i * d + ch);
    const float4 w1 = *reinterpret_cast<const float4*>(wt + (int64_t)i * d + ch + 4);
    const float tap[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = fmaf(tap[c], in[c], acc[c]);
  }
  store_bf16_vec<8>(out + (int64_t)row * out_ld + ch, acc);
  if (qo.q != nullptr) {
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = __bfloat162float(__float2bfloat16(acc[c]));
    quant_emit_8(qo, acc, row, ch, true);
  }
}

// Sliding-window formulation of the forward conv: a thread owns 8 channels and TT consecutive time steps of one
// sequence, keeps the last KT-1 input rows in registers and loads every further row once (TT + KT - 1 row loads
// for TT outputs instead of KT per output). The loads of a strip are independent, so the compiler keeps them
// all in flight.
// After a warp has stored its rows into a neighbour's slot: count it, and let the last one raise the flag.
__device__ __forceinline__ void sp_signal_after_store(const ConvSp& sp, int dst, uint32_t total) {
  __threadfence_system();
  __syncwarp();
  if ((threadIdx.x & 31) == 0) {
    const uint32_t prev = atomicAdd(sp.counter, 1u);
    if (prev == total - 1) {
      *sp.counter = 0u;               // ready for the next launch that uses this word
      __threadfence_system();
      st_release_sys(sp.flags[dst] + sp.flag_index, sp.seq);
    }
  }
}

// One lane polls this rank's flag; the result is broadcast. false = the wait ran out (reported).
__device__ __forceinline__ bool sp_wait_neighbour(const ConvSp& sp, int src, int site) {
  uint32_t ok = 1;
  if ((threadIdx.x & 31) == 0) {
    ok = wait_flag_ge(sp.flags[sp.rank] + sp.flag_index, sp.seq, budget_or_default(sp.budget_ns)) ? 1u : 0u;
    if (!ok) report(sp.status, STATUS_TIMEOUT_PEER_FLAG, site, src);
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

template <int KT, int TT, bool SP>
__global__ void __launch_bounds__(256)
dwconv_fwd_sw_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ halo,
                     const float* __restrict__ wt, __nv_bfloat16* __restrict__ out, int B, int T, int d,
                     int64_t x_ld, int64_t out_ld, const RowQuantOut qo, const ConvSp sp) {
  pdl_enter();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = (blockIdx.y * 32 + lane) * 8;
  int strip = blockIdx.x * 8 + warp;          // T % TT == 0: a strip never crosses a sequence boundary
  const int n_strips = B * (T / TT);
  if (strip >= n_strips) return;              // warp-uniform
  // sequence parallel: the strips that hold the rows the next rank waits for run first, the strips that wait
  // for the previous rank's rows run last
  if (SP) strip = n_strips - 1 - strip;
  const int row0 = strip * TT;
  const int b = row0 / T, t0 = row0 - b * T;
  const bool live = ch < d;
  if (!SP && !live) return;
  float tap[KT][8];
#pragma unroll
  for (int i = 0; i < KT; ++i) {
    const float4 w0 = live ? *reinterpret_cast<const float4*>(wt + (int64_t)i * d + ch) : make_float4(0, 0, 0, 0);
    const float4 w1 = live ? *reinterpret_cast<const float4*>(wt + (int64_t)i * d + ch + 4) : make_float4(0, 0, 0, 0);
    tap[i][0] = w0.x; tap[i][1] = w0.y; tap[i][2] = w0.z; tap[i][3] = w0.w;
    tap[i][4] = w1.x; tap[i][5] = w1.y; tap[i][6] = w1.z; tap[i][7] = w1.w;
  }
  uint4 in[TT + KT - 1];     // rows kept packed (bf16); unpacked at each use to stay within the register budget
#pragma unroll
  for (int j = 0; j < TT; ++j)
    in[KT - 1 + j] = live ? *reinterpret_cast<const uint4*>(x + (int64_t)(row0 + j) * x_ld + ch) : make_uint4(0, 0, 0, 0);
  if (SP && t0 + TT == T && sp.rank + 1 < sp.world) {
    // the last KT-1 rows of this sequence are the next rank's halo: straight from registers into its slot
    if (live) {
      uint4* dst = reinterpret_cast<uint4*>(sp.slots[sp.rank + 1] + sp.slot_offset);
#pragma unroll
      for (int i = 0; i < KT - 1; ++i)
        dst[((int64_t)b * (KT - 1) + i) * (d / 8) + ch / 8] = in[TT + i];
    }
    sp_signal_after_store(sp, sp.rank + 1, (uint32_t)B * gridDim.y);
  }
  bool halo_ok = true;
  if (SP && t0 == 0 && sp.rank > 0) halo_ok = sp_wait_neighbour(sp, sp.rank - 1, 41);
  if (!live) return;
#pragma unroll
  for (int i = 0; i < KT - 1; ++i) {
    const int t = t0 - (KT - 1) + i;
    in[i] = make_uint4(0, 0, 0, 0);
    if (t >= 0) {
      in[i] = *reinterpret_cast<const uint4*>(x + ((int64_t)b * T + t) * x_ld + ch);
    } else if (SP) {
      const int64_t at = ((int64_t)b * (KT - 1) + (t + KT - 1)) * (d / 8) + ch / 8;
      if (sp.rank > 0 && halo_ok)
        in[i] = __ldcv(reinterpret_cast<const uint4*>(sp.slots[sp.rank] + sp.slot_offset) + at);
      reinterpret_cast<uint4*>(sp.halo_out)[at] = in[i];
    } else if (halo != nullptr) {
      in[i] = *reinterpret_cast<const uint4*>(halo + ((int64_t)b * (KT - 1) + (t + KT - 1)) * d + ch);
    }
  }
#pragma unroll
  for (int j = 0; j < TT; ++j) {
    float acc[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = 0.0f;
#pragma unroll
    for (int i = 0; i < KT; ++i) {
      const uint32_t w[4] = {in[j + i].x, in[j + i].y, in[j + i].z, in[j + i].w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float2 f = unpack_bf16x2(w[c]);
        acc[2 * c] = fmaf(tap[i][2 * c], f.x, acc[2 * c]);
        acc[2 * c + 1] = fmaf(tap[i][2 * c + 1], f.y, acc[2 * c + 1]);
      }
    }
    store_bf16_vec<8>(out + (int64_t)(row0 + j) * out_ld + ch, acc);
    if (qo.q != nullptr) {
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = __bfloat162float(__float2bfloat16(acc[c]));
      quant_emit_8(qo, acc, row0 + j, ch, true);
    }
  }
}

// The forward conv as a walk on a persistent grid (no sequence parallelism): a warp owns 256 channels (8 per lane)
// and walks segments of `seg_rows` consecutive time steps of one sequence in strips of 8, the last KT-1 input rows
// of a strip staying in registers for the next. The rows of the next strip are on their way (per-thread
// asynchronous copies into a shared-memory slot of the thread's own) while the current strip is computed and
// quantised, so a warp always has 8 row loads in flight. Channel groups sit on blockIdx.x so that the blocks
// running at the same time cover whole rows of the same time steps.
constexpr int FWALK_SLOTS = 8 + 3;                // 8 strip rows, 3 window rows at a segment start (KT = 4)
constexpr int FWALK_SMEM = FWALK_SLOTS * 256 * 16;

template <int KT>
__global__ void __launch_bounds__(256, 2)
dwconv_fwd_walk_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ halo,
                       const float* __restrict__ wt, __nv_bfloat16* __restrict__ out, int B, int T, int d,
                       int64_t x_ld, int64_t out_ld, const RowQuantOut qo, int seg_rows) {
  pdl_enter();
  constexpr int TT = 8;
  static_assert(FWALK_SLOTS == TT + KT - 1, "slot layout");
  extern __shared__ __align__(16) uint8_t walk_smem[];
  uint4* buf = reinterpret_cast<uint4*>(walk_smem) + threadIdx.x;      // slot i of this thread: buf[i * 256]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = (blockIdx.x * 32 + lane) * 8;
  if (ch >= d) return;                    // with a quantised output d % 128 == 0: whole 16-lane groups leave
  const int n_segs = (int)((int64_t)B * T / seg_rows);
  const int strips_per_seg = seg_rows / TT;
  const int seg_step = gridDim.y * 8;
  float tap[KT][8];
#pragma unroll
  for (int i = 0; i < KT; ++i) {
    const float4 w0 = *reinterpret_cast<const float4*>(wt + (int64_t)i * d + ch);
    const float4 w1 = *reinterpret_cast<const float4*>(wt + (int64_t)i * d + ch + 4);
    tap[i][0] = w0.x; tap[i][1] = w0.y; tap[i][2] = w0.z; tap[i][3] = w0.w;
    tap[i][4] = w1.x; tap[i][5] = w1.y; tap[i][6] = w1.z; tap[i][7] = w1.w;
  }
  auto prefetch = [&](int seg, int sidx) {
    const int64_t row0 = (int64_t)seg * seg_rows;
    const int b = (int)(row0 / T), t0 = (int)(row0 - (int64_t)b * T), ts = t0 + sidx * TT;
    const __nv_bfloat16* x_b = x + (int64_t)b * T * x_ld + ch;
#pragma unroll
    for (int i = 0; i < TT; ++i) cp_async_16(buf + i * 256, x_b + (int64_t)(ts + i) * x_ld, true);
    if (sidx == 0) {
#pragma unroll
      for (int i = 0; i < KT - 1; ++i) {
        const int t = t0 - (KT - 1) + i;
        const __nv_bfloat16* src = x_b;
        bool valid = true;
        if (t >= 0) src = x_b + (int64_t)t * x_ld;
        else if (halo != nullptr) src = halo + ((int64_t)b * (KT - 1) + (t + KT - 1)) * d + ch;
        else valid = false;
        cp_async_16(buf + (TT + i) * 256, src, valid);
      }
    }
    cp_async_commit();
  };
  int seg = blockIdx.y * 8 + warp, sidx = 0;
  uint4 in[TT + KT - 1];     // in[i] = xpad[ts - (KT-1) + i], packed bf16
  if (seg < n_segs) prefetch(seg, 0);
  while (seg < n_segs) {
    const int64_t row0 = (int64_t)seg * seg_rows + sidx * TT;
    cp_async_wait_but<0>();
    if (sidx == 0) {
#pragma unroll
      for (int i = 0; i < KT - 1; ++i) in[i] = buf[(TT + i) * 256];
    } else {
#pragma unroll
      for (int i = 0; i < KT - 1; ++i) in[i] = in[TT + i];
    }
#pragma unroll
    for (int i = 0; i < TT; ++i) in[KT - 1 + i] = buf[i * 256];
    // the slot is free again (its rows are in registers): start the next strip's copies before computing this one
    int nseg = seg, nsidx = sidx + 1;
    if (nsidx == strips_per_seg) {
      nsidx = 0;
      nseg = seg + seg_step;
    }
    if (nseg < n_segs) prefetch(nseg, nsidx);
#pragma unroll
    for (int j = 0; j < TT; ++j) {
      float acc[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = 0.0f;
#pragma unroll
      for (int i = 0; i < KT; ++i) {
        const uint32_t w[4] = {in[j + i].x, in[j + i].y, in[j + i].z, in[j + i].w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float2 f = unpack_bf16x2(w[c]);
          acc[2 * c] = fmaf(tap[i][2 * c], f.x, acc[2 * c]);
          acc[2 * c + 1] = fmaf(tap[i][2 * c + 1], f.y, acc[2 * c + 1]);
        }
      }
      store_bf16_vec<8>(out + (row0 + j) * out_ld + ch, acc);
      if (qo.q != nullptr) {
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = __bfloat162float(__float2bfloat16(acc[c]));
        quant_emit_8(qo, acc, row0 + j, ch, true);
      }
    }
    seg = nseg;
    sidx = nsidx;
  }
}

// dx[t] = sum_j w[k-1-j] dc[t+j] for t in [t_lo, T), t_lo = -(k-1) when the halo gradient is wanted
template <int KT>
__global__ void __launch_bounds__(256)
dwconv_dx_pt_kernel(const __nv_bfloat16* __restrict__ dc, const float* __restrict__ wt,
                    const __nv_bfloat16* __restrict__ dx_tail_add, __nv_bfloat16* __restrict__ dx,
                    __nv_bfloat16* __restrict__ dhalo, int B, int T, int d, int k, int64_t dc_ld) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = (blockIdx.y * 32 + lane) * 8;
  if (KT > 0) k = KT;
  const int t_lo = dhalo != nullptr ? -(k - 1) : 0;
  const int rows_per_b = T - t_lo;
  const int r = blockIdx.x * 8 + warp;
  if (ch >= d || r >= B * rows_per_b) return;
  const int b = r / rows_per_b, t = r - b * rows_per_b + t_lo;
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = 0.0f;
#pragma unroll
  for (int j = 0; j < (KT > 0 ? KT : k); ++j) {
    const int tt = t + j;
    float g[8];
    if (tt >= 0 && tt < T) {
      load_bf16_vec<8>(dc + ((int64_t)b * T + tt) * dc_ld + ch, g);
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) g[c] = 0.0f;
    }
    const float4 w0 = *reinterpret_cast<const float4*>(wt + (int64_t)(k - 1 - j) * d + ch);
    const float4 w1 = *reinterpret_cast<const float4*>(wt + (int64_t)(k - 1 - j) * d + ch + 4);
    const float tap[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = fmaf(tap[c], g[c], acc[c]);
  }
  if (t >= 0) {
    if (dx_tail_add != nullptr && t >= T - (k - 1)) {
      float extra[8];
      load_bf16_vec<8>(dx_tail_add + ((int64_t)b * (k - 1) + (t - (T - (k - 1)))) * d + ch, extra);
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] += extra[c];
    }
    store_bf16_vec<8>(dx + ((int64_t)b * T + t) * d + ch, acc);
  } else {
    store_bf16_vec<8>(dhalo + ((int64_t)b * (k - 1) + (t + k - 1)) * d + ch, acc);
  }
}

// Sliding-window form of dx for t in [0, T): a thread owns 8 channels and TT consecutive time steps and loads
// the TT + KT - 1 rows of dc it needs once (rows past the end of the sequence are zero).
template <int KT, int TT, bool SP>
__global__ void __launch_bounds__(256)
dwconv_dx_sw_kernel(const __nv_bfloat16* __restrict__ dc, const float* __restrict__ wt,
                    const __nv_bfloat16* __restrict__ dx_tail_add, __nv_bfloat16* __restrict__ dx, int B, int T, int d,
                    int64_t dc_ld, const ConvSp sp) {
  pdl_enter();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = (blockIdx.y * 32 + lane) * 8;
  const int strip = blockIdx.x * 8 + warp;
  const int row0 = strip * TT;
  if (row0 >= B * T) return;                  // warp-uniform
  const bool live = ch < d;
  if (!SP && !live) return;
  const int b = row0 / T, t0 = row0 - b * T;
  float tap[KT][8];      // tap[j] multiplies dc[t + j]: w[KT-1-j]
#pragma unroll
  for (int j = 0; j < KT; ++j) {
    const float4 w0 = live ? *reinterpret_cast<const float4*>(wt + (int64_t)(KT - 1 - j) * d + ch) : make_float4(0, 0, 0, 0);
    const float4 w1 = live ? *reinterpret_cast<const float4*>(wt + (int64_t)(KT - 1 - j) * d + ch + 4) : make_float4(0, 0, 0, 0);
    tap[j][0] = w0.x; tap[j][1] = w0.y; tap[j][2] = w0.z; tap[j][3] = w0.w;
    tap[j][4] = w1.x; tap[j][5] = w1.y; tap[j][6] = w1.z; tap[j][7] = w1.w;
  }
  uint4 g[TT + KT - 1];
#pragma unroll
  for (int i = 0; i < TT + KT - 1; ++i) {
    g[i] = make_uint4(0, 0, 0, 0);
    if (live && t0 + i < T) g[i] = *reinterpret_cast<const uint4*>(dc + (int64_t)(row0 + i) * dc_ld + ch);
  }
  if (SP && t0 == 0 && sp.rank > 0) {
    // gradient of the halo rows t = -(KT-1) .. -1 (they are the previous rank's last rows): into its slot
    if (live) {
      uint4* dst = reinterpret_cast<uint4*>(sp.slots[sp.rank - 1] + sp.slot_offset);
#pragma unroll
      for (int r = 0; r < KT - 1; ++r) {        // row t = r - (KT-1): dc[t + j] exists for j >= KT-1-r
        float acc[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = 0.0f;
#pragma unroll
        for (int j = KT - 1 - r; j < KT; ++j) {
          const uint4 gv = g[r - (KT - 1) + j];
          const uint32_t w[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float2 f = unpack_bf16x2(w[c]);
            acc[2 * c] = fmaf(tap[j][2 * c], f.x, acc[2 * c]);
            acc[2 * c + 1] = fmaf(tap[j][2 * c + 1], f.y, acc[2 * c + 1]);
          }
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        dst[((int64_t)b * (KT - 1) + r) * (d / 8) + ch / 8] = o;
      }
    }
    sp_signal_after_store(sp, sp.rank - 1, (uint32_t)B * gridDim.y);
  }
  bool tail_ok = true;
  const bool has_tail = SP && t0 + TT == T && sp.rank + 1 < sp.world;
  if (has_tail) tail_ok = sp_wait_neighbour(sp, sp.rank + 1, 42);
  if (!live) return;
#pragma unroll
  for (int i = 0; i < TT; ++i) {
    float acc[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = 0.0f;
#pragma unroll
    for (int j = 0; j < KT; ++j) {
      const uint32_t w[4] = {g[i + j].x, g[i + j].y, g[i + j].z, g[i + j].w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float2 f = unpack_bf16x2(w[c]);
        acc[2 * c] = fmaf(tap[j][2 * c], f.x, acc[2 * c]);
        acc[2 * c + 1] = fmaf(tap[j][2 * c + 1], f.y, acc[2 * c + 1]);
      }
    }
    const int t = t0 + i;
    if (has_tail && tail_ok && t >= T - (KT - 1)) {
      // the next rank's halo gradient belongs to these rows: add it before they are stored
      const uint4 e = __ldcv(reinterpret_cast<const uint4*>(sp.slots[sp.rank] + sp.slot_offset) +
                             ((int64_t)b * (KT - 1) + (t - (T - (KT - 1)))) * (d / 8) + ch / 8);
      const uint32_t w[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float2 f = unpack_bf16x2(w[c]);
        acc[2 * c] += f.x;
        acc[2 * c + 1] += f.y;
      }
    }
    if (!SP && dx_tail_add != nullptr && t >= T - (KT - 1)) {
      float extra[8];
      load_bf16_vec<8>(dx_tail_add + ((int64_t)b * (KT - 1) + (t - (T - (KT - 1)))) * d + ch, extra);
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] += extra[c];
    }
    store_bf16_vec<8>(dx + (int64_t)(row0 + i) * d + ch, acc);
  }
}

// The k-1 halo-gradient rows of every sequence (t in [-(k-1), 0)), for the sequence-parallel exchange.
__global__ void __launch_bounds__(256)
dwconv_dhalo_kernel(const __nv_bfloat16* __restrict__ dc, const float* __restrict__ wt, __nv_bfloat16* __restrict__ dhalo,
                    int B, int T, int d, int k, int64_t dc_ld) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = (blockIdx.y * 32 + lane) * 8;
  const int r = blockIdx.x * 8 + warp;
  if (ch >= d || r >= B * (k - 1)) return;
  const int b = r / (k - 1), t = r - b * (k - 1) - (k - 1);   // t in [-(k-1), 0)
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = 0.0f;
  for (int j = 0; j < k; ++j) {
    const int tt = t + j;
    if (tt < 0 || tt >= T) continue;
    float g[8];
    load_bf16_vec<8>(dc + ((int64_t)b * T + tt) * dc_ld + ch, g);
    const float4 w0 = *reinterpret_cast<const float4*>(wt + (int64_t)(k - 1 - j) * d + ch);
    const float4 w1 = *reinterpret_cast<const float4*>(wt + (int64_t)(k - 1 - j) * d + ch + 4);
    const float tap[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = fmaf(tap[c], g[c], acc[c]);
  }
  store_bf16_vec<8>(dhalo + ((int64_t)b * (k - 1) + (t + k - 1)) * d + ch, acc);
}

// dw[ch][i] += sum_{b,t} dc[b,t,ch] * xpad[b, t-(k-1)+i, ch]: a lane owns 4 channels and walks a strip of
// DW_TT time steps with a sliding window of x; the 8 warps of a block (8 strips) are reduced in shared
// memory before one atomic per (channel, tap).
constexpr int DW_TT = 32;

template <int KMAX>
__global__ void __launch_bounds__(256)
dwconv_dw_kernel(const __nv_bfloat16* __restrict__ dc, const __nv_bfloat16* __restrict__ x,
                 const __nv_bfloat16* __restrict__ halo, float* __restrict__ dw, int B, int T, int d, int k,
                 int64_t dc_ld, int64_t x_ld) {
  pdl_enter();
  constexpr bool BLOCK_REDUCE = KMAX <= 8;     // the widest window would not fit the static shared-memory limit
  __shared__ float part[BLOCK_REDUCE ? 8 : 1][BLOCK_REDUCE ? KMAX : 1][128 + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = (blockIdx.y * 32 + lane) * 4;
  const int strips_per_b = (T + DW_TT - 1) / DW_TT;
  const int strip = blockIdx.x * 8 + warp;
  const int b = strip / strips_per_b;
  const int t0 = (strip % strips_per_b) * DW_TT;
  float acc[KMAX][4];
#pragma unroll
  for (int i = 0; i < KMAX; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] = 0.0f;
  if (ch < d && b < B) {
    float xw[KMAX][4];     // xw[i] = xpad[t - (KMAX-1) + i]
#pragma unroll
    for (int i = 0; i < KMAX - 1; ++i) load_conv_row<4>(x, halo, x_ld, T, k, b, t0 - (KMAX - 1) + i, ch, d, xw[i + 1]);
    const int t_end = min(t0 + DW_TT, T);
#pragma unroll 4
    for (int t = t0; t < t_end; ++t) {
#pragma unroll
      for (int i = 0; i < KMAX - 1; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) xw[i][c] = xw[i + 1][c];
      load_bf16_vec<4>(x + ((int64_t)b * T + t) * x_ld + ch, xw[KMAX - 1]);
      float g[4];
      load_bf16_vec<4>(dc + ((int64_t)b * T + t) * dc_ld + ch, g);
#pragma unroll
      for (int i = 0; i < KMAX; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][c] = fmaf(g[c], xw[i][c], acc[i][c]);
    }
  }
  if constexpr (!BLOCK_REDUCE) {
#pragma unroll
    for (int i = 0; i < KMAX; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int src = i - (KMAX - k);
        if (src >= 0 && ch + c < d && acc[i][c] != 0.0f) atomicAdd(dw + (int64_t)(ch + c) * k + src, acc[i][c]);
      }
    return;
  }
#pragma unroll
  for (int i = 0; i < KMAX; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) part[BLOCK_REDUCE ? warp : 0][BLOCK_REDUCE ? i : 0][lane * 4 + c] = acc[i][c];
  __syncthreads();
  for (int idx = threadIdx.x; idx < KMAX * 128; idx += blockDim.x) {
    const int i = idx / 128, cc = idx % 128;
    const int src = i - (KMAX - k);          // window slot i holds tap src (front-padded to KMAX)
    const int chan = blockIdx.y * 128 + cc;
    if (src < 0 || chan >= d) continue;
    float sum = 0.0f;
#pragma unroll
    for (int wq = 0; wq < 8; ++wq) sum += part[BLOCK_REDUCE ? wq : 0][BLOCK_REDUCE ? i : 0][cc];
    if (sum != 0.0f) atomicAdd(dw + (int64_t)chan * k + src, sum);
  }
}

// dx and dw in one walk over the rows. A warp owns 128 channels (4 per lane) and walks segments of `seg_rows`
// consecutive time steps of one sequence in strips of 8: the last KT-1 rows of dc and of x of a strip stay in
// registers for the next one, so within a segment every row of dc and of x is loaded exactly once (plus KT-1 rows
// at its start) and dx is written once. The rows of the next strip are on their way (per-thread asynchronous
// copies into a shared-memory slot of the thread's own) while the current strip is computed, so a warp always has
// 16 row loads in flight. The grid is persistent (about two blocks per SM): a warp takes every (gridDim.y * 8)-th
// segment and sums the tap gradients in registers over all of them; the 8 warps of a block combine in shared
// memory and leave one atomic per (channel, tap) and block. Channel groups sit on blockIdx.x so that the blocks
// running at the same time cover whole rows of the same time steps.
constexpr int WALK_SLOTS = 2 * 8 + 2 * 3;      // 8 + 8 strip rows, 3 + 3 window rows at a segment start (KT = 4)
constexpr int WALK_DEPTH = 1;                   // strips on their way per warp (2 measured slower: 59.8 against 53.1 us)
constexpr int WALK_COPY_BYTES = WALK_DEPTH * WALK_SLOTS * 256 * 8;
constexpr int WALK_SMEM = WALK_COPY_BYTES + 8 * 4 * (128 + 1) * 4;      // + the block's partial tap sums

template <int KT>
__global__ void __launch_bounds__(256, 2)
dwconv_bwd_walk_kernel(const __nv_bfloat16* __restrict__ dc, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ halo, const float* __restrict__ wt,
                       const __nv_bfloat16* __restrict__ dx_tail_add, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ dw, int B, int T, int d, int64_t dc_ld, int64_t x_ld, int seg_rows) {
  pdl_enter();
  constexpr int TT = 8, W = TT + KT - 1;
  static_assert(WALK_SLOTS == 2 * TT + 2 * (KT - 1), "slot layout");
  extern __shared__ __align__(16) uint8_t walk_smem[];
  uint2* buf0 = reinterpret_cast<uint2*>(walk_smem) + threadIdx.x;     // slot i of this thread in buffer n: buf0[(n * WALK_SLOTS + i) * 256]
  float (*part)[KT][128 + 1] = reinterpret_cast<float (*)[KT][128 + 1]>(walk_smem + WALK_COPY_BYTES);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cgroup = blockIdx.x;
  const int ch = (cgroup * 32 + lane) * 4;
  const int n_segs = (int)((int64_t)B * T / seg_rows);
  const int strips_per_seg = seg_rows / TT;
  const int seg_step = gridDim.y * 8;
  float acc[KT][4];
#pragma unroll
  for (int m = 0; m < KT; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[m][c] = 0.0f;
  if (ch < d) {
    float tap[KT][4];      // tap[j] multiplies dc[t + j]: w[KT-1-j]
#pragma unroll
    for (int j = 0; j < KT; ++j) {
      const float4 w4 = *reinterpret_cast<const float4*>(wt + (int64_t)(KT - 1 - j) * d + ch);
      tap[j][0] = w4.x; tap[j][1] = w4.y; tap[j][2] = w4.z; tap[j][3] = w4.w;
    }
    // the rows of strip `sidx` of segment `seg`: dc[ts + KT-1 .. +TT), x[ts .. ts + TT), and at a segment start also
    // dc[t0 .. t0 + KT-1) and xpad[t0 - (KT-1) .. t0)
    auto prefetch = [&](int seg, int sidx, uint2* buf) {
      const int64_t row0 = (int64_t)seg * seg_rows;
      const int b = (int)(row0 / T), t0 = (int)(row0 - (int64_t)b * T), ts = t0 + sidx * TT;
      const __nv_bfloat16* dc_b = dc + (int64_t)b * T * dc_ld + ch;
      const __nv_bfloat16* x_b = x + (int64_t)b * T * x_ld + ch;
#pragma unroll
      for (int i = 0; i < TT; ++i) {
        const int tg = ts + KT - 1 + i;
        cp_async_8(buf + i * 256, dc_b + (int64_t)(tg < T ? tg : 0) * dc_ld, tg < T);
        cp_async_8(buf + (TT + i) * 256, x_b + (int64_t)(ts + i) * x_ld, true);
      }
      if (sidx == 0) {
#pragma unroll
        for (int i = 0; i < KT - 1; ++i) {
          cp_async_8(buf + (2 * TT + i) * 256, dc_b + (int64_t)(t0 + i) * dc_ld, true);     // seg_rows >= TT > KT-1
          const int t = t0 - (KT - 1) + i;
          const __nv_bfloat16* src = x_b;
          bool valid = true;
          if (t >= 0) src = x_b + (int64_t)t * x_ld;
          else if (halo != nullptr) src = halo + ((int64_t)b * (KT - 1) + (t + KT - 1)) * d + ch;
          else valid = false;
          cp_async_8(buf + (2 * TT + KT - 1 + i) * 256, src, valid);
        }
      }
      cp_async_commit();
    };
    auto advance = [&](int& seg, int& sidx) {
      if (++sidx == strips_per_seg) {
        sidx = 0;
        seg += seg_step;
      }
    };
    int seg = blockIdx.y * 8 + warp, sidx = 0;
    uint2 g[W], xq[W];     // within a strip at ts: g[i] = dc[ts + i], xq[i] = xpad[ts - (KT-1) + i]
    // WALK_DEPTH strips ahead: pseg/psidx is the next strip to ask for, `cur` the buffer of the strip to compute
    int pseg = seg, psidx = 0, cur = 0;
#pragma unroll
    for (int i = 0; i < WALK_DEPTH; ++i) {
      if (pseg < n_segs) prefetch(pseg, psidx, buf0 + i * WALK_SLOTS * 256);
      else cp_async_commit();                       // keeps the group count uniform
      advance(pseg, psidx);
    }
    while (seg < n_segs) {
      const int64_t row0 = (int64_t)seg * seg_rows;
      const int b = (int)(row0 / T), ts = (int)(row0 - (int64_t)b * T) + sidx * TT;
      uint2* buf = buf0 + cur * WALK_SLOTS * 256;
      cp_async_wait_but<WALK_DEPTH - 1>();
      if (sidx == 0) {
#pragma unroll
        for (int i = 0; i < KT - 1; ++i) {
          g[i] = buf[(2 * TT + i) * 256];
          xq[i] = buf[(2 * TT + KT - 1 + i) * 256];
        }
      } else {
#pragma unroll
        for (int i = 0; i < KT - 1; ++i) {
          g[i] = g[TT + i];
          xq[i] = xq[TT + i];
        }
      }
#pragma unroll
      for (int i = 0; i < TT; ++i) {
        g[KT - 1 + i] = buf[i * 256];
        xq[KT - 1 + i] = buf[(TT + i) * 256];
      }
      // the buffer is free again (its rows are in registers): ask for the strip after the next one before computing
      if (pseg < n_segs) prefetch(pseg, psidx, buf);
      else cp_async_commit();
      advance(pseg, psidx);
      cur = (cur + 1) % WALK_DEPTH;
#pragma unroll
      for (int i = 0; i < TT; ++i) {
        float o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int j = 0; j < KT; ++j) {
          const float2 lo = unpack_bf16x2(g[i + j].x), hi = unpack_bf16x2(g[i + j].y);
          o[0] = fmaf(tap[j][0], lo.x, o[0]);
          o[1] = fmaf(tap[j][1], lo.y, o[1]);
          o[2] = fmaf(tap[j][2], hi.x, o[2]);
          o[3] = fmaf(tap[j][3], hi.y, o[3]);
        }
        const float2 glo = unpack_bf16x2(g[i].x), ghi = unpack_bf16x2(g[i].y);
#pragma unroll
        for (int m = 0; m < KT; ++m) {
          const float2 lo = unpack_bf16x2(xq[i + m].x), hi = unpack_bf16x2(xq[i + m].y);
          acc[m][0] = fmaf(glo.x, lo.x, acc[m][0]);
          acc[m][1] = fmaf(glo.y, lo.y, acc[m][1]);
          acc[m][2] = fmaf(ghi.x, hi.x, acc[m][2]);
          acc[m][3] = fmaf(ghi.y, hi.y, acc[m][3]);
        }
        const int t = ts + i;
        if (dx_tail_add != nullptr && t >= T - (KT - 1)) {
          float extra[4];
          load_bf16_vec<4>(dx_tail_add + ((int64_t)b * (KT - 1) + (t - (T - (KT - 1)))) * d + ch, extra);
#pragma unroll
          for (int c = 0; c < 4; ++c) o[c] += extra[c];
        }
        *reinterpret_cast<uint2*>(dx + ((int64_t)b * T + t) * d + ch) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
      }
      advance(seg, sidx);
    }
  }
#pragma unroll
  for (int m = 0; m < KT; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) part[warp][m][lane * 4 + c] = acc[m][c];
  __syncthreads();
  for (int idx = threadIdx.x; idx < KT * 128; idx += blockDim.x) {
    const int m = idx >> 7, cc = idx & 127;
    const int chan = cgroup * 128 + cc;
    if (chan >= d) continue;
    float sum = 0.0f;
#pragma unroll
    for (int wq = 0; wq < 8; ++wq) sum += part[wq][m][cc];
    if (sum != 0.0f) atomicAdd(dw + (int64_t)chan * KT + m, sum);
  }
}

template <int KMAX>
static const char* conv_dw_launch(const ConvBwdArgs& a, cudaStream_t st) {
  const int strips = a.B * ((a.T + DW_TT - 1) / DW_TT);
  dim3 grid((strips + 7) / 8, (a.d + 127) / 128);
  launch_pdl(dwconv_dw_kernel<KMAX>, grid, dim3(256), 0, st, a.dc, a.x, a.halo, a.dw, a.B, a.T, a.d, a.k, a.dc_ld, a.x_ld);
  return cudaGetLastError() == cudaSuccess ? nullptr : "dwconv_dw launch failed";
}

// Segment length and grid of a walk kernel: `ch_per_block` channels per block, about two blocks per SM; the segment
// length trades the KT-1 rows re-read at every segment start against an even spread of the segments over the warps.
static void walk_plan(int64_t rows, int T, int d, int ch_per_block, int& seg, dim3& grid) {
  const int cgroups = (d + ch_per_block - 1) / ch_per_block;
  const int walkers_max = std::max(1, 148 * 2 / cgroups) * 8;          // warps per channel group
  seg = 8;
  double best = 0.0;
  for (int cand : {64, 32, 16, 8}) {
    if (T % cand != 0) continue;
    const int64_t n = rows / cand;
    const int64_t walkers = std::min<int64_t>(walkers_max, (n + 7) / 8 * 8);
    const double balance = (double)n / (double)((n + walkers - 1) / walkers * walkers);
    const double score = balance * cand / (cand + 3.0);
    if (score > best) { best = score; seg = cand; }
  }
  const int64_t n_segs = rows / seg;
  grid = dim3(cgroups, (unsigned)std::min<int64_t>(walkers_max / 8, (n_segs + 7) / 8));
}

const char* launch_dwconv_fwd(const ConvArgs& a, cudaStream_t st) {
  if (a.k < 1 || a.k > 16) return "dwconv: kernel width must be in [1, 16]";
  if (a.d % 8 != 0) return "dwconv: d must be a multiple of 8";
  if ((int64_t)a.B * (a.T + 16) >= (1ll << 31)) return "dwconv: B*T must be below 2^31";
  dim3 grid((unsigned)(((int64_t)a.B * a.T + 7) / 8), (a.d + 255) / 256);
  if (a.quant.q != nullptr && a.d % 128 != 0) return "dwconv: a quantised output needs d % 128 == 0";
  if (a.sp.slots != nullptr && !(a.k == 4 && a.T % 8 == 0)) return "dwconv: the in-kernel halo exchange needs k == 4 and T % 8 == 0";
  if (a.k == 4 && a.T % 8 == 0) {
    dim3 sgrid((unsigned)(((int64_t)a.B * a.T / 8 + 7) / 8), (a.d + 255) / 256);
    static const bool walk_off = getenv("GDNET_CONV_WALK") != nullptr && atoi(getenv("GDNET_CONV_WALK")) == 0;
    if (a.sp.slots != nullptr) {
      dwconv_fwd_sw_kernel<4, 8, true><<<sgrid, 256, 0, st>>>(a.x, a.halo, a.w, a.out, a.B, a.T, a.d, a.x_ld, a.out_ld, a.quant, a.sp);
    } else if (!walk_off && a.x_ld % 8 == 0 && a.out_ld % 8 == 0) {
      int seg;
      dim3 wgrid;
      walk_plan((int64_t)a.B * a.T, a.T, a.d, 256, seg, wgrid);
      static bool attr = false;
      if (!attr) {
        cudaFuncSetAttribute(dwconv_fwd_walk_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, FWALK_SMEM);
        attr = true;
      }
      launch_pdl(dwconv_fwd_walk_kernel<4>, wgrid, dim3(256), FWALK_SMEM, st, a.x, a.halo, a.w, a.out, a.B, a.T, a.d, a.x_ld,
                 a.out_ld, a.quant, seg);
    } else {
      launch_pdl(dwconv_fwd_sw_kernel<4, 8, false>, sgrid, dim3(256), 0, st, a.x, a.halo, a.w, a.out, a.B, a.T, a.d, a.x_ld, a.out_ld, a.quant, a.sp);
    }
    return cudaGetLastError() == cudaSuccess ? nullptr : "dwconv_fwd launch failed";
  }
  if (a.k == 4) dwconv_fwd_pt_kernel<4><<<grid, 256, 0, st>>>(a.x, a.halo, a.w, a.out, a.B, a.T, a.d, a.k, a.x_ld, a.out_ld, a.quant);
  else dwconv_fwd_pt_kernel<0><<<grid, 256, 0, st>>>(a.x, a.halo, a.w, a.out, a.B, a.T, a.d, a.k, a.x_ld, a.out_ld, a.quant);
  return cudaGetLastError() == cudaSuccess ? nullptr : "dwconv_fwd launch failed";
}

const char* launch_dwconv_bwd(const ConvBwdArgs& a, cudaStream_t st) {
  if (a.k < 1 || a.k > 16) return "dwconv: kernel width must be in [1, 16]";
  if (a.d % 8 != 0) return "dwconv: d must be a multiple of 8";
  if ((int64_t)a.B * (a.T + 16) >= (1ll << 31)) return "dwconv: B*T must be below 2^31";
  const int rows_per_b = a.T + (a.dhalo != nullptr ? a.k - 1 : 0);
  dim3 grid((unsigned)(((int64_t)a.B * rows_per_b + 7) / 8), (a.d + 255) / 256);
  if (a.sp.slots != nullptr && !(a.k == 4 && a.T % 8 == 0)) return "dwconv: the in-kernel halo exchange needs k == 4 and T % 8 == 0";
  static const bool walk_off = getenv("GDNET_CONV_WALK") != nullptr && atoi(getenv("GDNET_CONV_WALK")) == 0;
  if (!walk_off && a.k == 4 && a.T % 8 == 0 && a.sp.slots == nullptr && a.x != nullptr && a.dw != nullptr && a.dx != nullptr &&
      a.dc_ld % 4 == 0 && a.x_ld % 4 == 0) {
    // one walk for dx and dw on a persistent grid
    int seg;
    dim3 wgrid;
    walk_plan((int64_t)a.B * a.T, a.T, a.d, 128, seg, wgrid);
    static bool attr = false;
    if (!attr) {
      cudaFuncSetAttribute(dwconv_bwd_walk_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, WALK_SMEM);
      attr = true;
    }
    launch_pdl(dwconv_bwd_walk_kernel<4>, wgrid, dim3(256), WALK_SMEM, st, a.dc, a.x, a.halo, a.w, a.dx_tail_add, a.dx, a.dw, a.B, a.T,
               a.d, a.dc_ld, a.x_ld, seg);
    if (a.dhalo != nullptr) {
      dim3 hgrid((unsigned)((a.B * (a.k - 1) + 7) / 8), (a.d + 255) / 256);
      dwconv_dhalo_kernel<<<hgrid, 256, 0, st>>>(a.dc, a.w, a.dhalo, a.B, a.T, a.d, a.k, a.dc_ld);
    }
    return cudaGetLastError() == cudaSuccess ? nullptr : "dwconv_bwd launch failed";
  }
  if (a.k == 4 && a.T % 8 == 0) {
    dim3 sgrid((unsigned)(((int64_t)a.B * a.T / 8 + 7) / 8), (a.d + 255) / 256);
    if (a.sp.slots != nullptr)
      dwconv_dx_sw_kernel<4, 8, true><<<sgrid, 256, 0, st>>>(a.dc, a.w, a.dx_tail_add, a.dx, a.B, a.T, a.d, a.dc_ld, a.sp);
    else
      launch_pdl(dwconv_dx_sw_kernel<4, 8, false>, sgrid, dim3(256), 0, st, a.dc, a.w, a.dx_tail_add, a.dx, a.B, a.T, a.d, a.dc_ld, a.sp);
    if (a.dhalo != nullptr) {
      dim3 hgrid((unsigned)((a.B * (a.k - 1) + 7) / 8), (a.d + 255) / 256);
      dwconv_dhalo_kernel<<<hgrid, 256, 0, st>>>(a.dc, a.w, a.dhalo, a.B, a.T, a.d, a.k, a.dc_ld);
    }
    if (cudaGetLastError() != cudaSuccess) return "dwconv_dx launch failed";
    return conv_dw_launch<4>(a, st);
  }
  if (a.k == 4) dwconv_dx_pt_kernel<4><<<grid, 256, 0, st>>>(a.dc, a.w, a.dx_tail_add, a.dx, a.dhalo, a.B, a.T, a.d, a.k, a.dc_ld);
  else dwconv_dx_pt_kernel<0><<<grid, 256, 0, st>>>(a.dc, a.w, a.dx_tail_add, a.dx, a.dhalo, a.B, a.T, a.d, a.k, a.dc_ld);
  if (cudaGetLastError() != cudaSuccess) return "dwconv_dx launch failed";
  if (a.k <= 4) return conv_dw_launch<4>(a, st);
  if (a.k <= 8) return conv_dw_launch<8>(a, st);
  return conv_dw_launch<16>(a, st);
}

// =======================================================================================
// gate / stream update: one warp per row, 8 columns per lane per step
// =======================================================================================
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&o)[8]) { load_bf16_vec<8>(p, o); }
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&v)[8]) { store_bf16_vec<8>(p, v); }

// ---------------------------------------------------------------------------------------
// stream update with both gates given (public kernel API): one warp per row
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gate_mix_fwd_kernel(const GateMixArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  for (int64_t row = (int64_t)blockIdx.x * wpb + warp; row < a.rows; row += (int64_t)gridDim.x * wpb) {
    for (int col = lane * 8; col < a.d; col += 256) {
      float gp[8], cv[8], sv[8], rv[8], fo[8], so[8];
      ld8(a.g_pre + row * a.d + col, gp);
      ld8(a.c + row * a.c_ld + col, cv);
      ld8(a.s + row * a.s_ld + col, sv);
      ld8(a.R + row * a.r_ld + col, rv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float g = sigmoidf_(gp[i]);
        fo[i] = cv[i] * g + sv[i] * rv[i];
        so[i] = cv[i] * (1.0f - g) + sv[i] * (1.0f - rv[i]);
      }
      st8(a.fwd_out + row * a.d + col, fo);
      st8(a.side_out + row * a.d + col, so);
    }
  }
}

__global__ void __launch_bounds__(256)
gate_mix_bwd_kernel(const GateMixArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  for (int64_t row = (int64_t)blockIdx.x * wpb + warp; row < a.rows; row += (int64_t)gridDim.x * wpb) {
    float r = 1.0f;
    if (a.ssq != nullptr) {
      float t = 0.0f;
      for (int p = lane; p < a.ssq_parts; p += 32) t += a.ssq[row * a.ssq_parts + p];
      t = warp_sum(t);
      r = rsqrtf(t / (float)a.d + a.eps);
    }
    float rowsum = 0.0f;
    for (int col = lane * 8; col < a.d; col += 256) {
      float gp[8], cv[8], sv[8], rv[8], df[8], dsv[8], dgp[8], dq[8], dc[8], ds[8], dR[8];
      ld8(a.g_pre + row * a.d + col, gp);
      ld8(a.c + row * a.c_ld + col, cv);
      ld8(a.s + row * a.s_ld + col, sv);
      ld8(a.R + row * a.r_ld + col, rv);
      ld8(a.dF + row * a.d + col, df);
      ld8(a.dS + row * a.d + col, dsv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float g = sigmoidf_(gp[i]);
        const float diff = df[i] - dsv[i];
        dgp[i] = diff * cv[i] * g * (1.0f - g);
        dc[i] = df[i] * g + dsv[i] * (1.0f - g);
        ds[i] = df[i] * rv[i] + dsv[i] * (1.0f - rv[i]);
        dR[i] = diff * sv[i];
        dq[i] = dgp[i] * r;
        const float b = a.b2 != nullptr ? a.b2[col + i] : 0.0f;
        rowsum = fmaf(dgp[i], gp[i] - b, rowsum);
      }
      st8(a.dgp + row * a.d + col, dgp);
      if (a.dq != nullptr) st8(a.dq + row * a.d + col, dq);
      st8(a.dc + row * a.d + col, dc);
      st8(a.ds + row * a.d + col, ds);
      st8(a.dR + row * a.d + col, dR);
    }
    if (a.rowcoef != nullptr) {
      rowsum = warp_sum(rowsum);
      if (lane == 0) a.rowcoef[row] = r * r / (float)a.d * rowsum;
    }
  }
}

// The forward for contiguous inputs: one 8-element vector per thread, as many blocks as vectors / 256, streaming
// stores. For this purely element-wise op the plain form measured faster than a persistent grid with asynchronous
// prefetch (234 against 251 us at 65536 x 2048, 62 against 66 us at 32768 x 1024).
__global__ void __launch_bounds__(256)
gate_mix_fwd_onevec_kernel(const GateMixArgs a) {
  const int64_t n_vec = a.rows * (int64_t)(a.d / 8);
  const int64_t v = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (v >= n_vec) return;
  const uint4 qg = __ldg(reinterpret_cast<const uint4*>(a.g_pre + v * 8)), qc = __ldg(reinterpret_cast<const uint4*>(a.c + v * 8));
  const uint4 qs = __ldg(reinterpret_cast<const uint4*>(a.s + v * 8)), qr = __ldg(reinterpret_cast<const uint4*>(a.R + v * 8));
  const uint32_t* gw = reinterpret_cast<const uint32_t*>(&qg);
  const uint32_t* cw = reinterpret_cast<const uint32_t*>(&qc);
  const uint32_t* sw = reinterpret_cast<const uint32_t*>(&qs);
  const uint32_t* rw = reinterpret_cast<const uint32_t*>(&qr);
  uint4 of, os;
  uint32_t* fw = reinterpret_cast<uint32_t*>(&of);
  uint32_t* ow = reinterpret_cast<uint32_t*>(&os);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 gp = unpack_bf16x2(gw[t]), cv = unpack_bf16x2(cw[t]), sv = unpack_bf16x2(sw[t]), rv = unpack_bf16x2(rw[t]);
    const float g0 = sigmoidf_(gp.x), g1 = sigmoidf_(gp.y);
    fw[t] = pack_bf16x2(cv.x * g0 + sv.x * rv.x, cv.y * g1 + sv.y * rv.y);
    ow[t] = pack_bf16x2(cv.x * (1.0f - g0) + sv.x * (1.0f - rv.x), cv.y * (1.0f - g1) + sv.y * (1.0f - rv.y));
  }
  __stcs(reinterpret_cast<uint4*>(a.fwd_out + v * 8), of);
  __stcs(reinterpret_cast<uint4*>(a.side_out + v * 8), os);
}

static int gate_mix_blocks(int64_t rows) {
  int64_t b = (rows + 7) / 8;
  return (int)(b < 148 * 8 ? (b < 1 ? 1 : b) : 148 * 8);
}

const char* launch_gate_mix_fwd(const GateMixArgs& a, cudaStream_t st) {
  if (a.d % 8 != 0) return "gate_mix: d must be a multiple of 8";
  if (a.rows == 0) return nullptr;
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(a.g_pre) | reinterpret_cast<uintptr_t>(a.c) | reinterpret_cast<uintptr_t>(a.s) |
                         reinterpret_cast<uintptr_t>(a.R) | reinterpret_cast<uintptr_t>(a.fwd_out) | reinterpret_cast<uintptr_t>(a.side_out);
  if (a.c_ld == a.d && a.s_ld == a.d && a.r_ld == a.d && ptrs % 16 == 0) {
    const int64_t blocks = (a.rows * (int64_t)(a.d / 8) + 255) / 256;
    if (blocks < (1ll << 31)) {
      gate_mix_fwd_onevec_kernel<<<(unsigned)blocks, 256, 0, st>>>(a);
      return cudaGetLastError() == cudaSuccess ? nullptr : "gate_mix_fwd launch failed";
    }
  }
  gate_mix_fwd_kernel<<<gate_mix_blocks(a.rows), 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "gate_mix_fwd launch failed";
}

const char* launch_gate_mix_bwd(const GateMixArgs& a, cudaStream_t st) {
  if (a.d % 8 != 0) return "gate_mix: d must be a multiple of 8";
  if (a.rows == 0) return nullptr;
  gate_mix_bwd_kernel<<<gate_mix_blocks(a.rows), 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "gate_mix_bwd launch failed";
}

// fwd' = c*g + s*R, side' = c*(1-g) + s*(1-R) with g = sigmoid(g_pre),
// R = sigmoid(z * rstd(z) * w_r). Also writes rstd(z) per row, optionally g, and adds the
// sum of g over the block's rows to gate_sum (for the mean forward-gate value).
__global__ void __launch_bounds__(256)
gate_update_fwd_kernel(const GateFwdArgs a) {
  pdl_enter();
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
      if (a.quant.q != nullptr) {   // the next step's recovery GEMM reads the side stream in FP8
#pragma unroll
        for (int i = 0; i < 8; ++i) so[i] = __bfloat162float(__float2bfloat16(so[i]));
        quant_emit_8(a.quant, so, row, col, true);
      }
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

// Barrier number 1 + slot (slot 0..3) for `threads` threads, with the number as an immediate: a number from a register
// makes the block claim all 16 hardware barriers and lets only one block live on an SM.
template <int THREADS>
__device__ __forceinline__ void row_group_barrier(int slot) {
  if (slot == 0) asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
  else if (slot == 1) asm volatile("bar.sync 2, %0;" ::"n"(THREADS) : "memory");
  else if (slot == 2) asm volatile("bar.sync 3, %0;" ::"n"(THREADS) : "memory");
  else asm volatile("bar.sync 4, %0;" ::"n"(THREADS) : "memory");
}

// The same for d == NW * 256 (NW = 1, 2, 4, 8) with every input read once: NW warps share a row, each lane owning 8
// of its columns, the 8 warps of a block work on 8 / NW rows at a time on a persistent grid, the warps of a row
// exchange their partial sums of squares through shared memory, and the next rows' inputs are on their way
// (per-thread asynchronous copies) while the current ones are computed.
template <int NW>
__global__ void __launch_bounds__(256, 3)
gate_update_fwd_rows_kernel(const GateFwdArgs a) {
  pdl_enter();
  constexpr int RPI = 8 / NW;
  extern __shared__ __align__(16) uint8_t gate_smem[];
  uint4* buf = reinterpret_cast<uint4*>(gate_smem) + threadIdx.x;               // slot i of this thread: buf[i * 256]
  float* part = reinterpret_cast<float*>(gate_smem + 4 * 256 * 16);             // [2][8 warps], then [8] for the gate sum
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rslot = warp / NW, wchunk = warp % NW;
  const int col = wchunk * 256 + lane * 8;
  float wr[8];
  {
    const float4 w0 = *reinterpret_cast<const float4*>(a.w_r + col), w1 = *reinterpret_cast<const float4*>(a.w_r + col + 4);
    wr[0] = w0.x; wr[1] = w0.y; wr[2] = w0.z; wr[3] = w0.w; wr[4] = w1.x; wr[5] = w1.y; wr[6] = w1.z; wr[7] = w1.w;
  }
  const int64_t n_groups = (a.rows + RPI - 1) / RPI;
  auto prefetch = [&](int64_t grp) {
    const int64_t row = grp * RPI + rslot;
    const bool ok = row < a.rows;
    const int64_t r = ok ? row : 0;
    cp_async_16(buf + 0 * 256, a.z + r * a.d + col, ok);
    cp_async_16(buf + 1 * 256, a.g_pre + r * a.d + col, ok);
    cp_async_16(buf + 2 * 256, a.c + r * a.c_ld + col, ok);
    cp_async_16(buf + 3 * 256, a.s + r * a.s_ld + col, ok);
    cp_async_commit();
  };
  float gsum = 0.0f;
  int64_t grp = blockIdx.x;
  int par = 0;
  if (grp < n_groups) prefetch(grp);
  for (; grp < n_groups; grp += gridDim.x, par ^= 1) {
    const int64_t row = grp * RPI + rslot;
    const bool live = row < a.rows;                    // warp-uniform
    cp_async_wait_but<0>();
    uint4 q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = buf[i * 256];
    if (grp + gridDim.x < n_groups) prefetch(grp + gridDim.x);
    const uint32_t* zw = reinterpret_cast<const uint32_t*>(&q[0]);
    const uint32_t* gw = reinterpret_cast<const uint32_t*>(&q[1]);
    const uint32_t* cw = reinterpret_cast<const uint32_t*>(&q[2]);
    const uint32_t* sw = reinterpret_cast<const uint32_t*>(&q[3]);
    float ssq = 0.0f;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 zv = unpack_bf16x2(zw[t]);
      ssq = fmaf(zv.x, zv.x, ssq);
      ssq = fmaf(zv.y, zv.y, ssq);
    }
    ssq = warp_sum(ssq);
    if (NW > 1) {
      float* mine = part + par * 8 + rslot * NW;
      if (lane == 0) mine[wchunk] = ssq;
      row_group_barrier<NW * 32>(rslot);
      ssq = 0.0f;
#pragma unroll
      for (int w = 0; w < NW; ++w) ssq += mine[w];
    }
    if (!live) continue;
    const float rstd = rsqrtf(ssq / (float)a.d + a.eps_r);
    if (lane == 0 && wchunk == 0 && a.rstd_out != nullptr) a.rstd_out[row] = rstd;
    float fo[8], so[8], gv[8];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 zv = unpack_bf16x2(zw[t]), gp = unpack_bf16x2(gw[t]), cv = unpack_bf16x2(cw[t]), sv = unpack_bf16x2(sw[t]);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = 2 * t + h;
        const float zz = h ? zv.y : zv.x, gg = h ? gp.y : gp.x, cc = h ? cv.y : cv.x, ss = h ? sv.y : sv.x;
        const float R = sigmoidf_(zz * rstd * wr[i]);
        const float g = sigmoidf_(gg);
        gv[i] = g;
        gsum += g;
        fo[i] = cc * g + ss * R;
        so[i] = cc * (1.0f - g) + ss * (1.0f - R);
      }
    }
    st8(a.fwd_out + row * a.d + col, fo);
    st8(a.side_out + row * a.d + col, so);
    if (a.gate_out != nullptr) st8(a.gate_out + row * a.d + col, gv);
    if (a.quant.q != nullptr) {   // the next step's recovery GEMM reads the side stream in FP8
#pragma unroll
      for (int i = 0; i < 8; ++i) so[i] = __bfloat162float(__float2bfloat16(so[i]));
      quant_emit_8(a.quant, so, row, col, true);
    }
  }
  if (a.gate_sum != nullptr) {
    gsum = warp_sum(gsum);
    float* gpart = part + 16;
    if (lane == 0) gpart[warp] = gsum;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.0f;
      for (int i = 0; i < 8; ++i) t += gpart[i];
      atomicAdd(a.gate_sum, t);
    }
  }
}

template <int NW>
static const char* gate_fwd_rows_launch(const GateFwdArgs& a, cudaStream_t st) {
  const size_t smem = 4 * 256 * 16 + 24 * sizeof(float);
  const int64_t groups = (a.rows + 8 / NW - 1) / (8 / NW);
  launch_pdl(gate_update_fwd_rows_kernel<NW>, dim3((unsigned)std::min<int64_t>(groups, 148 * 3)), dim3(256), smem, st, a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "gate_update_fwd launch failed";
}

const char* launch_gate_update_fwd(const GateFwdArgs& a, cudaStream_t st) {
  if (a.d % 8 != 0) return "gate_update: d must be a multiple of 8";
  static const bool rows_off = getenv("GDNET_GATE_ROWS") != nullptr && atoi(getenv("GDNET_GATE_ROWS")) == 0;
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(a.z) | reinterpret_cast<uintptr_t>(a.s) | reinterpret_cast<uintptr_t>(a.g_pre) |
                         reinterpret_cast<uintptr_t>(a.c);
  if (!rows_off && ptrs % 16 == 0 && (a.c_ld | a.s_ld) % 8 == 0) {
    if (a.d == 256) return gate_fwd_rows_launch<1>(a, st);
    if (a.d == 512) return gate_fwd_rows_launch<2>(a, st);
    if (a.d == 1024) return gate_fwd_rows_launch<4>(a, st);
    if (a.d == 2048) return gate_fwd_rows_launch<8>(a, st);
  }
  const int64_t blocks = (a.rows + 7) / 8;
  const int grid = (int)(blocks < 148 * 8 ? blocks : 148 * 8);
  launch_pdl(gate_update_fwd_kernel, dim3(grid), dim3(256), 0, st, a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "gate_update_fwd launch failed";
}

// Backward of the update and of both activations feeding it.
//   g = sigmoid(g_pre), zh = z*rstd, R = sigmoid(zh*w_r), D = dF - dS
//   dg_pre = (D*c + dgm) * g(1-g)            dgm = d(loss)/d(mean g) / (rows*d)
//   dq     = dg_pre * rstd_g                 (gradient of the un-normalised gate GEMM output)
//   T_row  = sum_n dg_pre * (g_pre - b2g)    (for the rstd term of the gate RMSNorm)
//   dc_dir = dF*g + dS*(1-g),  ds_dir = dF*R + dS*(1-R)
//   dy = D*s*R(1-R),  dzh = dy*w_r,  dz = rstd*(dzh - zh*mean_n(dzh*zh))
//   column sums: db2g += dg_pre, dw_r += dy*zh, db2r += dz
// One kernel, one warp per row, two passes over the row. The first pass gives the row statistics (mean_n(dzh*zh),
// rstd_g, rowcoef = rstd_g^2/d * T_row); the second reads the row again, which the first pass has just brought
// into L1 / L2, so HBM sees every input once, and writes the outputs. The three column sums are added into
// shared memory per element (native shared-memory float adds, laid out so that a warp's lanes hit different
// banks) and leave the block with one global atomic per column.
struct GateElem {
  float dgp, dy, zh, g, R;
};

__device__ __forceinline__ GateElem gate_elem(float dF, float dS, float z, float s, float gp, float c, float wr,
                                              float rstd, float dgm) {
  GateElem e;
  e.zh = z * rstd;
  e.R = sigmoidf_(e.zh * wr);
  e.g = sigmoidf_(gp);
  const float D = dF - dS;
  e.dgp = (D * c + dgm) * e.g * (1.0f - e.g);
  e.dy = D * s * e.R * (1.0f - e.R);
  return e;
}

// column c of the row lives at slot (c / 256) * 256 + (c % 8) * 32 + (c % 256) / 8 of a column-sum array: the eight
// columns of a lane are 32 words apart, so the 32 lanes of a warp add into 32 different banks
__device__ __forceinline__ int colsum_slot(int col0, int lane, int i) { return col0 - lane * 8 + i * 32 + lane; }

__global__ void __launch_bounds__(256, 3)
gate_update_bwd_kernel(const GateBwdArgs a) {
  pdl_enter();
  extern __shared__ float gate_acc[];      // [3][dpad]: db2g, dw_r, db2r
  const int dpad = (a.d + 255) / 256 * 256;
  for (int i = threadIdx.x; i < 3 * dpad; i += blockDim.x) gate_acc[i] = 0.0f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  const float dgm = (a.dgate_mean != nullptr) ? a.dgate_mean[0] / ((float)a.rows * (float)a.d) : 0.0f;
  for (int64_t row = (int64_t)blockIdx.x * wpb + warp; row < a.rows; row += (int64_t)gridDim.x * wpb) {
    const float rstd = a.rstd_z[row];
    float ssum = 0.0f;
    for (int p = lane; p < a.ssq_parts; p += 32) ssum += a.ssq_g[row * a.ssq_parts + p];
    ssum = warp_sum(ssum);
    const float rstd_g = rsqrtf(ssum / (float)a.d + a.eps_g);
    float dot_z = 0.0f, t_row = 0.0f;
    for (int col = lane * 8; col < a.d; col += 256) {
      float dF[8], dS[8], zv[8], sv[8], gp[8], cv[8];
      ld8(a.dF + row * a.dF_ld + col, dF);
      ld8(a.dS + row * a.dS_ld + col, dS);
      ld8(a.z + row * a.d + col, zv);
      ld8(a.s + row * a.s_ld + col, sv);
      ld8(a.g_pre + row * a.d + col, gp);
      ld8(a.c + row * a.c_ld + col, cv);
      const float4 w0 = *reinterpret_cast<const float4*>(a.w_r + col), w1 = *reinterpret_cast<const float4*>(a.w_r + col + 4);
      const float4 b0 = *reinterpret_cast<const float4*>(a.b2g + col), b1 = *reinterpret_cast<const float4*>(a.b2g + col + 4);
      const float wr[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      const float b2[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const GateElem e = gate_elem(dF[i], dS[i], zv[i], sv[i], gp[i], cv[i], wr[i], rstd, dgm);
        dot_z = fmaf(e.dy * wr[i], e.zh, dot_z);
        t_row = fmaf(e.dgp, gp[i] - b2[i], t_row);
      }
    }
    dot_z = warp_sum(dot_z) / (float)a.d;
    t_row = warp_sum(t_row);
    if (lane == 0) a.rowcoef[row] = rstd_g * rstd_g / (float)a.d * t_row;
    for (int col = lane * 8; col < a.d; col += 256) {
      float dF[8], dS[8], zv[8], sv[8], gp[8], cv[8], dq[8], dz[8], dcd[8], dsd[8];
      ld8(a.dF + row * a.dF_ld + col, dF);
      ld8(a.dS + row * a.dS_ld + col, dS);
      ld8(a.z + row * a.d + col, zv);
      ld8(a.s + row * a.s_ld + col, sv);
      ld8(a.g_pre + row * a.d + col, gp);
      ld8(a.c + row * a.c_ld + col, cv);
      const float4 w0 = *reinterpret_cast<const float4*>(a.w_r + col), w1 = *reinterpret_cast<const float4*>(a.w_r + col + 4);
      const float wr[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const GateElem e = gate_elem(dF[i], dS[i], zv[i], sv[i], gp[i], cv[i], wr[i], rstd, dgm);
        const float dzv = rstd * (e.dy * wr[i] - e.zh * dot_z);
        dq[i] = e.dgp * rstd_g;
        dz[i] = dzv;
        dcd[i] = dF[i] * e.g + dS[i] * (1.0f - e.g);
        dsd[i] = dF[i] * e.R + dS[i] * (1.0f - e.R);
        const int slot = colsum_slot(col, lane, i);
        atomicAdd(&gate_acc[slot], e.dgp);
        atomicAdd(&gate_acc[dpad + slot], e.dy * e.zh);
        atomicAdd(&gate_acc[2 * dpad + slot], dzv);
      }
      st8(a.dq + row * a.d + col, dq);
      st8(a.dz + row * a.d + col, dz);
      st8(a.dsc + row * 2 * a.d + col, dsd);
      st8(a.dsc + row * 2 * a.d + a.d + col, dcd);
      if (a.quant_dz.q != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) dz[i] = __bfloat162float(__float2bfloat16(dz[i]));
        quant_emit_8(a.quant_dz, dz, row, col, true);
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < a.d; c += blockDim.x) {
    const int in = c & 255;
    const int slot = (c - in) + (in & 7) * 32 + (in >> 3);
    atomicAdd(a.db2g + c, gate_acc[slot]);
    atomicAdd(a.dw_r + c, gate_acc[dpad + slot]);
    atomicAdd(a.db2r + c, gate_acc[2 * dpad + slot]);
  }
}

// The same computation for d == NW * 256 (NW = 1, 2, 4, 8) with every input read once and every element evaluated
// once. NW warps share a row, each lane owning 8 of its columns; the 8 warps of a block work on 8 / NW rows at a
// time on a persistent grid. A lane keeps what the second pass needs of its 8 elements in registers, the NW warps
// of a row exchange their partial row sums through shared memory (one named barrier per row), and the three column
// sums stay in registers over all rows of the lane (its columns never change), leaving the block through shared
// memory once at the end. The next rows' inputs are on their way (per-thread asynchronous copies) while the
// current ones are computed.
template <int NW>
__global__ void __launch_bounds__(256, 2)
gate_update_bwd_rows_kernel(const GateBwdArgs a) {
  pdl_enter();
  constexpr int RPI = 8 / NW;                          // rows per block iteration
  extern __shared__ __align__(16) uint8_t gate_smem[];
  uint4* buf = reinterpret_cast<uint4*>(gate_smem) + threadIdx.x;               // slot i of this thread: buf[i * 256]
  float* gate_acc = reinterpret_cast<float*>(gate_smem + 6 * 256 * 16);         // [3][d]: db2g, dw_r, db2r
  float* part = gate_acc + 3 * a.d;                                             // [2][8 warps][2]
  for (int i = threadIdx.x; i < 3 * a.d; i += blockDim.x) gate_acc[i] = 0.0f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rslot = warp / NW, wchunk = warp % NW;
  const int col = wchunk * 256 + lane * 8;
  const float dgm = (a.dgate_mean != nullptr) ? a.dgate_mean[0] / ((float)a.rows * (float)a.d) : 0.0f;
  float wr[8];
  {
    const float4 w0 = *reinterpret_cast<const float4*>(a.w_r + col), w1 = *reinterpret_cast<const float4*>(a.w_r + col + 4);
    wr[0] = w0.x; wr[1] = w0.y; wr[2] = w0.z; wr[3] = w0.w; wr[4] = w1.x; wr[5] = w1.y; wr[6] = w1.z; wr[7] = w1.w;
  }
  float cs[3][8];
#pragma unroll
  for (int k = 0; k < 3; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) cs[k][i] = 0.0f;
  const int64_t n_groups = (a.rows + RPI - 1) / RPI;
  auto prefetch = [&](int64_t grp) {
    const int64_t row = grp * RPI + rslot;
    const bool ok = row < a.rows;
    const int64_t r = ok ? row : 0;
    cp_async_16(buf + 0 * 256, a.dF + r * a.dF_ld + col, ok);
    cp_async_16(buf + 1 * 256, a.dS + r * a.dS_ld + col, ok);
    cp_async_16(buf + 2 * 256, a.z + r * a.d + col, ok);
    cp_async_16(buf + 3 * 256, a.s + r * a.s_ld + col, ok);
    cp_async_16(buf + 4 * 256, a.g_pre + r * a.d + col, ok);
    cp_async_16(buf + 5 * 256, a.c + r * a.c_ld + col, ok);
    cp_async_commit();
  };
  int64_t grp = blockIdx.x;
  int par = 0;
  if (grp < n_groups) prefetch(grp);
  for (; grp < n_groups; grp += gridDim.x, par ^= 1) {
    const int64_t row = grp * RPI + rslot;
    const bool live = row < a.rows;                    // warp-uniform
    cp_async_wait_but<0>();
    uint4 q[6];
#pragma unroll
    for (int i = 0; i < 6; ++i) q[i] = buf[i * 256];
    if (grp + gridDim.x < n_groups) prefetch(grp + gridDim.x);
    const float rstd = live ? a.rstd_z[row] : 0.0f;
    float ssum = 0.0f;
    if (live && lane < a.ssq_parts) ssum = a.ssq_g[row * a.ssq_parts + lane];
    ssum = warp_sum(ssum);
    const float rstd_g = rsqrtf(ssum / (float)a.d + a.eps_g);
    float dgp[8], dy[8], zh[8], gg[8], RR[8];
    float dot_z = 0.0f, t_row = 0.0f;
    {
      const float4 b0 = *reinterpret_cast<const float4*>(a.b2g + col), b1 = *reinterpret_cast<const float4*>(a.b2g + col + 4);
      const float b2[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&q[0]);
      const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&q[1]);
      const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&q[2]);
      const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&q[3]);
      const uint32_t* w4 = reinterpret_cast<const uint32_t*>(&q[4]);
      const uint32_t* w5 = reinterpret_cast<const uint32_t*>(&q[5]);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 dF = unpack_bf16x2(w0[t]), dS = unpack_bf16x2(w1[t]), zv = unpack_bf16x2(w2[t]);
        const float2 sv = unpack_bf16x2(w3[t]), gp = unpack_bf16x2(w4[t]), cv = unpack_bf16x2(w5[t]);
        const GateElem e0 = gate_elem(dF.x, dS.x, zv.x, sv.x, gp.x, cv.x, wr[2 * t], rstd, dgm);
        const GateElem e1 = gate_elem(dF.y, dS.y, zv.y, sv.y, gp.y, cv.y, wr[2 * t + 1], rstd, dgm);
        dgp[2 * t] = e0.dgp; dy[2 * t] = e0.dy; zh[2 * t] = e0.zh; gg[2 * t] = e0.g; RR[2 * t] = e0.R;
        dgp[2 * t + 1] = e1.dgp; dy[2 * t + 1] = e1.dy; zh[2 * t + 1] = e1.zh; gg[2 * t + 1] = e1.g; RR[2 * t + 1] = e1.R;
        dot_z = fmaf(e0.dy * wr[2 * t], e0.zh, dot_z);
        dot_z = fmaf(e1.dy * wr[2 * t + 1], e1.zh, dot_z);
        t_row = fmaf(e0.dgp, gp.x - b2[2 * t], t_row);
        t_row = fmaf(e1.dgp, gp.y - b2[2 * t + 1], t_row);
      }
    }
    dot_z = warp_sum(dot_z);
    t_row = warp_sum(t_row);
    if (NW > 1) {
      float* mine = part + (par * 8 + rslot * NW) * 2;
      if (lane == 0) {
        mine[wchunk * 2] = dot_z;
        mine[wchunk * 2 + 1] = t_row;
      }
      row_group_barrier<NW * 32>(rslot);
      dot_z = 0.0f;
      t_row = 0.0f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        dot_z += mine[w * 2];
        t_row += mine[w * 2 + 1];
      }
    }
    dot_z /= (float)a.d;
    if (!live) continue;
    if (lane == 0 && wchunk == 0) a.rowcoef[row] = rstd_g * rstd_g / (float)a.d * t_row;
    float dq[8], dz[8], dcd[8], dsd[8];
    const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&q[0]);
    const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&q[1]);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 dF = unpack_bf16x2(w0[t]), dS = unpack_bf16x2(w1[t]);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = 2 * t + h;
        const float f = h ? dF.y : dF.x, sg = h ? dS.y : dS.x;
        const float dzv = rstd * (dy[i] * wr[i] - zh[i] * dot_z);
        dq[i] = dgp[i] * rstd_g;
        dz[i] = dzv;
        dcd[i] = fmaf(f - sg, gg[i], sg);         // dF*g + dS*(1-g)
        dsd[i] = fmaf(f - sg, RR[i], sg);
        cs[0][i] += dgp[i];
        cs[1][i] = fmaf(dy[i], zh[i], cs[1][i]);
        cs[2][i] += dzv;
      }
    }
    st8(a.dq + row * a.d + col, dq);
    st8(a.dz + row * a.d + col, dz);
    st8(a.dsc + row * 2 * a.d + col, dsd);
    st8(a.dsc + row * 2 * a.d + a.d + col, dcd);
    if (a.quant_dz.q != nullptr) {
#pragma unroll
      for (int i = 0; i < 8; ++i) dz[i] = __bfloat162float(__float2bfloat16(dz[i]));
      quant_emit_8(a.quant_dz, dz, row, col, true);
    }
  }
#pragma unroll
  for (int k = 0; k < 3; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) atomicAdd(&gate_acc[k * a.d + wchunk * 256 + i * 32 + lane], cs[k][i]);   // lanes on 32 banks
  __syncthreads();
  for (int c = threadIdx.x; c < a.d; c += blockDim.x) {
    const int in = c & 255;
    const int slot = (c - in) + (in & 7) * 32 + (in >> 3);
    atomicAdd(a.db2g + c, gate_acc[slot]);
    atomicAdd(a.dw_r + c, gate_acc[a.d + slot]);
    atomicAdd(a.db2r + c, gate_acc[2 * a.d + slot]);
  }
}

template <int NW>
static const char* gate_bwd_rows_launch(const GateBwdArgs& a, cudaStream_t st) {
  const size_t smem = 6 * 256 * 16 + 3 * (size_t)a.d * sizeof(float) + 2 * 8 * 2 * sizeof(float);
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gate_update_bwd_rows_kernel<NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    attr = true;
  }
  const int64_t groups = (a.rows + 8 / NW - 1) / (8 / NW);
  launch_pdl(gate_update_bwd_rows_kernel<NW>, dim3((unsigned)std::min<int64_t>(groups, 148 * 2)), dim3(256), smem, st, a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "gate_update_bwd launch failed";
}

const char* launch_gate_update_bwd(const GateBwdArgs& a, cudaStream_t st) {
  if (a.d % 8 != 0) return "gate_update_bwd: d must be a multiple of 8";
  if (!a.b2g_f32) return "gate_update_bwd: the gate bias must be fp32";
  if (a.quant_dz.q != nullptr && a.d % 128 != 0) return "gate_update_bwd: a quantised dz needs d % 128 == 0";
  static const bool rows_off = getenv("GDNET_GATE_ROWS") != nullptr && atoi(getenv("GDNET_GATE_ROWS")) == 0;
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(a.dF) | reinterpret_cast<uintptr_t>(a.dS) | reinterpret_cast<uintptr_t>(a.z) |
                         reinterpret_cast<uintptr_t>(a.s) | reinterpret_cast<uintptr_t>(a.g_pre) | reinterpret_cast<uintptr_t>(a.c);
  if (!rows_off && ptrs % 16 == 0 && (a.dF_ld | a.dS_ld | a.c_ld | a.s_ld) % 8 == 0 && a.ssq_parts <= 32) {
    if (a.d == 256) return gate_bwd_rows_launch<1>(a, st);
    if (a.d == 512) return gate_bwd_rows_launch<2>(a, st);
    if (a.d == 1024) return gate_bwd_rows_launch<4>(a, st);
    if (a.d == 2048) return gate_bwd_rows_launch<8>(a, st);
  }
  const int dpad = (a.d + 255) / 256 * 256;
  const size_t smem = 3 * (size_t)dpad * sizeof(float);
  if (smem > 96 * 1024) return "gate_update_bwd: d too large for the column sums in shared memory";
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gate_update_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    attr = true;
  }
  // enough blocks to fill the GPU, few enough that the per-block global atomics of the column sums stay cheap
  int64_t blocks = (a.rows + 7) / 8;
  if (blocks > 148 * 6) blocks = 148 * 6;
  launch_pdl(gate_update_bwd_kernel, dim3((unsigned)blocks), dim3(256), smem, st, a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "gate_update_bwd launch failed";
}

// =======================================================================================
// stream update of a step with an all-zero side stream
// =======================================================================================
// One warp per row (NCH chunks of 256 columns, 8 per lane and chunk), persistent grid, the next row's inputs on
// their way (per-thread asynchronous copies) while the current one is computed.
template <int NCH>
__global__ void __launch_bounds__(256, 2)
gate_only_fwd_kernel(const GateOnlyFwdArgs a) {
  pdl_enter();
  extern __shared__ __align__(16) uint8_t gate_smem[];
  uint4* buf = reinterpret_cast<uint4*>(gate_smem) + threadIdx.x;               // slot i of this thread: buf[i * 256]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t step = (int64_t)gridDim.x * 8;
  auto prefetch = [&](int64_t row) {
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      cp_async_16(buf + (2 * ch) * 256, a.g_pre + row * a.d + ch * 256 + lane * 8, true);
      cp_async_16(buf + (2 * ch + 1) * 256, a.c + row * a.c_ld + ch * 256 + lane * 8, true);
    }
    cp_async_commit();
  };
  float gsum = 0.0f;
  int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row < a.rows) prefetch(row);
  for (; row < a.rows; row += step) {
    cp_async_wait_but<0>();
    uint4 q[2 * NCH];
#pragma unroll
    for (int i = 0; i < 2 * NCH; ++i) q[i] = buf[i * 256];
    if (row + step < a.rows) prefetch(row + step);
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int col = ch * 256 + lane * 8;
      const uint32_t* gw = reinterpret_cast<const uint32_t*>(&q[2 * ch]);
      const uint32_t* cw = reinterpret_cast<const uint32_t*>(&q[2 * ch + 1]);
      float fo[8], so[8];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 gp = unpack_bf16x2(gw[t]), cv = unpack_bf16x2(cw[t]);
        const float g0 = sigmoidf_(gp.x), g1 = sigmoidf_(gp.y);
        gsum += g0 + g1;
        fo[2 * t] = cv.x * g0;
        fo[2 * t + 1] = cv.y * g1;
        so[2 * t] = cv.x * (1.0f - g0);
        so[2 * t + 1] = cv.y * (1.0f - g1);
      }
      st8(a.fwd_out + row * a.d + col, fo);
      st8(a.side_out + row * a.d + col, so);
      if (a.quant.q != nullptr) {   // the next step's recovery GEMM reads the side stream in FP8
#pragma unroll
        for (int i = 0; i < 8; ++i) so[i] = __bfloat162float(__float2bfloat16(so[i]));
        quant_emit_8(a.quant, so, row, col, true);
      }
    }
  }
  if (a.gate_sum != nullptr) {
    gsum = warp_sum(gsum);
    __shared__ float gpart[8];
    if (lane == 0) gpart[warp] = gsum;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.0f;
      for (int i = 0; i < 8; ++i) t += gpart[i];
      atomicAdd(a.gate_sum, t);
    }
  }
}

// A row is worked through in NP parts of CH chunks (CH <= 2, so that a part's inputs fit the registers); the
// prefetch runs one part ahead.
template <int NCH>
__global__ void __launch_bounds__(256, 2)
gate_only_bwd_kernel(const GateOnlyBwdArgs a) {
  pdl_enter();
  constexpr int CH = NCH > 2 ? 2 : NCH, NP = NCH / CH;
  extern __shared__ __align__(16) uint8_t gate_smem[];
  uint4* buf = reinterpret_cast<uint4*>(gate_smem) + threadIdx.x;               // slot i of this thread: buf[i * 256]
  float* colacc = reinterpret_cast<float*>(gate_smem + 4 * CH * 256 * 16);      // [d]
  for (int i = threadIdx.x; i < a.d; i += blockDim.x) colacc[i] = 0.0f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float dgm = (a.dgate_mean != nullptr) ? a.dgate_mean[0] / ((float)a.rows * (float)a.d) : 0.0f;
  const int64_t step = (int64_t)gridDim.x * 8;
  auto prefetch = [&](int64_t row, int part) {
#pragma unroll
    for (int ch = 0; ch < CH; ++ch) {
      const int col = (part * CH + ch) * 256 + lane * 8;
      cp_async_16(buf + (4 * ch) * 256, a.dF + row * a.dF_ld + col, true);
      cp_async_16(buf + (4 * ch + 1) * 256, a.dS + row * a.dS_ld + col, true);
      cp_async_16(buf + (4 * ch + 2) * 256, a.g_pre + row * a.d + col, true);
      cp_async_16(buf + (4 * ch + 3) * 256, a.c + row * a.c_ld + col, true);
    }
    cp_async_commit();
  };
  float cs[NCH][8];
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
    for (int i = 0; i < 8; ++i) cs[ch][i] = 0.0f;
  int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row < a.rows) prefetch(row, 0);
  for (; row < a.rows; row += step) {
    float ssum = 0.0f;
    if (lane < a.ssq_parts) ssum = a.ssq_g[row * a.ssq_parts + lane];
    ssum = warp_sum(ssum);
    const float rstd_g = rsqrtf(ssum / (float)a.d + a.eps_g);
    float t_row = 0.0f;
#pragma unroll
    for (int part = 0; part < NP; ++part) {
      cp_async_wait_but<0>();
      uint4 q[4 * CH];
#pragma unroll
      for (int i = 0; i < 4 * CH; ++i) q[i] = buf[i * 256];
      if (part + 1 < NP) prefetch(row, part + 1);
      else if (row + step < a.rows) prefetch(row + step, 0);
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) {
        const int col = (part * CH + ch) * 256 + lane * 8;
        const uint32_t* fw = reinterpret_cast<const uint32_t*>(&q[4 * ch]);
        const uint32_t* sw = reinterpret_cast<const uint32_t*>(&q[4 * ch + 1]);
        const uint32_t* gw = reinterpret_cast<const uint32_t*>(&q[4 * ch + 2]);
        const uint32_t* cw = reinterpret_cast<const uint32_t*>(&q[4 * ch + 3]);
        const float4 b0 = *reinterpret_cast<const float4*>(a.b2g + col), b1 = *reinterpret_cast<const float4*>(a.b2g + col + 4);
        const float b2[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        float dq[8], dc[8];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 dF = unpack_bf16x2(fw[t]), dS = unpack_bf16x2(sw[t]), gp = unpack_bf16x2(gw[t]), cv = unpack_bf16x2(cw[t]);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int i = 2 * t + h;
            const float f = h ? dF.y : dF.x, sg = h ? dS.y : dS.x, gpre = h ? gp.y : gp.x, cc = h ? cv.y : cv.x;
            const float g = sigmoidf_(gpre);
            const float D = f - sg;
            const float dgp = (D * cc + dgm) * g * (1.0f - g);
            t_row = fmaf(dgp, gpre - b2[i], t_row);
            dq[i] = dgp * rstd_g;
            dc[i] = fmaf(D, g, sg);               // dF g + dS (1 - g)
            cs[part * CH + ch][i] += dgp;
          }
        }
        st8(a.dq + row * a.d + col, dq);
        st8(a.dc + row * a.d + col, dc);
      }
    }
    t_row = warp_sum(t_row);
    if (lane == 0) a.rowcoef[row] = rstd_g * rstd_g / (float)a.d * t_row;
  }
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
    for (int i = 0; i < 8; ++i) atomicAdd(&colacc[ch * 256 + i * 32 + lane], cs[ch][i]);      // lanes on 32 banks
  __syncthreads();
  for (int c = threadIdx.x; c < a.d; c += blockDim.x) {
    const int in = c & 255;
    atomicAdd(a.db2g + c, colacc[(c - in) + (in & 7) * 32 + (in >> 3)]);
  }
}

template <int NCH>
static void gate_only_launch_both(const GateOnlyFwdArgs* f, const GateOnlyBwdArgs* b, cudaStream_t st) {
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(gate_only_fwd_kernel<NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * NCH * 256 * 16);
    cudaFuncSetAttribute(gate_only_bwd_kernel<NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * (NCH > 2 ? 2 : NCH) * 256 * 16 + NCH * 256 * 4);
    attr = true;
  }
  const int64_t rows = f != nullptr ? f->rows : b->rows;
  const unsigned grid = (unsigned)std::min<int64_t>((rows + 7) / 8, 148 * 2);
  if (f != nullptr) launch_pdl(gate_only_fwd_kernel<NCH>, dim3(grid), dim3(256), (size_t)2 * NCH * 256 * 16, st, *f);
  else launch_pdl(gate_only_bwd_kernel<NCH>, dim3(grid), dim3(256), (size_t)4 * (NCH > 2 ? 2 : NCH) * 256 * 16 + NCH * 256 * 4, st, *b);
}

static const char* gate_only_dispatch(int d, const GateOnlyFwdArgs* f, const GateOnlyBwdArgs* b, cudaStream_t st) {
  switch (d / 256) {
    case 1: gate_only_launch_both<1>(f, b, st); break;
    case 2: gate_only_launch_both<2>(f, b, st); break;
    case 4: gate_only_launch_both<4>(f, b, st); break;
    case 8: gate_only_launch_both<8>(f, b, st); break;
    default: return "gate_only: d must be 256, 512, 1024 or 2048";
  }
  return cudaGetLastError() == cudaSuccess ? nullptr : "gate_only launch failed";
}

const char* launch_gate_only_fwd(const GateOnlyFwdArgs& a, cudaStream_t st) {
  if (a.d % 256 != 0) return "gate_only: d must be 256, 512, 1024 or 2048";
  if (a.c_ld % 8 != 0 || (reinterpret_cast<uintptr_t>(a.g_pre) | reinterpret_cast<uintptr_t>(a.c)) % 16 != 0)
    return "gate_only: rows must be 16-byte aligned";
  return gate_only_dispatch(a.d, &a, nullptr, st);
}

const char* launch_gate_only_bwd(const GateOnlyBwdArgs& a, cudaStream_t st) {
  if (a.d % 256 != 0) return "gate_only: d must be 256, 512, 1024 or 2048";
  if ((a.c_ld | a.dF_ld | a.dS_ld) % 8 != 0 ||
      (reinterpret_cast<uintptr_t>(a.g_pre) | reinterpret_cast<uintptr_t>(a.c) | reinterpret_cast<uintptr_t>(a.dF) |
       reinterpret_cast<uintptr_t>(a.dS)) % 16 != 0)
    return "gate_only: rows must be 16-byte aligned";
  if (a.ssq_parts > 32) return "gate_only: at most 32 partial sums of squares per row";
  return gate_only_dispatch(a.d, nullptr, &a, st);
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
// One warp per row. NCH > 0: d == NCH * 256; a lane keeps its 8 * NCH elements of dy and x in registers between the
// row dot product and the output (one read of each row) and sums its columns of dw in registers over all its rows;
// the warps of a block combine through shared memory and add once per column. NCH == 0: any d (a multiple of 8),
// two reads per row and shared-memory atomics for the column sums.
template <int NCH>
__global__ void __launch_bounds__(256, NCH <= 4 ? 2 : 1)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const float* __restrict__ w, const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw, int64_t rows, int d) {
  extern __shared__ float colacc[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  for (int i = threadIdx.x; i < d; i += blockDim.x) colacc[i] = 0.0f;
  __syncthreads();
  if constexpr (NCH > 0) {
    float acc[NCH][8];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[c][i] = 0.0f;
    }
    for (int64_t row = (int64_t)blockIdx.x * wpb + warp; row < rows; row += (int64_t)gridDim.x * wpb) {
      const float rstd = rstd_in[row];
      uint4 gq[NCH], vq[NCH];
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        gq[c] = __ldg(reinterpret_cast<const uint4*>(dy + row * d + c * 256 + lane * 8));
        vq[c] = __ldg(reinterpret_cast<const uint4*>(x + row * d + c * 256 + lane * 8));
      }
      float dot = 0.0f;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const uint32_t* gw = reinterpret_cast<const uint32_t*>(&gq[c]);
        const uint32_t* vw = reinterpret_cast<const uint32_t*>(&vq[c]);
        const float4 wa = __ldg(reinterpret_cast<const float4*>(w + c * 256 + lane * 8));
        const float4 wb = __ldg(reinterpret_cast<const float4*>(w + c * 256 + lane * 8 + 4));
        const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 g = unpack_bf16x2(gw[t]), v = unpack_bf16x2(vw[t]);
          dot = fmaf(g.x * wv[2 * t], v.x, dot);
          dot = fmaf(g.y * wv[2 * t + 1], v.y, dot);
        }
      }
      dot *= rstd;
      dot = warp_sum(dot) / (float)d;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const uint32_t* gw = reinterpret_cast<const uint32_t*>(&gq[c]);
        const uint32_t* vw = reinterpret_cast<const uint32_t*>(&vq[c]);
        const float4 wa = __ldg(reinterpret_cast<const float4*>(w + c * 256 + lane * 8));
        const float4 wb = __ldg(reinterpret_cast<const float4*>(w + c * 256 + lane * 8 + 4));
        const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 g = unpack_bf16x2(gw[t]), v = unpack_bf16x2(vw[t]);
          const float xh0 = v.x * rstd, xh1 = v.y * rstd;
          acc[c][2 * t] = fmaf(g.x, xh0, acc[c][2 * t]);
          acc[c][2 * t + 1] = fmaf(g.y, xh1, acc[c][2 * t + 1]);
          ow[t] = pack_bf16x2(rstd * (g.x * wv[2 * t] - xh0 * dot), rstd * (g.y * wv[2 * t + 1] - xh1 * dot));
        }
        *reinterpret_cast<uint4*>(dx + row * d + c * 256 + lane * 8) = o;
      }
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(&colacc[c * 256 + lane * 8 + i], acc[c][i]);
    }
  } else {
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
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) atomicAdd(dw + i, colacc[i]);
}

// ---------------------------------------------------------------------------------------
// read-out blend of the content-addressed memory: one warp per row
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
cam_blend_fwd_kernel(const CamBlendArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  for (int64_t row = (int64_t)blockIdx.x * wpb + warp; row < a.rows; row += (int64_t)gridDim.x * wpb) {
    const __nv_bfloat16* zr = a.z + row * a.d;
    const __nv_bfloat16* rr = a.retr + (row / a.T) * a.d;
    float ssq = 0.0f;
    for (int col = lane * 8; col < a.d; col += 256) {
      float zv[8];
      ld8(zr + col, zv);
#pragma unroll
      for (int i = 0; i < 8; ++i) ssq = fmaf(zv[i], zv[i], ssq);
    }
    ssq = warp_sum(ssq);
    const float rstd = rsqrtf(ssq / (float)a.d + a.eps);
    if (lane == 0) a.rstd[row] = rstd;
    for (int col = lane * 8; col < a.d; col += 256) {
      float zv[8], fv[8], rv[8], o[8];
      ld8(zr + col, zv);
      ld8(a.fwd + row * a.d + col, fv);
      ld8(rr + col, rv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float R = sigmoidf_(zv[i] * rstd * a.w[col + i]);
        o[i] = fv[i] + (rv[i] - fv[i]) * R;
      }
      st8(a.out + row * a.d + col, o);
    }
  }
}

// A block walks CAM_ROWS consecutive rows (all of one batch row when T % CAM_ROWS == 0), sums the column terms of
// dw and dretrieved in shared memory and adds them once per column at the end.
constexpr int CAM_ROWS = 32;

__global__ void __launch_bounds__(256)
cam_blend_bwd_kernel(const CamBlendArgs a) {
  extern __shared__ float cam_acc[];     // [2][d]: dw, dretr
  float* acc_w = cam_acc;
  float* acc_r = cam_acc + a.d;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  for (int i = threadIdx.x; i < 2 * a.d; i += blockDim.x) cam_acc[i] = 0.0f;
  __syncthreads();
  const int64_t row0 = (int64_t)blockIdx.x * CAM_ROWS;
  const int64_t b0 = row0 / a.T;
  for (int64_t row = row0 + warp; row < row0 + CAM_ROWS && row < a.rows; row += wpb) {
    const bool same = (row / a.T) == b0;     // rows of another batch row add to global memory directly
    const __nv_bfloat16* rr = a.retr + (row / a.T) * a.d;
    const float rstd = a.rstd[row];
    float dot = 0.0f;
    for (int col = lane * 8; col < a.d; col += 256) {
      float zv[8], fv[8], rv[8], g[8];
      ld8(a.z + row * a.d + col, zv);
      ld8(a.fwd + row * a.d + col, fv);
      ld8(rr + col, rv);
      ld8(a.dout + row * a.d + col, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float zh = zv[i] * rstd;
        const float R = sigmoidf_(zh * a.w[col + i]);
        const float dzn = g[i] * (rv[i] - fv[i]) * R * (1.0f - R);
        dot = fmaf(dzn * a.w[col + i], zh, dot);
      }
    }
    dot = warp_sum(dot) / (float)a.d;
    for (int col = lane * 8; col < a.d; col += 256) {
      float zv[8], fv[8], rv[8], g[8], dz[8], df[8];
      ld8(a.z + row * a.d + col, zv);
      ld8(a.fwd + row * a.d + col, fv);
      ld8(rr + col, rv);
      ld8(a.dout + row * a.d + col, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float zh = zv[i] * rstd;
        const float R = sigmoidf_(zh * a.w[col + i]);
        const float dzn = g[i] * (rv[i] - fv[i]) * R * (1.0f - R);
        dz[i] = rstd * (dzn * a.w[col + i] - zh * dot);
        df[i] = g[i] * (1.0f - R);
        atomicAdd(&acc_w[col + i], dzn * zh);
        if (same) atomicAdd(&acc_r[col + i], g[i] * R);
        else atomicAdd(a.dretr + (row / a.T) * a.d + col + i, g[i] * R);
      }
      st8(a.dz + row * a.d + col, dz);
      st8(a.dfwd + row * a.d + col, df);
    }
  }
  __syncthreads();
  if (row0 < a.rows) {
    for (int i = threadIdx.x; i < a.d; i += blockDim.x) {
      atomicAdd(a.dw + i, acc_w[i]);
      atomicAdd(a.dretr + b0 * a.d + i, acc_r[i]);
    }
  }
}

const char* launch_cam_blend_fwd(const CamBlendArgs& a, cudaStream_t st) {
  if (a.d % 8 != 0 || a.T < 1) return "cam_blend: d must be a multiple of 8";
  if (a.rows == 0) return nullptr;
  const int64_t blocks = (a.rows + 7) / 8;
  cam_blend_fwd_kernel<<<(int)(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "cam_blend_fwd launch failed";
}

const char* launch_cam_blend_bwd(const CamBlendArgs& a, cudaStream_t st) {
  if (a.d % 8 != 0 || a.d > 6144 || a.T < 1) return "cam_blend_bwd: d must be a multiple of 8 and at most 6144";
  if (a.rows == 0) return nullptr;
  const int64_t blocks = (a.rows + CAM_ROWS - 1) / CAM_ROWS;
  if (blocks >= (1ll << 31)) return "cam_blend_bwd: too many rows";
  cam_blend_bwd_kernel<<<(unsigned)blocks, 256, 2 * a.d * sizeof(float), st>>>(a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "cam_blend_bwd launch failed";
}

// d == NCH * 256: a lane keeps its 8 * NCH elements of the row in registers between the sum of squares and the
// output, so the row is read once (the generic kernel reads it twice).
template <int NCH>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_rows_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, __nv_bfloat16* __restrict__ y,
                        float* __restrict__ rstd_out, int64_t rows, float eps) {
  constexpr int d = NCH * 256;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t row = (int64_t)blockIdx.x * 8 + warp; row < rows; row += (int64_t)gridDim.x * 8) {
    uint4 q[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) q[c] = __ldg(reinterpret_cast<const uint4*>(x + row * d + c * 256 + lane * 8));
    float ssq = 0.0f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const uint32_t* xw = reinterpret_cast<const uint32_t*>(&q[c]);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 v = unpack_bf16x2(xw[t]);
        ssq = fmaf(v.x, v.x, ssq);
        ssq = fmaf(v.y, v.y, ssq);
      }
    }
    const float rstd = rsqrtf(warp_sum(ssq) / (float)d + eps);
    if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const uint32_t* xw = reinterpret_cast<const uint32_t*>(&q[c]);
      const float4 wa = __ldg(reinterpret_cast<const float4*>(w + c * 256 + lane * 8));
      const float4 wb = __ldg(reinterpret_cast<const float4*>(w + c * 256 + lane * 8 + 4));
      const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
      uint4 o;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 v = unpack_bf16x2(xw[t]);
        ow[t] = pack_bf16x2(v.x * rstd * wv[2 * t], v.y * rstd * wv[2 * t + 1]);
      }
      *reinterpret_cast<uint4*>(y + row * d + c * 256 + lane * 8) = o;
    }
  }
}

const char* launch_rmsnorm_fwd(const __nv_bfloat16* x, const float* w, __nv_bfloat16* y, float* rstd, int64_t rows,
                               int d, float eps, cudaStream_t st) {
  if (d % 8 != 0) return "rmsnorm: d must be a multiple of 8";
  const int64_t blocks = (rows + 7) / 8;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w)) % 16 == 0 && rows > 0) {
    const int grid = (int)(blocks < 148 * 8 ? blocks : 148 * 8);
    bool done = true;
    switch (d) {
      case 256: rmsnorm_fwd_rows_kernel<1><<<grid, 256, 0, st>>>(x, w, y, rstd, rows, eps); break;
      case 512: rmsnorm_fwd_rows_kernel<2><<<grid, 256, 0, st>>>(x, w, y, rstd, rows, eps); break;
      case 1024: rmsnorm_fwd_rows_kernel<4><<<grid, 256, 0, st>>>(x, w, y, rstd, rows, eps); break;
      case 2048: rmsnorm_fwd_rows_kernel<8><<<grid, 256, 0, st>>>(x, w, y, rstd, rows, eps); break;
      default: done = false;
    }
    if (done) return cudaGetLastError() == cudaSuccess ? nullptr : "rmsnorm_fwd launch failed";
  }
  rmsnorm_fwd_kernel<<<(int)(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, st>>>(x, w, y, rstd, rows, d, eps);
  return cudaGetLastError() == cudaSuccess ? nullptr : "rmsnorm_fwd launch failed";
}

const char* launch_rmsnorm_bwd(const __nv_bfloat16* dy, const __nv_bfloat16* x, const float* w, const float* rstd,
                               __nv_bfloat16* dx, float* dw, int64_t rows, int d, cudaStream_t st) {
  if (d % 8 != 0 || d > 16384) return "rmsnorm_bwd: d must be a multiple of 8 and at most 16384";
  const int64_t blocks = (rows + 7) / 8;
  const int grid = (int)(blocks < 148 * 4 ? blocks : 148 * 4);
  auto go = [&](auto kern) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    kern<<<grid, 256, d * sizeof(float), st>>>(dy, x, w, rstd, dx, dw, rows, d);
  };
  const bool vec = (reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx)) % 16 == 0;
  if (vec && d == 1024) go(rmsnorm_bwd_kernel<4>);
  else if (vec && d == 2048) go(rmsnorm_bwd_kernel<8>);
  else if (vec && d == 512) go(rmsnorm_bwd_kernel<2>);
  else if (vec && d == 256) go(rmsnorm_bwd_kernel<1>);
  else go(rmsnorm_bwd_kernel<0>);
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
// store to the local output and to the same place in every peer copy (see QuantArgs::peer_delta)
template <typename T>
__device__ __forceinline__ void store_all(const QuantArgs& a, T* p, const T& v) {
  *p = v;
  for (int r = 0; r < a.n_peer; ++r) *reinterpret_cast<T*>(reinterpret_cast<uint8_t*>(p) + a.peer_delta[r]) = v;
}

__global__ void __launch_bounds__(256, 3)
quant_tile_kernel(const QuantArgs a) {
  pdl_enter();
  __shared__ float s_colmax[16][128];
  __shared__ float s_scale_col[128];
  __shared__ float s_tilemax;
  // e4m3 tile, transposed: row = source column, 128 bytes = the 128 source rows in 8-byte slots; the slot index
  // is XORed with a function of the row so that the 8-byte column writes spread over the banks while every
  // aligned pair of slots (16 bytes) stays contiguous for the row-wise reads
  __shared__ __align__(16) uint8_t s_q8t[128][128];

  const int tid = threadIdx.x;
  const int tr = tid >> 4;          // 0..15: this thread's rows are tr*8 .. tr*8+7
  const int tc = (tid & 15) * 8;    // first of 8 columns
  const int64_t r0 = (int64_t)blockIdx.y * 128;
  const int c0 = blockIdx.x * 128;
  const int n_cb = gridDim.x, n_rb = gridDim.y;

  float v[8][8];
  float colmax[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) colmax[i] = 0.0f;

  const int c = c0 + tc;
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const int64_t r = r0 + tr * 8 + p;
    if (r < a.rows && c < a.cols) {
      load_bf16_vec<8>(a.x + r * a.x_ld + c, v[p]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[p][i] = 0.0f;
    }
  }
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const int64_t r = r0 + tr * 8 + p;
    if (a.pre_silu) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[p][i] = __bfloat162float(__float2bfloat16(siluf_(v[p][i])));
    }
    float rmax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float av = fabsf(v[p][i]);
      rmax = fmaxf(rmax, av);
      colmax[i] = fmaxf(colmax[i], av);
    }
    if (a.q_row != nullptr && a.row_mode == QUANT_ROWS) {
      // row amax across the 16 threads that share this row
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
      const float sc = block_scale(rmax, a.pow2);
      const float inv = 1.0f / sc;
      if (r < a.rows && c < a.cols) {
        store_all(a, reinterpret_cast<uint2*>(a.q_row + r * a.q_row_ld + c), pack8_e4m3(v[p], inv));
        if ((tid & 15) == 0) {
          store_all(a, a.s_row + (int64_t)blockIdx.x * a.s_row_ld + r, sc);
          if (a.p_row != nullptr)
            store_packed_scale(a.p_row, (int64_t)blockIdx.y * a.p_row_stride + blockIdx.x, (int)(r - r0), ue8m0_word(sc));
        }
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
  const float tile_scale = block_scale(s_tilemax, a.pow2);

  if (a.q_row != nullptr && a.row_mode == QUANT_BLOCK) {
    const float inv = 1.0f / tile_scale;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      const int64_t r = r0 + tr * 8 + p;
      if (r < a.rows && c < a.cols) {
        store_all(a, reinterpret_cast<uint2*>(a.q_row + r * a.q_row_ld + c), pack8_e4m3(v[p], inv));
      }
    }
    if (tid == 0) store_all(a, a.s_row + (int64_t)blockIdx.y * n_cb + blockIdx.x, tile_scale);
    if (a.p_row != nullptr && tid < 128)
      store_all(a, reinterpret_cast<uint32_t*>(a.p_row + ((int64_t)blockIdx.y * a.p_row_stride + blockIdx.x) * 512) + tid, ue8m0_word(tile_scale));
  }

  if (a.q_col != nullptr) {
    // quantise in registers, then one 8-byte shared store per column: the thread's 8 consecutive rows of it
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int col = tc + i;
      const float sc = a.col_mode == QUANT_COLS ? block_scale(s_scale_col[col], a.pow2) : tile_scale;
      const float inv = 1.0f / sc;
      uint8_t q[8];
#pragma unroll
      for (int p = 0; p < 8; ++p) q[p] = to_e4m3(v[p][i] * inv);
      const int slot = tr ^ (((col >> 3) & 7) << 1);
      *reinterpret_cast<uint2*>(&s_q8t[col][slot * 8]) = *reinterpret_cast<uint2*>(q);
    }
    __syncthreads();
    // rows of the transposed tile leave as full 128-byte lines: 8 threads per row, 4 rows per warp and pass
    const int piece = tid & 7;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int oc = j * 32 + (tid >> 3);
      const int slot = (2 * piece) ^ (((oc >> 3) & 7) << 1);
      const uint4 u = *reinterpret_cast<const uint4*>(&s_q8t[oc][slot * 8]);
      const int64_t rr = r0 + piece * 16;
      if (c0 + oc < a.cols && rr < a.rows)
        store_all(a, reinterpret_cast<uint4*>(a.q_col + (int64_t)(c0 + oc) * a.q_col_ld + rr), u);
    }
    if (a.col_mode == QUANT_COLS) {
      if (tid < 128 && c0 + tid < a.cols) {
        const float sc_c = block_scale(s_scale_col[tid], a.pow2);
        store_all(a, a.s_col + (int64_t)blockIdx.y * a.s_col_ld + c0 + tid, sc_c);
        if (a.p_col != nullptr)
          store_packed_scale(a.p_col, (int64_t)blockIdx.x * n_rb + blockIdx.y, tid, ue8m0_word(sc_c));
      }
    } else {
      if (tid == 0) store_all(a, a.s_col + (int64_t)blockIdx.x * n_rb + blockIdx.y, tile_scale);
      if (a.p_col != nullptr && tid < 128)
        store_all(a, reinterpret_cast<uint32_t*>(a.p_col + ((int64_t)blockIdx.x * n_rb + blockIdx.y) * 512) + tid, ue8m0_word(tile_scale));
    }
  }
}

// Row-only quantiser (1x128 blocks): 16 lanes own one block of one row (8 values each), the block
// amax is a 4-step shuffle; no shared memory, every byte moved once with 16-byte loads.
__global__ void __launch_bounds__(256)
quant_rows_kernel(const QuantArgs a) {
  pdl_enter();
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
  const float sc = block_scale(m, a.pow2);
  const float inv = 1.0f / sc;
  if (!live) return;
  *reinterpret_cast<uint2*>(a.q_row + r * a.q_row_ld + c) = pack8_e4m3(v, inv);
  if ((threadIdx.x & 15) == 0) {
    a.s_row[(int64_t)(c >> 7) * a.s_row_ld + r] = sc;
    if (a.p_row != nullptr)
      store_packed_scale(a.p_row, (r >> 7) * a.p_row_stride + (c >> 7), (int)(r & 127), ue8m0_word(sc));
  }
}

const char* launch_quant_tile(const QuantArgs& a, cudaStream_t st) {
  if (a.cols % 8 != 0) return "quantise: cols must be a multiple of 8";
  if (a.n_peer > 0 && (a.q_col == nullptr || a.row_mode != QUANT_BLOCK || a.col_mode != QUANT_BLOCK))
    return "quantise: peer copies are for weights (both outputs, 128x128 blocks)";
  if (a.q_col == nullptr && a.q_row != nullptr && a.row_mode == QUANT_ROWS && a.cols % 128 == 0) {
    const int64_t threads = a.rows * (a.cols / 8);
    launch_pdl(quant_rows_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, st, a);
    return cudaGetLastError() == cudaSuccess ? nullptr : "quant_rows launch failed";
  }
  if (a.q_col != nullptr && a.rows % 16 != 0) return "quantise: transposed output needs rows % 16 == 0";
  dim3 grid((a.cols + 127) / 128, (unsigned)((a.rows + 127) / 128));
  launch_pdl(quant_tile_kernel, grid, dim3(256), 0, st, a);
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

// The same for whole 64 x 64 tiles and 16-byte aligned rows: a thread converts 16 consecutive elements (two 16-byte
// loads, one 16-byte store) and the transposed copy leaves shared memory in 16-byte pieces.
__global__ void __launch_bounds__(256)
quant_tensor_vec_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale, uint8_t* __restrict__ q_row,
                        uint8_t* __restrict__ q_col, float* __restrict__ amax_out, int64_t rows, int cols) {
  __shared__ __align__(16) uint8_t s_t[64][64 + 16];
  __shared__ float s_max[8];
  const int64_t r0 = (int64_t)blockIdx.y * 64;
  const int c0 = blockIdx.x * 64;
  const float sc = scale[0];
  const int rr = threadIdx.x >> 2, cc = (threadIdx.x & 3) * 16;
  const __nv_bfloat16* src = x + (r0 + rr) * cols + c0 + cc;
  float va[8], vb[8], v[16];
  ld8(src, va);
  ld8(src + 8, vb);
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float t = i < 8 ? va[i] : vb[i - 8];
    amax = fmaxf(amax, fabsf(t));
    v[i] = fminf(fmaxf(t * sc, -448.0f), 448.0f);
  }
  uint4 q;
  q.x = pack4_e4m3(v[0], v[1], v[2], v[3]);
  q.y = pack4_e4m3(v[4], v[5], v[6], v[7]);
  q.z = pack4_e4m3(v[8], v[9], v[10], v[11]);
  q.w = pack4_e4m3(v[12], v[13], v[14], v[15]);
  *reinterpret_cast<uint4*>(q_row + (r0 + rr) * cols + c0 + cc) = q;
  if (q_col != nullptr) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 16; ++i) s_t[cc + i][rr] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0 && amax_out != nullptr) {
    float m = 0.0f;
    for (int i = 0; i < 8; ++i) m = fmaxf(m, s_max[i]);
    atomicMax(reinterpret_cast<int*>(amax_out), __float_as_int(m));  // valid for non-negative floats
  }
  if (q_col != nullptr)   // here rr indexes the source column and cc the first of 16 source rows
    *reinterpret_cast<uint4*>(q_col + (int64_t)(c0 + rr) * rows + r0 + cc) = *reinterpret_cast<const uint4*>(&s_t[rr][cc]);
}

const char* launch_quant_tensor(const __nv_bfloat16* x, const float* scale, uint8_t* q_row, uint8_t* q_col,
                                float* amax_out, int64_t rows, int cols, cudaStream_t st) {
  dim3 grid((cols + 63) / 64, (unsigned)((rows + 63) / 64));
  const uintptr_t align = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q_row) | reinterpret_cast<uintptr_t>(q_col);
  if (rows % 64 == 0 && cols % 64 == 0 && align % 16 == 0 && q_row != nullptr) {
    quant_tensor_vec_kernel<<<grid, 256, 0, st>>>(x, scale, q_row, q_col, amax_out, rows, cols);
    return cudaGetLastError() == cudaSuccess ? nullptr : "quant_tensor launch failed";
  }
  quant_tensor_kernel<<<grid, 256, 0, st>>>(x, scale, q_row, q_col, amax_out, rows, cols);
  return cudaGetLastError() == cudaSuccess ? nullptr : "quant_tensor launch failed";
}

// =======================================================================================
// column sums: out[c] += sum_r x[r][c]
// =======================================================================================
__global__ void __launch_bounds__(256)
colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int64_t rows, int cols, int64_t ld,
              int rows_per_block) {
  pdl_enter();
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
  launch_pdl(colsum_kernel, grid, dim3(256), 0, st, x, out, rows, cols, ld, rpb);
  return cudaGetLastError() == cudaSuccess ? nullptr : "colsum launch failed";
}

// dst_s[j] += src[off_s + j] for the segments s of a table: one launch delivers the gradients of all small
// parameters of a layer step (biases, norm weights, conv taps) from one packed buffer to their places in the
// flat gradient buffer.
__global__ void __launch_bounds__(256)
segment_add_kernel(const float* __restrict__ src, const int64_t* __restrict__ dst_addr, const int* __restrict__ seg_off,
                   int n_seg, int total) {
  pdl_enter();
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= total) return;
  int s = 0;
  while (s + 1 < n_seg && seg_off[s + 1] <= i) ++s;     // a handful of segments
  float* dst = reinterpret_cast<float*>(dst_addr[s]);
  dst[i - seg_off[s]] += src[i];
}

const char* launch_segment_add(const float* src, const int64_t* dst_addr, const int* seg_off, int n_seg, int total,
                               cudaStream_t st) {
  if (n_seg < 1 || n_seg > 64) return "segment_add: between 1 and 64 segments";
  if (total <= 0) return nullptr;
  launch_pdl(segment_add_kernel, dim3((total + 255) / 256), dim3(256), 0, st, src, dst_addr, seg_off, n_seg, total);
  return cudaGetLastError() == cudaSuccess ? nullptr : "segment_add launch failed";
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
constexpr int UNSCALE_ROWS = 8;

__global__ void __launch_bounds__(256)
unscale_cols_bwd_kernel(const float* __restrict__ dW2w, const __nv_bfloat16* __restrict__ W2,
                        const float* __restrict__ colw, float* __restrict__ dW2, float* __restrict__ dcolw, int rows,
                        int cols) {
  pdl_enter();
  // 8 rows per block (64 left most SMs idle on a 1024 x 1024 matrix and made every thread a chain of 64 dependent
  // read-modify-writes); all loads of a thread are issued before the first use
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= cols) return;
  const int r_begin = blockIdx.y * UNSCALE_ROWS;
  const float wn = colw[c];
  float g[UNSCALE_ROWS], old[UNSCALE_ROWS], w[UNSCALE_ROWS];
#pragma unroll
  for (int i = 0; i < UNSCALE_ROWS; ++i) {
    const int r = r_begin + i;
    const bool live = r < rows;
    const int64_t idx = (int64_t)(live ? r : 0) * cols + c;
    g[i] = live ? dW2w[idx] : 0.0f;
    old[i] = live ? dW2[idx] : 0.0f;
    w[i] = live ? __bfloat162float(W2[idx]) : 0.0f;
  }
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < UNSCALE_ROWS; ++i) {
    const int r = r_begin + i;
    if (r < rows) dW2[(int64_t)r * cols + c] = old[i] + g[i] * wn;
    acc = fmaf(g[i], w[i], acc);
  }
  atomicAdd(dcolw + c, acc);
}

const char* launch_unscale_cols_bwd(const float* dW2w, const __nv_bfloat16* W2, const float* colw, float* dW2,
                                    float* dcolw, int rows, int cols, cudaStream_t st) {
  dim3 grid((cols + 255) / 256, (rows + UNSCALE_ROWS - 1) / UNSCALE_ROWS);
  launch_pdl(unscale_cols_bwd_kernel, grid, dim3(256), 0, st, dW2w, W2, colw, dW2, dcolw, rows, cols);
  return cudaGetLastError() == cudaSuccess ? nullptr : "unscale_cols_bwd launch failed";
}

}  // namespace gd
