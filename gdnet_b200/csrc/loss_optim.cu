// Cross-entropy, fused CAM read, gradient projection + AdamW, batched matrix-vector products.
#include "kernels.h"

#include "common.cuh"

namespace gd {

// =======================================================================================
// cross-entropy: one block per row, online softmax over the first `vocab` columns
// =======================================================================================
__global__ void __launch_bounds__(256)
cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                     float* __restrict__ row_loss, const float* __restrict__ inv_count, int vocab, int64_t ld,
                     int ignore_index, float grad_scale, int write_grad, Status* status) {
  __shared__ float red[8];
  __shared__ float s_max, s_sum;
  const int64_t row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const int64_t tgt = targets[row];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // a target outside [0, vocab) that is not the ignore index is never used as an index: the row counts as
  // ignored (loss 0, gradient 0) and the status word records it for the host
  const bool out_of_range = tgt != ignore_index && (tgt < 0 || tgt >= vocab);
  if (out_of_range && threadIdx.x == 0) report(status, STATUS_BAD_ARGUMENT, 60, (int)row);
  const bool ignored = tgt == ignore_index || out_of_range;

  if (ignored && !write_grad) {
    if (threadIdx.x == 0) row_loss[row] = 0.0f;
    return;
  }

  // pass 1: running max and rescaled sum (8 columns per thread per step; vocab % 8 handled scalar)
  float mx = -INFINITY, sm = 0.0f;
  const int vec_end = vocab & ~7;
  for (int c = threadIdx.x * 8; c < vec_end; c += 256 * 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(lr + c);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    float v[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack_bf16x2(w[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
    float lm = v[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) lm = fmaxf(lm, v[i]);
    if (lm > mx) {
      sm *= __expf(mx - lm);
      mx = lm;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sm += __expf(v[i] - mx);
  }
  for (int c = vec_end + threadIdx.x; c < vocab; c += 256) {
    const float v = __bfloat162float(lr[c]);
    if (v > mx) {
      sm *= __expf(mx - v);
      mx = v;
    }
    sm += __expf(v - mx);
  }
  // block reduce (max, then sum rescaled to the block max)
  float wm = warp_max(mx);
  if (lane == 0) red[warp] = wm;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    s_max = m;
  }
  __syncthreads();
  const float bmax = s_max;
  float contrib = (mx == -INFINITY) ? 0.0f : sm * __expf(mx - bmax);
  contrib = warp_sum(contrib);
  __syncthreads();
  if (lane == 0) red[warp] = contrib;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.0f;
    for (int i = 0; i < 8; ++i) s += red[i];
    s_sum = s;
  }
  __syncthreads();
  const float lse = bmax + __logf(s_sum);
  if (threadIdx.x == 0) row_loss[row] = ignored ? 0.0f : (lse - __bfloat162float(lr[tgt]));
  if (!write_grad) return;

  // pass 2: d loss / d logits, in place
  const float gs = ignored ? 0.0f : grad_scale * inv_count[0];
  const int64_t ldp = ld;
  for (int c = threadIdx.x * 8; c < (int)ldp; c += 256 * 8) {
    if (c + 8 <= vocab) {
      const uint4 u = *reinterpret_cast<const uint4*>(lr + c);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack_bf16x2(w[i]);
        float a = __expf(f.x - lse), b = __expf(f.y - lse);
        if (c + 2 * i == tgt) a -= 1.0f;
        if (c + 2 * i + 1 == tgt) b -= 1.0f;
        o[i] = pack_bf16x2(a * gs, b * gs);
      }
      *reinterpret_cast<uint4*>(lr + c) = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
      for (int j = c; j < c + 8 && j < (int)ldp; ++j) {
        float g = 0.0f;
        if (j < vocab) {
          g = __expf(__bfloat162float(lr[j]) - lse);
          if (j == tgt) g -= 1.0f;
          g *= gs;
        }
        lr[j] = __float2bfloat16(g);
      }
    }
  }
}

const char* launch_cross_entropy(__nv_bfloat16* logits, const int64_t* targets, float* row_loss,
                                 const float* inv_count, int64_t rows, int vocab, int64_t ld, int ignore_index,
                                 float grad_scale, int write_grad, Status* status, cudaStream_t st) {
  if (ld % 8 != 0) return "cross_entropy: row pitch must be a multiple of 8";
  if (rows == 0) return nullptr;
  cross_entropy_kernel<<<(unsigned)rows, 256, 0, st>>>(logits, targets, row_loss, inv_count, vocab, ld, ignore_index,
                                                       grad_scale, write_grad, status);
  return cudaGetLastError() == cudaSuccess ? nullptr : "cross_entropy launch failed";
}

// =======================================================================================
// fused CAM read: sim = <tags,q> + alpha <e,gamma>; w = softmax(sim); out = w . vals
// one block (128 threads) per batch row; S <= 1024
// =======================================================================================
__global__ void __launch_bounds__(128)
mem_read_fwd_kernel(const float* __restrict__ q, const float* __restrict__ gamma, const float* __restrict__ e,
                    const float* __restrict__ tags, const float* __restrict__ vals, const float* __restrict__ alpha,
                    float* __restrict__ w, float* __restrict__ out, int S, int dsig, int dc) {
  extern __shared__ float sm[];  // [S] similarities / weights
  __shared__ float s_red[4];
  const int b = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float al = alpha[0];
  const float* qb = q + (int64_t)b * dsig;
  const float* gb = gamma + (int64_t)b * dsig;
  for (int s = warp; s < S; s += 4) {
    const float* tg = tags + ((int64_t)b * S + s) * dsig;
    const float* es = e + (int64_t)s * dsig;
    float a0 = 0.0f, a1 = 0.0f;
    for (int i = lane; i < dsig; i += 32) {
      a0 = fmaf(tg[i], qb[i], a0);
      a1 = fmaf(es[i], gb[i], a1);
    }
    a0 = warp_sum(a0);
    a1 = warp_sum(a1);
    if (lane == 0) sm[s] = a0 + al * a1;
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int s = threadIdx.x; s < S; s += 128) mx = fmaxf(mx, sm[s]);
  mx = warp_max(mx);
  if (lane == 0) s_red[warp] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
  __syncthreads();
  float sum = 0.0f;
  for (int s = threadIdx.x; s < S; s += 128) {
    const float ex = __expf(sm[s] - mx);
    sm[s] = ex;
    sum += ex;
  }
  sum = warp_sum(sum);
  if (lane == 0) s_red[warp] = sum;
  __syncthreads();
  const float inv = 1.0f / (s_red[0] + s_red[1] + s_red[2] + s_red[3]);
  for (int s = threadIdx.x; s < S; s += 128) {
    const float ws = sm[s] * inv;
    sm[s] = ws;
    w[(int64_t)b * S + s] = ws;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < dc; j += 128) {
    float acc = 0.0f;
    for (int s = 0; s < S; ++s) acc = fmaf(sm[s], vals[((int64_t)b * S + s) * dc + j], acc);
    out[(int64_t)b * dc + j] = acc;
  }
}

// Backward; d_e and d_alpha are accumulated across batch rows with atomics (both zeroed by the caller).
__global__ void __launch_bounds__(128)
mem_read_bwd_kernel(const float* __restrict__ d_out, const float* __restrict__ q, const float* __restrict__ gamma,
                    const float* __restrict__ e, const float* __restrict__ tags, const float* __restrict__ vals,
                    const float* __restrict__ w, const float* __restrict__ alpha, float* __restrict__ d_q,
                    float* __restrict__ d_gamma, float* __restrict__ d_e, float* __restrict__ d_tags,
                    float* __restrict__ d_vals, float* __restrict__ d_alpha, int S, int dsig, int dc) {
  extern __shared__ float sm[];  // [S] d_w then d_sim, [S] sim_pos
  float* dsim = sm;
  float* simpos = sm + S;
  __shared__ float s_red[4];
  const int b = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float al = alpha[0];
  const float* wb = w + (int64_t)b * S;
  const float* dob = d_out + (int64_t)b * dc;
  const float* qb = q + (int64_t)b * dsig;
  const float* gb = gamma + (int64_t)b * dsig;

  for (int s = warp; s < S; s += 4) {
    const float* vs = vals + ((int64_t)b * S + s) * dc;
    float* dvs = d_vals + ((int64_t)b * S + s) * dc;
    const float ws = wb[s];
    float acc = 0.0f;
    for (int j = lane; j < dc; j += 32) {
      acc = fmaf(vs[j], dob[j], acc);
      dvs[j] = ws * dob[j];
    }
    acc = warp_sum(acc);
    const float* es = e + (int64_t)s * dsig;
    float sp = 0.0f;
    for (int i = lane; i < dsig; i += 32) sp = fmaf(es[i], gb[i], sp);
    sp = warp_sum(sp);
    if (lane == 0) {
      dsim[s] = acc;  // d_w
      simpos[s] = sp;
    }
  }
  __syncthreads();
  float dot = 0.0f;
  for (int s = threadIdx.x; s < S; s += 128) dot = fmaf(wb[s], dsim[s], dot);
  dot = warp_sum(dot);
  if (lane == 0) s_red[warp] = dot;
  __syncthreads();
  dot = s_red[0] + s_red[1] + s_red[2] + s_red[3];
  __syncthreads();
  float dal = 0.0f;
  for (int s = threadIdx.x; s < S; s += 128) {
    const float ds = wb[s] * (dsim[s] - dot);
    dsim[s] = ds;
    dal = fmaf(ds, simpos[s], dal);
  }
  dal = warp_sum(dal);
  if (lane == 0) s_red[warp] = dal;
  __syncthreads();
  if (threadIdx.x == 0) atomicAdd(d_alpha, s_red[0] + s_red[1] + s_red[2] + s_red[3]);

  for (int i = threadIdx.x; i < dsig; i += 128) {
    float dq = 0.0f, dg = 0.0f;
    const float qi = qb[i], gi = gb[i];
    for (int s = 0; s < S; ++s) {
      const float ds = dsim[s];
      dq = fmaf(ds, tags[((int64_t)b * S + s) * dsig + i], dq);
      dg = fmaf(ds, e[(int64_t)s * dsig + i], dg);
      d_tags[((int64_t)b * S + s) * dsig + i] = ds * qi;
      atomicAdd(d_e + (int64_t)s * dsig + i, al * ds * gi);
    }
    d_q[(int64_t)b * dsig + i] = dq;
    d_gamma[(int64_t)b * dsig + i] = al * dg;
  }
}

const char* launch_mem_read_fwd(const float* q, const float* gamma, const float* e, const float* tags,
                                const float* vals, const float* alpha, float* w, float* out, int B, int S, int dsig,
                                int dc, cudaStream_t st) {
  if (S > 4096) return "mem_read: at most 4096 slots";
  mem_read_fwd_kernel<<<B, 128, S * sizeof(float), st>>>(q, gamma, e, tags, vals, alpha, w, out, S, dsig, dc);
  return cudaGetLastError() == cudaSuccess ? nullptr : "mem_read_fwd launch failed";
}

const char* launch_mem_read_bwd(const float* d_out, const float* q, const float* gamma, const float* e,
                                const float* tags, const float* vals, const float* w, const float* alpha, float* d_q,
                                float* d_gamma, float* d_e, float* d_tags, float* d_vals, float* d_alpha, int B, int S,
                                int dsig, int dc, cudaStream_t st) {
  if (S > 4096) return "mem_read: at most 4096 slots";
  mem_read_bwd_kernel<<<B, 128, 2 * S * sizeof(float), st>>>(d_out, q, gamma, e, tags, vals, w, alpha, d_q, d_gamma,
                                                             d_e, d_tags, d_vals, d_alpha, S, dsig, dc);
  return cudaGetLastError() == cudaSuccess ? nullptr : "mem_read_bwd launch failed";
}

// =======================================================================================
// gradient dots and projected AdamW over flat fp32 gradient buffers
// =======================================================================================
__global__ void __launch_bounds__(256)
grad_dots_kernel(const float* __restrict__ gt, const float* __restrict__ gi, float* __restrict__ sums, int64_t n) {
  __shared__ float red[3][8];
  float a = 0.0f, b = 0.0f, c = 0.0f;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      const float4 t = *reinterpret_cast<const float4*>(gt + i);
      const float4 f = gi ? *reinterpret_cast<const float4*>(gi + i) : make_float4(0, 0, 0, 0);
      a += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
      b += t.x * f.x + t.y * f.y + t.z * f.z + t.w * f.w;
      c += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
    } else {
      for (int64_t j = i; j < n; ++j) {
        const float t = gt[j], f = gi ? gi[j] : 0.0f;
        a += t * t; b += t * f; c += f * f;
      }
    }
  }
  a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { red[0][warp] = a; red[1][warp] = b; red[2][warp] = c; }
  __syncthreads();
  if (threadIdx.x < 3) {
    float s = 0.0f;
    for (int i = 0; i < 8; ++i) s += red[threadIdx.x][i];
    atomicAdd(sums + threadIdx.x, s);
  }
}

const char* launch_grad_dots(const float* gt, const float* gi, float* sums, int64_t n, cudaStream_t st) {
  if (n == 0) return nullptr;
  if ((reinterpret_cast<uintptr_t>(gt) & 15) || (gi && (reinterpret_cast<uintptr_t>(gi) & 15)))
    return "grad_dots: buffers must be 16-byte aligned";
  int64_t blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  grad_dots_kernel<<<(unsigned)blocks, 256, 0, st>>>(gt, gi, sums, n);
  return cudaGetLastError() == cudaSuccess ? nullptr : "grad_dots launch failed";
}

__global__ void __launch_bounds__(256)
projected_adamw_kernel(const AdamWArgs a) {
  const float coef = a.scalars[0], gscale = a.scalars[1];
  const float k_t = (1.0f - a.beta_proj * coef) * gscale;  // g = k_t * gt + k_i * gi
  const float k_i = a.beta_proj * gscale;
  const float decay = 1.0f - a.lr * a.weight_decay;
  const float step = a.lr / a.bc1;
  const float inv_bc2 = 1.0f / a.bc2;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += stride) {
    const float g = k_t * a.gt[i] + (a.gi ? k_i * a.gi[i] : 0.0f);
    const float m = a.beta1 * a.m[i] + (1.0f - a.beta1) * g;
    const float v = a.beta2 * a.v[i] + (1.0f - a.beta2) * g * g;
    a.m[i] = m;
    a.v[i] = v;
    const float upd = step * m / (sqrtf(v * inv_bc2) + a.eps);
    if (a.p_bf16 != nullptr) {
      const float p = __bfloat162float(a.p_bf16[i]);
      a.p_bf16[i] = __float2bfloat16(p * decay - upd);
    } else {
      a.p_f32[i] = a.p_f32[i] * decay - upd;
    }
  }
}

const char* launch_projected_adamw(const AdamWArgs& a, cudaStream_t st) {
  if (a.n == 0) return nullptr;
  if ((a.p_bf16 == nullptr) == (a.p_f32 == nullptr)) return "adamw: exactly one parameter buffer must be given";
  int64_t blocks = (a.n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  projected_adamw_kernel<<<(unsigned)blocks, 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "projected_adamw launch failed";
}

// =======================================================================================
// batched y = W v (one warp per output row); matrices bf16 or fp32, row-major
// =======================================================================================
__global__ void __launch_bounds__(256)
batched_gemv_kernel(const void* const* __restrict__ mats, const float* const* __restrict__ vecs,
                    float* const* __restrict__ outs, const int* __restrict__ rows, const int* __restrict__ cols,
                    const int* __restrict__ is_bf16) {
  const int mi = blockIdx.y;
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int R = rows[mi], C = cols[mi];
  if (r >= R) return;
  const float* v = vecs[mi];
  float acc = 0.0f;
  if (is_bf16[mi]) {
    const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(mats[mi]) + (int64_t)r * C;
    for (int c = lane * 2; c + 1 < C; c += 64) {
      const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + c));
      acc = fmaf(f.x, v[c], acc);
      acc = fmaf(f.y, v[c + 1], acc);
    }
    if ((C & 1) && lane == 0) acc = fmaf(__bfloat162float(w[C - 1]), v[C - 1], acc);
  } else {
    const float* w = reinterpret_cast<const float*>(mats[mi]) + (int64_t)r * C;
    for (int c = lane; c < C; c += 32) acc = fmaf(w[c], v[c], acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) outs[mi][r] = acc;
}

const char* launch_batched_gemv(const void* const* mats, const float* const* vecs, float* const* outs,
                                const int* rows, const int* cols, const int* is_bf16, int n_mats, int max_rows,
                                cudaStream_t st) {
  if (n_mats == 0) return nullptr;
  dim3 grid((max_rows + 7) / 8, n_mats);
  batched_gemv_kernel<<<grid, 256, 0, st>>>(mats, vecs, outs, rows, cols, is_bf16);
  return cudaGetLastError() == cudaSuccess ? nullptr : "batched_gemv launch failed";
}

// dst_i[r][c] += coef[i] * y_i[r] * v_i[c] for a batch of fp32 matrices given by pointer tables: the rank-1
// gradients of all spectral estimates in one launch (one warp per row, lanes along the columns).
__global__ void __launch_bounds__(256)
batched_outer_add_kernel(float* const* __restrict__ dsts, const float* const* __restrict__ ys,
                         const float* const* __restrict__ vecs, const float* __restrict__ coef,
                         const int* __restrict__ rows, const int* __restrict__ cols) {
  const int mi = blockIdx.y;
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int R = rows[mi], C = cols[mi];
  if (r >= R) return;
  const float a = coef[mi] * ys[mi][r];
  if (a == 0.0f) return;
  const float* v = vecs[mi];
  float* d = dsts[mi] + (int64_t)r * C;
  for (int c = lane; c < C; c += 32) d[c] = fmaf(a, v[c], d[c]);
}

const char* launch_batched_outer_add(float* const* dsts, const float* const* ys, const float* const* vecs,
                                     const float* coef, const int* rows, const int* cols, int n_mats, int max_rows,
                                     cudaStream_t st) {
  if (n_mats == 0) return nullptr;
  dim3 grid((max_rows + 7) / 8, n_mats);
  batched_outer_add_kernel<<<grid, 256, 0, st>>>(dsts, ys, vecs, coef, rows, cols);
  return cudaGetLastError() == cudaSuccess ? nullptr : "batched_outer_add launch failed";
}

// =======================================================================================
// hard spectral norm: one power iteration and sigma for one matrix, in one block
// =======================================================================================
// torch.nn.utils.spectral_norm (what the reference wraps cam.W_r1 in, gdnet/memory.py:68) does, per training forward,
//   v <- normalize(W^T u),  u <- normalize(W v),  sigma = u^T W v
// and divides the weight by sigma. The matrix is small (d x (3d+1)), so one block of 1024 threads does all of it
// without any cross-block synchronisation; rows and columns may be odd (scalar loads). u, v: fp32, updated in
// place when do_iter is set. sigma_out[0] = u^T W v with the final u, v.
template <typename T>
__device__ __forceinline__ float sn_load(const T* w, int64_t i);
template <>
__device__ __forceinline__ float sn_load<float>(const float* w, int64_t i) { return w[i]; }
template <>
__device__ __forceinline__ float sn_load<__nv_bfloat16>(const __nv_bfloat16* w, int64_t i) { return __bfloat162float(w[i]); }

__device__ __forceinline__ float block_sum_1024(float x, float* red) {
  x = warp_sum(x);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = x;
  __syncthreads();
  float t = (threadIdx.x < 32) ? red[threadIdx.x] : 0.0f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

template <typename T>
__global__ void __launch_bounds__(1024)
sn_power_iter_kernel(const T* __restrict__ W, float* __restrict__ u, float* __restrict__ v, float* __restrict__ t,
                     float* __restrict__ sigma_out, int rows, int cols, int do_iter, float eps) {
  __shared__ float red[33];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (do_iter) {
    // v = W^T u: a thread owns columns tid, tid + 1024, ... (consecutive threads read consecutive addresses)
    float ssq = 0.0f;
    for (int c = tid; c < cols; c += 1024) {
      float acc = 0.0f;
      for (int r = 0; r < rows; ++r) acc = fmaf(sn_load(W, (int64_t)r * cols + c), u[r], acc);
      v[c] = acc;
      ssq = fmaf(acc, acc, ssq);
    }
    const float nv = sqrtf(block_sum_1024(ssq, red));
    const float iv = 1.0f / fmaxf(nv, eps);
    for (int c = tid; c < cols; c += 1024) v[c] *= iv;
    __syncthreads();
  }
  // t = W v: one warp per row
  float ssq_t = 0.0f, dot_ut = 0.0f;
  for (int r = warp; r < rows; r += 32) {
    float acc = 0.0f;
    for (int c = lane; c < cols; c += 32) acc = fmaf(sn_load(W, (int64_t)r * cols + c), v[c], acc);
    acc = warp_sum(acc);
    if (lane == 0) {
      t[r] = acc;
      ssq_t = fmaf(acc, acc, ssq_t);
      dot_ut = fmaf(u[r], acc, dot_ut);
    }
  }
  const float nt = sqrtf(block_sum_1024(ssq_t, red));
  if (do_iter) {
    const float it = 1.0f / fmaxf(nt, eps);
    for (int r = tid; r < rows; r += 1024) u[r] = t[r] * it;
    // sigma = u^T W v with the new u = t / |t|
    if (tid == 0) sigma_out[0] = nt * nt * it;
  } else {
    const float s = block_sum_1024(dot_ut, red);
    if (tid == 0) sigma_out[0] = s;
  }
}

const char* launch_sn_power_iter(const void* W, int w_is_bf16, float* u, float* v, float* t, float* sigma_out, int rows,
                                 int cols, int do_iter, float eps, cudaStream_t st) {
  if (rows < 1 || cols < 1) return "sn_power_iter: empty matrix";
  if (w_is_bf16)
    sn_power_iter_kernel<__nv_bfloat16><<<1, 1024, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(W), u, v, t, sigma_out, rows,
                                                            cols, do_iter, eps);
  else
    sn_power_iter_kernel<float><<<1, 1024, 0, st>>>(reinterpret_cast<const float*>(W), u, v, t, sigma_out, rows, cols, do_iter, eps);
  return cudaGetLastError() == cudaSuccess ? nullptr : "sn_power_iter launch failed";
}

}  // namespace gd

// =======================================================================================
// allocation-free mean cross-entropy (see noalloc.h; no counterpart in the reference)
// =======================================================================================
#include "noalloc.h"

#include <atomic>

namespace gd {

// Scratch of the allocation-free entry point: [0, MAX_ROWS) per-row losses, [MAX_ROWS] unused pad.
// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_noalloc_scratch[GD_NOALLOC_MAX_ROWS + 64];

// One block: loss_out = sum(row_loss) / max(1, #targets != ignore_index). Reads every row loss the
// preceding kernel wrote (rows beyond `rows` hold stale values from earlier calls and are not read).
__global__ void __launch_bounds__(1024)
noalloc_finalize_kernel(const float* __restrict__ row_loss, const int64_t* __restrict__ targets, int64_t rows,
                        int ignore_index, int vocab, float* __restrict__ loss_out) {
  __shared__ float s_sum[32];
  __shared__ float s_cnt[32];
  float sum = 0.0f, cnt = 0.0f;
  for (int64_t r = threadIdx.x; r < rows; r += blockDim.x) {
    sum += row_loss[r];
    const int64_t t = targets[r];      // rows with a target outside [0, vocab) contribute nothing, like ignored rows
    cnt += (t != ignore_index && t >= 0 && t < vocab) ? 1.0f : 0.0f;
  }
  sum = warp_sum(sum);
  cnt = warp_sum(cnt);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { s_sum[warp] = sum; s_cnt[warp] = cnt; }
  __syncthreads();
  if (warp == 0) {
    sum = s_sum[lane];
    cnt = s_cnt[lane];
    sum = warp_sum(sum);
    cnt = warp_sum(cnt);
    if (lane == 0) loss_out[0] = sum / fmaxf(cnt, 1.0f);
  }
}

}  // namespace gd

extern "C" int gd_cross_entropy_mean_noalloc(const void* logits_bf16, const int64_t* targets, int64_t rows, int vocab,
                                             int64_t ld, int ignore_index, float* loss_out, void* stream) {
  if (rows < 0 || rows > GD_NOALLOC_MAX_ROWS) return 1;
  if (logits_bf16 == nullptr || targets == nullptr || loss_out == nullptr) return 2;
  if ((reinterpret_cast<uintptr_t>(logits_bf16) & 15) != 0 || ld % 8 != 0 || vocab < 1 || vocab > ld) return 2;

  // device address of the scratch array, looked up once per device with that device current
  // (atomic slots: host threads that make their first call on a device at the same time all store the same value)
  static std::atomic<float*> scratch_of_device[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 3;
  float* row_loss = scratch_of_device[dev].load(std::memory_order_acquire);
  if (row_loss == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), gd::g_noalloc_scratch) != cudaSuccess || p == nullptr)
      return 3;
    scratch_of_device[dev].store(p, std::memory_order_release);
    row_loss = p;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  if (rows > 0) {
    // write_grad = 0: the logits stay untouched and inv_count is not read; every row in [0, rows) is
    // overwritten, so nothing of an earlier call survives where this call looks
    gd::cross_entropy_kernel<<<(unsigned)rows, 256, 0, st>>>(
        reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(logits_bf16)), targets, row_loss, row_loss, vocab, ld,
        ignore_index, 1.0f, 0, nullptr);
    if (cudaGetLastError() != cudaSuccess) return 3;
  }
  gd::noalloc_finalize_kernel<<<1, 1024, 0, st>>>(row_loss, targets, rows, ignore_index, vocab, loss_out);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}
