#include "comm.h"

#include "common.cuh"

namespace gd {

// ---------------------------------------------------------------------------------------
// gradient reduce-scatter + projection + AdamW + parameter all-gather
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void shard_range(int64_t n, int rank, int world, int64_t& lo, int64_t& hi) {
  int64_t per = (n + world - 1) / world;
  per = (per + 127) / 128 * 128;
  lo = (int64_t)rank * per;
  if (lo > n) lo = n;
  hi = lo + per;
  if (hi > n) hi = n;
}

// Cross-rank barrier slot `slot`: block 0 announces, every block waits for all ranks.
__device__ __forceinline__ bool rank_barrier(const FusedReduceAdamWArgs& a, int slot, uint32_t value) {
  if (a.world == 1) return true;
  if (blockIdx.x == 0 && threadIdx.x < a.world && (int)threadIdx.x != a.rank)
    st_release_sys(a.signals[threadIdx.x] + slot * a.world + a.rank, value);
  bool ok = true;
  if (threadIdx.x < a.world && (int)threadIdx.x != a.rank)
    ok = wait_flag_ge(a.signals[a.rank] + slot * a.world + threadIdx.x, value);
  if (!ok) report(a.status, STATUS_TIMEOUT_PEER_FLAG, 30 + slot, (int)threadIdx.x);
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

__global__ void __launch_bounds__(512)
fused_reduce_adamw_kernel(const FusedReduceAdamWArgs a) {
  int64_t lo, hi;
  shard_range(a.n, a.rank, a.world, lo, hi);
  // phases 0-2: the peers' buffers hold per-rank gradients and this kernel reduces them;
  // phases 3-5: the shard already holds the sum over ranks (added there by the producers' epilogues)
  const bool task_only = a.phase == 6;
  const bool scattered = a.phase >= 3 && !task_only;
  const bool do_open = a.phase == 0 || a.phase == 1 || a.phase == 3 || a.phase == 5 || task_only;
  const bool do_reduce = a.phase == 0 || a.phase == 1;
  const bool do_dots = do_open && !task_only;
  const bool do_update = a.phase == 0 || a.phase == 2 || a.phase == 4 || a.phase == 5;
  const float inv_world = 1.0f / (float)a.world;
  if (a.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0) a.timing[0] = globaltimer_ns();

  if (do_open) {
    __threadfence_system();
    // every rank's gradients are complete (the task-only pass has a flag slot of its own: it runs beside backward)
    if (!rank_barrier(a, task_only ? 2 : 0, a.seq)) return;
  }
  if (a.timing != nullptr && blockIdx.x == 0 && threadIdx.x == 0) a.timing[1] = globaltimer_ns();

  if (task_only) {
    const int64_t stride6 = (int64_t)gridDim.x * blockDim.x * 4;
    for (int64_t i = lo + ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < hi; i += stride6) {
      float4 T = make_float4(0, 0, 0, 0);
      if (a.gt_mc != nullptr) {
        T = multimem_ld_reduce_add_f32x4(a.gt_mc + i);
      } else {
        for (int r = 0; r < a.world; ++r) {
          const int peer = (a.rank + r) % a.world;
          const float4 t = *reinterpret_cast<const float4*>(a.gt[peer] + i);
          T.x += t.x; T.y += t.y; T.z += t.z; T.w += t.w;
        }
      }
      T.x *= inv_world; T.y *= inv_world; T.z *= inv_world; T.w *= inv_world;
      *reinterpret_cast<float4*>(a.t_red + (i - lo)) = T;
    }
    return;
  }

  const float coef = a.scalars[0], gscale = a.scalars[1];
  const float k_t = (1.0f - a.beta_proj * coef) * gscale, k_i = a.beta_proj * gscale;
  const float decay = 1.0f - a.lr * a.weight_decay, step = a.lr / a.bc1, inv_bc2 = 1.0f / a.bc2;
  float s_tt = 0.0f, s_ti = 0.0f, s_ii = 0.0f;

  const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
  for (int64_t i = lo + ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < hi; i += stride) {
    float4 T, I;
    if (do_reduce) {
      T = make_float4(0, 0, 0, 0);
      I = make_float4(0, 0, 0, 0);
      if (a.t_red != nullptr) {        // the task gradient of this shard was reduced while backward ran
        if (a.gi_mc != nullptr) {
          I = multimem_ld_reduce_add_f32x4(a.gi_mc + i);
        } else {
          for (int r = 0; r < a.world; ++r) {
            const int peer = (a.rank + r) % a.world;
            const float4 f = *reinterpret_cast<const float4*>(a.gi[peer] + i);
            I.x += f.x; I.y += f.y; I.z += f.z; I.w += f.w;
          }
        }
        T = *reinterpret_cast<const float4*>(a.t_red + (i - lo));
      } else if (a.gt_mc != nullptr && a.gi_mc != nullptr) {
        T = multimem_ld_reduce_add_f32x4(a.gt_mc + i);
        I = multimem_ld_reduce_add_f32x4(a.gi_mc + i);
        T.x *= inv_world; T.y *= inv_world; T.z *= inv_world; T.w *= inv_world;
      } else {
        for (int r = 0; r < a.world; ++r) {
          const int peer = (a.rank + r) % a.world;   // start at the local copy, spread peers
          const float4 t = *reinterpret_cast<const float4*>(a.gt[peer] + i);
          const float4 f = *reinterpret_cast<const float4*>(a.gi[peer] + i);
          T.x += t.x; T.y += t.y; T.z += t.z; T.w += t.w;
          I.x += f.x; I.y += f.y; I.z += f.z; I.w += f.w;
        }
        T.x *= inv_world; T.y *= inv_world; T.z *= inv_world; T.w *= inv_world;
      }
      I.x *= inv_world; I.y *= inv_world; I.z *= inv_world; I.w *= inv_world;
      s_tt += T.x * T.x + T.y * T.y + T.z * T.z + T.w * T.w;
      s_ti += T.x * I.x + T.y * I.y + T.z * I.z + T.w * I.w;
      s_ii += I.x * I.x + I.y * I.y + I.z * I.z + I.w * I.w;
      if (!do_update) {
        *reinterpret_cast<float4*>(a.gt[a.rank] + i) = T;
        *reinterpret_cast<float4*>(a.gi[a.rank] + i) = I;
      }
    } else {
      T = *reinterpret_cast<const float4*>(a.gt[a.rank] + i);
      I = *reinterpret_cast<const float4*>(a.gi[a.rank] + i);
      if (scattered) {
        T.x *= inv_world; T.y *= inv_world; T.z *= inv_world; T.w *= inv_world;
        I.x *= inv_world; I.y *= inv_world; I.z *= inv_world; I.w *= inv_world;
        if (do_dots) {
          s_tt += T.x * T.x + T.y * T.y + T.z * T.z + T.w * T.w;
          s_ti += T.x * I.x + T.y * I.y + T.z * I.z + T.w * I.w;
          s_ii += I.x * I.x + I.y * I.y + I.z * I.z + I.w * I.w;
        }
        if (do_update) {   // the shard is consumed: clear it for the next step's remote additions
          *reinterpret_cast<float4*>(a.gt[a.rank] + i) = make_float4(0, 0, 0, 0);
          *reinterpret_cast<float4*>(a.gi[a.rank] + i) = make_float4(0, 0, 0, 0);
        }
      }
    }
    if (do_update) {
      const float g[4] = {k_t * T.x + k_i * I.x, k_t * T.y + k_i * I.y, k_t * T.z + k_i * I.z, k_t * T.w + k_i * I.w};
      const int64_t j = i - lo;
      float4 mm = *reinterpret_cast<float4*>(a.m + j), vv = *reinterpret_cast<float4*>(a.v + j);
      float mo[4] = {mm.x, mm.y, mm.z, mm.w}, vo[4] = {vv.x, vv.y, vv.z, vv.w}, upd[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        mo[q] = a.beta1 * mo[q] + (1.0f - a.beta1) * g[q];
        vo[q] = a.beta2 * vo[q] + (1.0f - a.beta2) * g[q] * g[q];
        upd[q] = step * mo[q] / (sqrtf(vo[q] * inv_bc2) + a.eps);
      }
      *reinterpret_cast<float4*>(a.m + j) = make_float4(mo[0], mo[1], mo[2], mo[3]);
      *reinterpret_cast<float4*>(a.v + j) = make_float4(vo[0], vo[1], vo[2], vo[3]);
      if (a.p_is_bf16) {
        __nv_bfloat16* pl = reinterpret_cast<__nv_bfloat16*>(a.p[a.rank]) + i;
        const uint2 old = *reinterpret_cast<const uint2*>(pl);
        const float2 p01 = unpack_bf16x2(old.x), p23 = unpack_bf16x2(old.y);
        const uint2 nw = make_uint2(pack_bf16x2(p01.x * decay - upd[0], p01.y * decay - upd[1]),
                                    pack_bf16x2(p23.x * decay - upd[2], p23.y * decay - upd[3]));
        const int n_dst = a.gather_params ? a.world : 1;
        if (a.p_mc != nullptr && a.gather_params) {
          multimem_st_bf16x4(reinterpret_cast<__nv_bfloat16*>(a.p_mc) + i, nw);
        } else {
          for (int r = 0; r < n_dst; ++r) {
            const int peer = (a.rank + r) % a.world;
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.p[peer]) + i) = nw;
          }
        }
      } else {
        float* pl = reinterpret_cast<float*>(a.p[a.rank]) + i;
        const float4 old = *reinterpret_cast<const float4*>(pl);
        const float4 nw = make_float4(old.x * decay - upd[0], old.y * decay - upd[1], old.z * decay - upd[2],
                                      old.w * decay - upd[3]);
        const int n_dst = a.gather_params ? a.world : 1;
        if (a.p_mc != nullptr && a.gather_params) {
          multimem_st_f32x4(reinterpret_cast<float*>(a.p_mc) + i, nw);
        } else {
          for (int r = 0; r < n_dst; ++r) {
            const int peer = (a.rank + r) % a.world;
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.p[peer]) + i) = nw;
          }
        }
      }
    }
  }

  if (do_dots) {
    __shared__ float red[3][16];
    s_tt = warp_sum(s_tt); s_ti = warp_sum(s_ti); s_ii = warp_sum(s_ii);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { red[0][warp] = s_tt; red[1][warp] = s_ti; red[2][warp] = s_ii; }
    __syncthreads();
    if (threadIdx.x < 3) {
      float s = 0.0f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += red[threadIdx.x][w];
      atomicAdd(a.shard_sums + threadIdx.x, s);
    }
  }

  if (a.timing != nullptr && threadIdx.x == 0) atomicMax(a.timing + 2, (unsigned long long)globaltimer_ns());
  if (do_update && a.world > 1) {
    // closing barrier: the last block to finish tells every peer that this rank's parameter
    // writes are done, then waits until every peer has said the same
    __threadfence_system();
    __syncthreads();
    __shared__ int is_last;
    if (threadIdx.x == 0) {
      const unsigned prev = atomicAdd(reinterpret_cast<unsigned*>(a.shard_sums + 4), 1u);
      is_last = (prev == gridDim.x - 1);
    }
    __syncthreads();
    if (is_last) {
      if (threadIdx.x == 0) *reinterpret_cast<unsigned*>(a.shard_sums + 4) = 0u;
      if (threadIdx.x < a.world && (int)threadIdx.x != a.rank) {
        st_release_sys(a.signals[threadIdx.x] + 1 * a.world + a.rank, a.seq);
        if (!wait_flag_ge(a.signals[a.rank] + 1 * a.world + threadIdx.x, a.seq))
          report(a.status, STATUS_TIMEOUT_PEER_FLAG, 33, (int)threadIdx.x);
      }
      __syncthreads();
      if (a.timing != nullptr && threadIdx.x == 0) a.timing[3] = globaltimer_ns();
    }
  }
}

const char* launch_fused_reduce_adamw(const FusedReduceAdamWArgs& a, cudaStream_t st) {
  if (a.world < 1 || a.world > 16) return "fused_reduce_adamw: world size must be in [1, 16]";
  if (a.n % 4 != 0) return "fused_reduce_adamw: n must be a multiple of 4";
  int64_t lo = 0, per = (a.n + a.world - 1) / a.world;
  per = (per + 127) / 128 * 128;
  (void)lo;
  int64_t blocks = (per / 4 + 511) / 512;
  if (blocks > 148 * 2) blocks = 148 * 2;
  if (a.phase == 6 && blocks > 32) blocks = 32;    // runs beside the second backward pass: leave it the SMs
  if (a.phase == 6 && a.t_red == nullptr) return "fused_reduce_adamw: the task-only pass needs t_red";
  if (blocks < 1) blocks = 1;
  fused_reduce_adamw_kernel<<<(unsigned)blocks, 512, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "fused_reduce_adamw launch failed";
}

// ---------------------------------------------------------------------------------------
// add a local gradient into the flat buffers of the ranks that own its range
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
peer_add_kernel(const PeerAddArgs a) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= a.n) return;
  float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  const int cnt = (a.n - i) < 4 ? (int)(a.n - i) : 4;
  for (int q = 0; q < cnt; ++q)
    v[q] = a.src_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.src)[i + q])
                      : reinterpret_cast<const float*>(a.src)[i + q];
  const int64_t idx = a.flat_off + i;                 // flat_off and shard_elems are multiples of 4
  float* dst = a.table[idx / a.shard_elems] + idx;
  if (cnt == 4) {
    red_add_v4(dst, v[0], v[1], v[2], v[3]);
  } else {
    for (int q = 0; q < cnt; ++q) atomicAdd(dst + q, v[q]);
  }
}

const char* launch_peer_add(const PeerAddArgs& a, cudaStream_t st) {
  if (a.n <= 0) return nullptr;
  if (a.flat_off % 4 != 0 || a.shard_elems % 4 != 0) return "peer_add: offsets must be multiples of 4 elements";
  const int64_t blocks = (a.n + 1023) / 1024;
  peer_add_kernel<<<(unsigned)blocks, 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "peer_add launch failed";
}

// ---------------------------------------------------------------------------------------
// one-shot MAX all-reduce of a small vector
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
max_allreduce_kernel(const MaxAllReduceArgs a) {
  // push: this rank's vector into slot `rank` of every rank's area (its own included). Two sets of slots
  // alternate with the sequence number: a rank may already be pushing call k+1 while a slower one still reads
  // call k, but it cannot reach call k+2 before every rank has started k+1, i.e. finished reading k.
  const size_t set = (size_t)(a.seq & 1u) * a.world * a.slot_elems;
  for (int r = 0; r < a.world; ++r) {
    float* dst = a.areas[r] + set + (size_t)a.rank * a.slot_elems;
    for (int i = threadIdx.x; i < a.n; i += blockDim.x) dst[i] = a.vec[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < a.world) st_release_sys(a.flags[threadIdx.x] + a.rank, a.seq);
  __shared__ int ok_all;
  if (threadIdx.x == 0) ok_all = 1;
  __syncthreads();
  if (threadIdx.x < a.world) {
    if (!wait_flag_ge(a.flags[a.rank] + threadIdx.x, a.seq, budget_or_default(a.budget_ns))) {
      report(a.status, STATUS_TIMEOUT_PEER_FLAG, 50, (int)threadIdx.x);
      ok_all = 0;
    }
  }
  __syncthreads();
  if (!ok_all) return;      // the vector keeps this rank's own values
  const float* mine = a.areas[a.rank] + set;
  if (a.gather_out != nullptr) {     // all-gather: every rank's vector, in rank order
    for (int r = 0; r < a.world; ++r)
      for (int i = threadIdx.x; i < a.n; i += blockDim.x) a.gather_out[(size_t)r * a.n + i] = __ldcv(mine + (size_t)r * a.slot_elems + i);
    return;
  }
  for (int i = threadIdx.x; i < a.n; i += blockDim.x) {
    float m = __ldcv(mine + i);
    for (int r = 1; r < a.world; ++r) m = fmaxf(m, __ldcv(mine + (size_t)r * a.slot_elems + i));
    a.vec[i] = m;
  }
}

const char* launch_max_allreduce(const MaxAllReduceArgs& a, cudaStream_t st) {
  if (a.world < 1 || a.world > 64) return "max_allreduce: world size must be in [1, 64]";
  if (a.n > a.slot_elems) return "max_allreduce: vector longer than a slot";
  max_allreduce_kernel<<<1, 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "max_allreduce launch failed";
}

// ---------------------------------------------------------------------------------------
// neighbour exchange for sequence parallelism
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
halo_push_wait_kernel(const HaloArgs a) {
  const int dst = a.reverse ? a.rank - 1 : a.rank + 1;   // rank that receives my tail
  const int src = a.reverse ? a.rank + 1 : a.rank - 1;   // rank whose tail I receive
  const int64_t nvec = a.nbytes / 16;
  if (dst >= 0 && dst < a.world) {
    const uint4* from = reinterpret_cast<const uint4*>(a.tail);
    uint4* to = reinterpret_cast<uint4*>(a.slots[dst] + a.slot_offset);
    for (int64_t i = threadIdx.x; i < nvec; i += blockDim.x) to[i] = from[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(a.flags[dst] + a.flag_index, a.seq);
  }
  uint4* out = reinterpret_cast<uint4*>(a.halo_out);
  if (src >= 0 && src < a.world) {
    __shared__ int ok;
    if (threadIdx.x == 0) {
      ok = wait_flag_ge(a.flags[a.rank] + a.flag_index, a.seq, budget_or_default(a.budget_ns)) ? 1 : 0;
      if (!ok) report(a.status, STATUS_TIMEOUT_PEER_FLAG, 40, src);
    }
    __syncthreads();
    const uint4* mine = reinterpret_cast<const uint4*>(a.slots[a.rank] + a.slot_offset);
    for (int64_t i = threadIdx.x; i < nvec; i += blockDim.x)
      out[i] = ok ? __ldcv(mine + i) : make_uint4(0, 0, 0, 0);
  } else {
    for (int64_t i = threadIdx.x; i < nvec; i += blockDim.x) out[i] = make_uint4(0, 0, 0, 0);
  }
}

const char* launch_halo_push_wait(const HaloArgs& a, cudaStream_t st) {
  if (a.nbytes % 16 != 0) return "halo exchange: message must be a multiple of 16 bytes";
  halo_push_wait_kernel<<<1, 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? nullptr : "halo_push_wait launch failed";
}

}  // namespace gd
