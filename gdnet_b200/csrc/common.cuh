// Device-side building blocks shared by the sm_100a kernels: mbarrier, TMA (bulk tensor
// copies, never with a cluster-wide broadcast), tcgen05 (tensor-core MMA with TMEM
// accumulators), bounded waits and the status word kernels report errors through.
#pragma once

#include "quant_out.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gd {

// ---------------------------------------------------------------------------------------
// status word: kernels never trap or spin forever; they record what went wrong and return
// ---------------------------------------------------------------------------------------
enum StatusCode : int {
  STATUS_OK = 0,
  STATUS_TIMEOUT_SMEM_FULL = 1,   // consumer waited for a TMA stage that never landed
  STATUS_TIMEOUT_SMEM_EMPTY = 2,  // producer waited for a stage that was never released
  STATUS_TIMEOUT_TMEM_FULL = 3,   // epilogue waited for an accumulator that never completed
  STATUS_TIMEOUT_TMEM_EMPTY = 4,  // MMA issuer waited for an accumulator never drained
  STATUS_TIMEOUT_PEER_FLAG = 5,   // waited for a flag another rank should have written
  STATUS_BAD_ARGUMENT = 6,
};

struct Status {
  int code;      // first error (StatusCode); 0 when clean
  int site;      // kernel-specific site id
  int block;     // blockIdx.x of the reporter
  int detail;    // e.g. stage index, peer rank, sequence number
};

__device__ __forceinline__ void report(Status* st, int code, int site, int detail) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0, code) == 0) {
    st->site = site;
    st->block = (int)blockIdx.x;
    st->detail = detail;
    __threadfence_system();
  }
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Default budget for any single wait inside a kernel.
#ifndef GD_WAIT_BUDGET_NS
#define GD_WAIT_BUDGET_NS 2000000000ull
#endif

// ---------------------------------------------------------------------------------------
// flags in global memory (sequence numbers that only grow) and peer -> local gather jobs
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Orders generic-proxy accesses to global memory against bulk tensor copies (async proxy) of the same data.
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

// Bounded wait until *p >= want, written by another CTA of this GPU. false = the budget ran out.
__device__ __forceinline__ bool wait_flag_ge_gpu(const uint32_t* p, uint32_t want, uint64_t budget_ns) {
  for (int i = 0; i < 1024; ++i)
    if ((int32_t)(ld_acquire_gpu(p) - want) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    for (int i = 0; i < 128; ++i) {
      if ((int32_t)(ld_acquire_gpu(p) - want) >= 0) return true;
      __nanosleep(100);
    }
    if (globaltimer_ns() - t0 > budget_ns) return false;
  }
}

// System-scope flags: written by one GPU, read by another over NVLink.
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait until *p >= want (sequence numbers only grow). false = budget exhausted.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t want, uint64_t budget_ns = GD_WAIT_BUDGET_NS) {
  for (int i = 0; i < 2048; ++i)
    if ((int32_t)(ld_acquire_sys(p) - want) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    for (int i = 0; i < 256; ++i) {
      if ((int32_t)(ld_acquire_sys(p) - want) >= 0) return true;
      __nanosleep(200);
    }
    if (globaltimer_ns() - t0 > budget_ns) return false;
  }
}

__device__ __forceinline__ uint64_t budget_or_default(uint64_t budget_ns) {
  return budget_ns != 0 ? budget_ns : (uint64_t)GD_WAIT_BUDGET_NS;
}

// A gather job copies `n_vec` 16-byte vectors from `src` (usually another GPU's memory, read with plain
// uncached loads over NVLink) to `dst` (this GPU's memory) and then adds one to the counter `*flag` (release,
// device scope; may be null). Jobs are four int64 words each: src, dst, flag, n_vec. A range that a consumer
// waits for is cut into several jobs that share one counter, so the consumer waits for the counter to reach
// (uses so far) x (jobs per range). One warp works through jobs worker, worker + n_workers, ... with sixteen
// loads per lane in flight.
__device__ __forceinline__ void run_gather_jobs(const int64_t* __restrict__ jobs, int n_jobs, int worker,
                                                int n_workers, int lane) {
  for (int j = worker; j < n_jobs; j += n_workers) {
    const uint4* src = reinterpret_cast<const uint4*>(jobs[4 * j]);
    uint4* dst = reinterpret_cast<uint4*>(jobs[4 * j + 1]);
    uint32_t* flag = reinterpret_cast<uint32_t*>(jobs[4 * j + 2]);
    const int64_t n = jobs[4 * j + 3];
    int64_t i = lane;
    for (; i + 15 * 32 < n; i += 16 * 32) {
      uint4 v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) v[u] = __ldcv(src + i + u * 32);
#pragma unroll
      for (int u = 0; u < 16; ++u) dst[i + u * 32] = v[u];
    }
    for (; i < n; i += 32) dst[i] = __ldcv(src + i);
    __threadfence();
    fence_proxy_async_global();     // the consumer reads these bytes with bulk tensor copies
    __syncwarp();
    if (lane == 0 && flag != nullptr)
      asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(flag) : "memory");
  }
}

// ---------------------------------------------------------------------------------------
// shared memory / mbarrier
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Make generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Non-suspending variant: polls with test_wait (the thread is never parked by the hardware).
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < 100000; ++i)
    if (mbar_test_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    for (int i = 0; i < 1024; ++i)
      if (mbar_test_wait(bar, parity)) return true;
    if (globaltimer_ns() - t0 > GD_WAIT_BUDGET_NS) return false;
  }
}

// Wait for the phase with the given parity to complete. Returns false when the time
// budget ran out (the caller reports and leaves its loop); never spins forever.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < 4096; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    for (int i = 0; i < 1024; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (globaltimer_ns() - t0 > GD_WAIT_BUDGET_NS) return false;
  }
}

// Whole-warp wait with a single polling lane: 32 lanes spinning on try_wait flood the shared-memory
// pipeline and slow the one-thread producer and MMA loops that share the SM. Lane 0 polls (with a
// short back-off), the result is broadcast, and the warp reconverges before touching the data.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity) {
  uint32_t ok = 1;
  if ((threadIdx.x & 31) == 0) {
    ok = 0;
    for (int i = 0; i < 64 && !ok; ++i) ok = mbar_try_wait(bar, parity);
    if (!ok) {
      const uint64_t t0 = globaltimer_ns();
      while (!(ok = mbar_try_wait(bar, parity))) {
        __nanosleep(32);
        if (globaltimer_ns() - t0 > GD_WAIT_BUDGET_NS) break;
      }
    }
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}

// One lane of a converged warp (all 32 lanes must call it). The producer and MMA loops run warp-wide with
// uniform control flow and only the instruction that starts an asynchronous operation sits behind this
// predicate: loop counters, shared-memory addresses and descriptors then stay warp-uniform values, which the
// bulk-copy and tensor-core instructions take directly. Inside `if (lane == 0)` the same values are per-thread
// values that have to be moved over for every operand of every instruction, which made each issue cost
// 100-200 cycles of the single thread.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------
// TMA: tiled bulk tensor loads into this CTA's shared memory
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// x = innermost coordinate (elements); x * elemsize must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Tiled bulk store shared -> global (bulk-group completion). Rows and columns of the box that fall outside the
// tensor are not written. x * elemsize must be a multiple of 16 bytes and no coordinate may be negative.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Every bulk store this thread has committed has finished READING its shared-memory source.
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// All but the most recently committed bulk store of this thread have finished reading their shared-memory source.

// Per-thread asynchronous copy of 8 bytes from global to shared memory (zeros when !valid; src must still be a
// mapped address). The data is visible to the issuing thread after cp_async_wait_but<N>().
__device__ __forceinline__ void cp_async_8(void* smem_dst, const void* src, bool valid) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(smem_u32(smem_dst)), "l"(src), "r"(valid ? 8 : 0)
               : "memory");
}
// NVLink multicast (NVLS): one load returns the sum over all GPUs bound to the multicast address, added inside the
// switch; one store reaches all of them. Addresses must be 16-byte (v4.f32) or 8-byte (v2.bf16x2) aligned.
__device__ __forceinline__ float4 multimem_ld_reduce_add_f32x4(const float* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st_f32x4(float* mc_addr, const float4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void multimem_st_bf16x4(void* mc_addr, const uint2& v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.bf16x2 [%0], {%1, %2};" ::"l"(mc_addr), "r"(v.x), "r"(v.y) : "memory");
}

// The same for 16 bytes, not kept in L1.
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* src, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(src), "r"(valid ? 16 : 0)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// all of this thread's copy groups but the N most recent ones are complete
template <int N>
__device__ __forceinline__ void cp_async_wait_but() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Plain (untiled) bulk copy global -> this CTA's shared memory; both addresses 16-byte aligned,
// size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}

// ---------------------------------------------------------------------------------------
// tcgen05: TMEM allocation, MMA, commit, loads
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {  // whole warp
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void mma_fp8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Block-scaled e4m3 MMA: every 32-deep K step of A (rows) and B (rows) is multiplied by a UE8M0
// scale that the tensor core reads from TMEM (sfa/sfb), so block scaling costs no extra pass.
__device__ __forceinline__ void mma_mxfp8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate, uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

// Copy 32 rows x 16 bytes of scale factors from shared memory into 4 TMEM columns, replicated into
// all four 32-lane quarters (one 512-byte packed chunk = 128 rows x 4 K steps).
__device__ __forceinline__ void tmem_cp_scales(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Shared-memory descriptor without swizzle: rows of 16 bytes, 8-row groups sbo_bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc_noswizzle(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

// Instruction descriptor of the block-scaled MMA (e4m3 x e4m3, UE8M0 scales, K-major operands).
__host__ __device__ constexpr uint32_t make_instr_desc_mx(uint32_t M, uint32_t N, uint32_t a_sf_id, uint32_t b_sf_id) {
  return (b_sf_id << 4) | ((N >> 3) << 17) | (1u << 23) | ((M >> 4) << 24) | (a_sf_id << 29);
}

// Descriptor bits that make an MMA read byte ``k`` (0..3) of each row's 32-bit scale word, for both operands.
__host__ __device__ constexpr uint32_t mx_sf_ids(uint32_t k) { return (k << 4) | (k << 29); }

// The mbarrier receives one arrival once every MMA issued so far by this thread is done.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// ---------------------------------------------------------------------------------------
// CTA pairs (cluster of two CTAs on neighbouring SMs, tcgen05 cta_group::2)
// ---------------------------------------------------------------------------------------
// One MMA spans both CTAs: D is 256 rows (128 in each CTA's TMEM), each CTA supplies its own 128 rows of A
// and half of the N rows of B from its own shared memory, so every CTA loads half as much of B. The MMA
// is issued by the CTA of rank 0 only.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// shared::cluster address of `addr` (a shared::cta address of this CTA's layout) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {   // every thread of both CTAs
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// Tiled load into this CTA's shared memory whose completion bytes are counted on a barrier that may live
// in the other CTA of the pair (bar is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t ncols) {  // same warp of both CTAs
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void mma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Block-scaled e4m3 MMA over the CTA pair: D is 256 rows (128 per CTA); each CTA reads its scale factors from its
// own TMEM at the given column addresses.
__device__ __forceinline__ void mma_mxfp8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate, uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

// Scale-factor copy in both CTAs of the pair: each copies the chunk at this offset of its own shared memory
// into its own TMEM.
__device__ __forceinline__ void tmem_cp_scales_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// One arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair once every MMA issued so
// far by this thread is done (a signal to two barriers, not a data transfer).
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(both)
               : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp gets lane (base_lane + i),
// v[j] = column (base_col + j).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 16-byte vector reduction into global memory (local or a peer's over NVLink); no return value.
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// ---------------------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a 128-byte-swizzled tile (version 1 = sm_100).
//   K-major : rows of 128 B (one row per M/N index), 8-row groups SBO = 1024 B apart.
//   MN-major: rows of 128 B (one row per K index, 64 16-bit / 128 8-bit MN elements),
//             8-row groups SBO = 1024 B apart, next MN block LBO bytes away.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version
  d |= (uint64_t)2 << 61;  // 128-byte swizzle
  return d;
}

// Instruction descriptor: fp32 accumulate, dense, no negation.
//   fmt: kind::f16 -> 0 f16, 1 bf16; kind::f8f6f4 -> 0 e4m3, 1 e5m2.   major: 0 K, 1 MN.
__host__ __device__ constexpr uint32_t make_instr_desc(uint32_t fmt_a, uint32_t fmt_b, uint32_t a_mn, uint32_t b_mn,
                                                       uint32_t M, uint32_t N) {
  return (1u << 4) | (fmt_a << 7) | (fmt_b << 10) | (a_mn << 15) | (b_mn << 16) | ((N >> 3) << 17) |
         ((M >> 4) << 24);
}

// ---------------------------------------------------------------------------------------
// small math helpers
// ---------------------------------------------------------------------------------------
// sigmoid(x) = 0.5 + 0.5 tanh(x / 2): one special-function operation (tanh.approx, relative error about 2^-11)
// instead of two (exp and reciprocal). The fused epilogues and the gate kernels evaluate one or two sigmoids per
// element and the special-function unit issues 16 results per cycle per SM, which made it their bottleneck.
__device__ __forceinline__ float sigmoidf_(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(0.5f, t, 0.5f);
}
__device__ __forceinline__ float siluf_(float x) { return x * sigmoidf_(x); }
__device__ __forceinline__ float silu_grad_(float x) {
  const float s = sigmoidf_(x);
  return s * (1.0f + x * (1.0f - s));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 t = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(t);
}

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// Four values -> four e4m3 bytes (a in the lowest byte), two conversions of a pair each: same rounding and
// saturation as to_e4m3, half the conversion instructions and no byte shuffling.
__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// Eight values times inv -> eight e4m3 bytes as they lie in memory.
__device__ __forceinline__ uint2 pack8_e4m3(const float (&v)[8], float inv) {
  return make_uint2(pack4_e4m3(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv),
                    pack4_e4m3(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv));
}

// ---------------------------------------------------------------------------------------
// programmatic dependent launch
// ---------------------------------------------------------------------------------------
// Kernels launched through launch_pdl() (launch.h) may start while the previous kernel of the stream is still
// draining: their blocks become resident as its blocks retire and run whatever does not touch global memory
// (barrier setup, TMEM allocation). pdl_enter() is where they wait until the previous kernel has completed and
// its memory operations are visible; every thread calls it before its first global access. It then lets the
// next kernel do the same with this one. Without such a launch both instructions do nothing.
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------------------------------
// FP8 block quantisation helpers
// ---------------------------------------------------------------------------------------
// Scale of a block with the given amax: amax/448, or, for the hardware block-scaled MMA, the next
// power of two (UE8M0: the tensor core multiplies by 2^(e-127)); 1 for an all-zero block.
__device__ __forceinline__ float block_scale(float amax, int pow2) {
  if (!(amax > 0.0f)) return 1.0f;
  const float s = amax / 448.0f;
  if (!pow2) return s;
  // next power of two >= s, on the bits: exponent field + 1 unless the mantissa is zero
  const uint32_t b = __float_as_uint(s);
  uint32_t e = (b >> 23) + ((b & 0x7FFFFFu) != 0u ? 1u : 0u);
  e = e < 1u ? 1u : (e > 254u ? 254u : e);
  return __uint_as_float(e << 23);
}

// UE8M0 byte of a power-of-two scale (its biased exponent), replicated into the four bytes of a word: the
// four K steps of a 128-deep block share the scale.
__device__ __forceinline__ uint32_t ue8m0_word(float pow2_scale) {
  uint32_t e = __float_as_uint(pow2_scale) >> 23;
  e = e > 254u ? 254u : e;
  return e * 0x01010101u;
}

// Packed scale chunks for tcgen05 block-scaled MMA: 512 bytes per (128 rows, 128-deep K block);
// the four scale bytes of row r sit at (r % 32) * 16 + (r / 32) * 4.
__device__ __forceinline__ void store_packed_scale(uint8_t* packed, int64_t chunk, int row_in_128, uint32_t word) {
  *reinterpret_cast<uint32_t*>(packed + chunk * 512 + (row_in_128 & 31) * 16 + (row_in_128 >> 5) * 4) = word;
}

// 16 consecutive lanes hold the 128 values of one block of row r (8 each, this lane's start at column c; the
// values are already rounded to bf16). The 16 lanes of a group call together (the other half of the warp
// need not); `live` = this lane's row exists.
__device__ __forceinline__ void quant_emit_8(const RowQuantOut& o, const float (&v)[8], int64_t r, int c, bool live) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
  const uint32_t group = 0xffffu << (threadIdx.x & 16);
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(group, m, off));
  const float sc = block_scale(m, 1);
  const float inv = 1.0f / sc;
  if (!live) return;
  *reinterpret_cast<uint2*>(o.q + r * o.q_ld + c) = pack8_e4m3(v, inv);
  if ((threadIdx.x & 15) == 0) {
    o.s[(int64_t)(c >> 7) * o.s_ld + r] = sc;
    store_packed_scale(o.p, (r >> 7) * o.p_stride + (c >> 7), (int)(r & 127), ue8m0_word(sc));
  }
}

}  // namespace gd
