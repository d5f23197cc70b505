// Tensor-core GEMMs for sm_100a: D[M,N] = A[M,K] * B[N,K]^T with fused epilogues.
//
// Two persistent, warp-specialised kernels share one structure:
//
//   warp 0      TMA producer: tiled bulk tensor loads (128-byte swizzle) into a ring of
//               shared-memory stages; one mbarrier pair (full/empty) per stage
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma with shared-memory
//               descriptors; accumulators live in tensor memory (TMEM), which this warp
//               allocates and frees; tcgen05.commit releases stages / publishes accumulators
//   warps 2..9  epilogue: tcgen05.ld the accumulator (a warp may only touch TMEM lanes
//               32*(warp%4)..+31, so two warps share a lane quarter and split the columns),
//               apply the fused epilogue, store to global memory
//
//   gemm_bf16_kernel   bf16 x bf16 -> fp32 in TMEM over the whole K; tile 128 x 256;
//                      two accumulator stages so the epilogue of a tile overlaps the
//                      main loop of the next. Operands may be K-major or MN-major (the
//                      weight-gradient GEMM reduces over tokens and reads both of its
//                      row-major operands MN-major, so nothing is transposed in memory).
//   gemm_fp8_kernel    e4m3 x e4m3 with block scales (1x128 on A rows, 128x128 on B):
//                      every 128-deep K block is a fresh accumulation in one of four
//                      TMEM stages; the epilogue warps scale it by sa[m,kb]*sb[nb,kb] and
//                      add it to fp32 registers (two-level accumulation); tile 128 x 128.
//
// Every wait is bounded (see common.cuh); on expiry the CTA records a status code,
// raises a CTA-wide abort flag, drains, frees its TMEM and returns.
#include "gemm_sm100.h"

#include <cstdlib>

#include "common.cuh"
#include "launch.h"

namespace gd {

constexpr int BM = 128;
constexpr int EPI_WARPS = 8;
constexpr int NUM_THREADS = 64 + EPI_WARPS * 32;
constexpr int STAGE_ROW_BYTES = 128;  // one swizzle row: 64 bf16 or 128 e4m3 along the box's inner dim

struct __align__(8) PipeBars {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[4];
  uint64_t tmem_empty[4];
  uint64_t aux_full[32];   // up to four per epilogue warp: a slice of the next tile's auxiliary input has landed
  uint32_t tmem_base;
  int abort;
};

__device__ __forceinline__ bool aborted(const PipeBars* b) { return *((volatile const int*)&b->abort) != 0; }

__device__ __forceinline__ void raise_abort(PipeBars* b, Status* st, int code, int site, int detail) {
  report(st, code, site, detail);
  *((volatile int*)&b->abort) = 1;
}

// Tile order: bands of RASTER_M row-blocks; inside a band consecutive tiles walk down the rows of one
// column block first, so CTAs that run at the same time share a handful of A and B tiles in L2
// (row-major order would stream the whole B matrix once per row block when N is large).
constexpr int RASTER_M = 8;

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& mb, int& nb) {
  const int band_tiles = RASTER_M * tiles_n;
  const int band = tile / band_tiles;
  const int in_band = tile - band * band_tiles;
  const int rows_here = min(RASTER_M, tiles_m - band * RASTER_M);
  nb = in_band / rows_here;
  mb = band * RASTER_M + (in_band - nb * rows_here);
}

// ---------------------------------------------------------------------------------------
// fused epilogue on one row x 32 columns held in registers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float load_bias(const GemmEpilogue& e, int n, int N) {
  if (e.bias == nullptr || n >= N) return 0.0f;
  return e.bias_f32 ? reinterpret_cast<const float*>(e.bias)[n]
                    : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(e.bias)[n]);
}

constexpr int AUX_BOX_BYTES = 32 * 128;

// A global load issued by an epilogue warp queues behind the bulk tensor loads the producer keeps in flight
// (several stages, microseconds of traffic), so the epilogue must not wait for one per chunk. Per-row and
// per-column vectors are fetched before the wait for the accumulator; the auxiliary matrix is fetched one
// tile ahead by bulk tensor copies into a per-warp buffer (one thread, one or two boxes per tile).
// `boxes` boxes of 32 rows x 64 bf16 columns (4 KB each, 128-byte swizzle) starting at (m_warp, nbase).
__device__ __forceinline__ bool aux_prefetch(const CUtensorMap* tmap, int M, int N, int m_warp, int lane, int nbase,
                                             int boxes, uint32_t buf, uint32_t bar) {
  if (m_warp >= M || nbase >= N) return false;     // warp-uniform
  if (lane == 0) {
    mbar_arrive_expect_tx(bar, (uint32_t)(boxes * AUX_BOX_BYTES));
    for (int b = 0; b < boxes; ++b) tma_load_2d(buf + b * AUX_BOX_BYTES, tmap, bar, nbase + b * 64, m_warp);
  }
  return true;
}

// One chunk of the auxiliary matrix (32 rows x 32 bf16 columns, 2 KB, 64-byte swizzle) into a slot of its own with
// a barrier of its own. A slot is asked for again as soon as its chunk has been consumed, so every chunk of the next
// tile has a whole tile's time to arrive (a request made only when the whole tile was done left the epilogue waiting
// out the memory latency at the start of every tile once the epilogue, not the main loop, set the pace). Rows or
// columns outside the matrix read as zero. Warp-collective.
constexpr int AUX_CHUNK_BYTES = 32 * 64;

__device__ __forceinline__ void aux_request(const CUtensorMap* tmap, int m_warp, int ncol, uint32_t slot, uint32_t bar) {
  if (elect_one()) {
    mbar_arrive_expect_tx(bar, (uint32_t)AUX_CHUNK_BYTES);
    tma_load_2d(slot, tmap, bar, ncol, m_warp);
  }
  __syncwarp();
}

__device__ __forceinline__ float row_scale_for(const GemmEpilogue& e, int m) {
  if (e.row_scale != nullptr) return e.row_scale[m];
  if (e.ssq_in != nullptr) {
    float s = 0.0f;
    for (int p = 0; p < e.ssq_parts; ++p) s += e.ssq_in[(size_t)m * e.ssq_parts + p];
    return rsqrtf(s / (float)e.norm_dim + e.norm_eps);
  }
  return 1.0f;
}

// Per-warp staging area for the bf16 side of the epilogue: 32 rows x 64 bytes. A thread owns one row of the
// accumulator, but a warp-wide store of one 16-byte piece per thread touches 32 different cache lines; the
// rows therefore go through shared memory and leave (or arrive) as 8 rows x 64 contiguous bytes per
// instruction. The 16-byte slots are XOR-swizzled so both access patterns are free of bank conflicts.
constexpr int EPI_STAGE_BYTES_PER_WARP = 32 * 64;
constexpr int EPI_STAGE_BYTES = EPI_WARPS * EPI_STAGE_BYTES_PER_WARP;

__device__ __forceinline__ uint32_t stage_off(int row, int slot) {
  return (uint32_t)(row * 64 + ((slot ^ ((row >> 1) & 3)) << 4));
}

// this lane's row (32 bf16 in w) -> global rows base[row * ld + 0..31], rows < rows_valid
// The staging area may still be the source of a bulk store issued by this warp's elected lane (store_rows_tma):
// that lane waits until the store has read it before anyone overwrites it. Warp-collective.
__device__ __forceinline__ void stage_acquire() {
  if (elect_one()) bulk_wait_read_all();
  __syncwarp();
}

// this lane's row (32 bf16, or 64 e4m3, in w) -> the box of 32 rows x 64 bytes at column x (elements), row m_warp of
// the tensor behind tmap, as one tiled bulk store: the rows are laid down in the staging area in the 64-byte-swizzle
// order and an elected lane hands them to the copy engine, so the warp neither reads them back nor issues the
// global stores itself. Rows and columns outside the tensor are clipped by the copy. Warp-collective.
__device__ __forceinline__ void store_rows_tma(uint8_t* stage, int lane, const uint32_t (&w)[16], const CUtensorMap* tmap,
                                               int x, int m_warp) {
  stage_acquire();
#pragma unroll
  for (int q = 0; q < 4; ++q)
    *reinterpret_cast<uint4*>(stage + stage_off(lane, q)) = make_uint4(w[q * 4], w[q * 4 + 1], w[q * 4 + 2], w[q * 4 + 3]);
  fence_proxy_async_smem();
  __syncwarp();
  if (elect_one()) {
    tma_store_2d(tmap, smem_u32(stage), x, m_warp);
    bulk_commit_group();
  }
  __syncwarp();
}

__device__ __forceinline__ void store_rows_bf16(uint8_t* stage, int lane, const uint32_t (&w)[16],
                                                __nv_bfloat16* base, int64_t ld, int rows_valid) {
  stage_acquire();
#pragma unroll
  for (int q = 0; q < 4; ++q)
    *reinterpret_cast<uint4*>(stage + stage_off(lane, q)) = make_uint4(w[q * 4], w[q * 4 + 1], w[q * 4 + 2], w[q * 4 + 3]);
  __syncwarp();
  const int r_in = lane >> 2, slot = lane & 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int row = r_in + 8 * j;
    const uint4 u = *reinterpret_cast<const uint4*>(stage + stage_off(row, slot));
    if (row < rows_valid) *reinterpret_cast<uint4*>(base + (size_t)row * ld + slot * 8) = u;
  }
  __syncwarp();
}

// global rows base[row * ld + 0..31] -> this lane's row in w (rows >= rows_valid read as zero)
__device__ __forceinline__ void load_rows_bf16(uint8_t* stage, int lane, uint32_t (&w)[16],
                                               const __nv_bfloat16* base, int64_t ld, int rows_valid) {
  stage_acquire();
  const int r_in = lane >> 2, slot = lane & 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int row = r_in + 8 * j;
    uint4 u = make_uint4(0, 0, 0, 0);
    if (row < rows_valid) u = *reinterpret_cast<const uint4*>(base + (size_t)row * ld + slot * 8);
    *reinterpret_cast<uint4*>(stage + stage_off(row, slot)) = u;
  }
  __syncwarp();
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint4 u = *reinterpret_cast<const uint4*>(stage + stage_off(lane, q));
    w[q * 4] = u.x; w[q * 4 + 1] = u.y; w[q * 4 + 2] = u.z; w[q * 4 + 3] = u.w;
  }
  __syncwarp();
}

// v: 32 consecutive columns starting at n0 of row m = m_warp + lane. Warp-collective (all lanes call it with
// the same n0). Returns this chunk's sum of squares of the stored values (for the RMSNorm that follows).
//
// bias_lane: the bias of column n0 + lane (0 without bias). aux_row: this lane's row inside the prefetched
// box (128 bytes, 16-byte pieces XOR-swizzled with the row number), the chunk starting at piece aux_piece0;
// null to read the auxiliary values from global memory here.
__device__ __forceinline__ float epilogue_chunk(const GemmEpilogue& e, int M, int N, int m_warp, int lane, int n0,
                                                float rs, float rowcoef, float (&v)[32], uint8_t* stage,
                                                float bias_lane, const uint8_t* aux_row, int aux_piece0,
                                                bool aux64 = false, const CUtensorMap* t_out = nullptr,
                                                const CUtensorMap* t_pre = nullptr) {
  float ssq = 0.0f;
  if (m_warp >= M || n0 >= N) return 0.0f;   // warp-uniform
  const int m = m_warp + lane;
  const int rows_valid = min(32, M - m_warp);
  if (e.bias != nullptr) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = v[j] * rs + __shfl_sync(0xffffffffu, bias_lane, j);
  } else if (e.row_scale != nullptr || e.ssq_in != nullptr) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= rs;
  }

  if (e.aux != nullptr) {
    uint32_t w[16];
    if (aux_row != nullptr) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        // aux64: a box of 32 rows x 64 bytes of its own per chunk (64-byte swizzle), aux_row = this lane's row
        const int piece = aux64 ? (q ^ ((lane >> 1) & 3)) : ((aux_piece0 + q) ^ (lane & 7));
        const uint4 u = *reinterpret_cast<const uint4*>(aux_row + (piece << 4));
        w[q * 4] = u.x; w[q * 4 + 1] = u.y; w[q * 4 + 2] = u.z; w[q * 4 + 3] = u.w;
      }
    } else {
      load_rows_bf16(stage, lane, w, e.aux + (size_t)m_warp * e.aux_ld + n0, e.aux_ld, rows_valid);
    }
    // one loop per mode (the mode is the same for the whole launch): with the test inside the loop the compiler
    // evaluated all three forms for every element and selected, so a plain add paid for two sigmoids
    if (e.aux_mode == AUX_ADD) {
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const float2 a = unpack_bf16x2(w[t]);
        v[2 * t] += a.x;
        v[2 * t + 1] += a.y;
      }
    } else if (e.aux_mode == AUX_MUL_SILU_GRAD) {
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const float2 a = unpack_bf16x2(w[t]);
        v[2 * t] *= silu_grad_(a.x);
        v[2 * t + 1] *= silu_grad_(a.y);
      }
    } else {  // AUX_RMS_SILU_BWD: (v - silu(aux) * rowcoef) * silu'(aux)
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const float2 a = unpack_bf16x2(w[t]);
        const float s0 = sigmoidf_(a.x), s1 = sigmoidf_(a.y);
        v[2 * t] = (v[2 * t] - a.x * s0 * rowcoef) * (s0 * (1.0f + a.x * (1.0f - s0)));
        v[2 * t + 1] = (v[2 * t + 1] - a.y * s1 * rowcoef) * (s1 * (1.0f + a.y * (1.0f - s1)));
      }
    }
  }

  if (e.pre_out != nullptr) {
    uint32_t w[16];
#pragma unroll
    for (int t = 0; t < 16; ++t) w[t] = pack_bf16x2(v[t * 2], v[t * 2 + 1]);
    if (t_pre != nullptr) store_rows_tma(stage, lane, w, t_pre, n0, m_warp);
    else store_rows_bf16(stage, lane, w, e.pre_out + (size_t)m_warp * e.pre_ld + n0, e.pre_ld, rows_valid);
  }

  if (e.act == ACT_SILU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = siluf_(v[j]);
  }

  if (e.out == nullptr) return 0.0f;   // only the quantised copy is wanted (written by the caller)
  if (e.out_f32) {
    if (m >= M) return 0.0f;
    float4* op = reinterpret_cast<float4*>(reinterpret_cast<float*>(e.out) + (size_t)m * e.out_ld + n0);
    if (e.peer_out != nullptr) {
      // gradient reduce-scatter from the epilogue: add this chunk into the owner rank's flat buffer
      const int64_t idx = e.flat_off + (int64_t)m * e.out_ld + n0;
      op = reinterpret_cast<float4*>(e.peer_out[idx / e.shard_elems] + idx);
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
      if (e.atomic || e.peer_out != nullptr) {   // split-K shares and peers add into the same tile
        red_add_v4(reinterpret_cast<float*>(op + q), o.x, o.y, o.z, o.w);
        continue;
      }
      if (e.accumulate) {
        const float4 old = op[q];
        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
      }
      op[q] = o;
    }
  } else {
    __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(e.out) + (size_t)m_warp * e.out_ld + n0;
    if (e.accumulate) {
      uint32_t old[16];
      load_rows_bf16(stage, lane, old, ob, e.out_ld, rows_valid);
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const float2 o = unpack_bf16x2(old[t]);
        v[t * 2] += o.x;
        v[t * 2 + 1] += o.y;
      }
    }
    uint32_t w[16];
#pragma unroll
    for (int t = 0; t < 16; ++t) w[t] = pack_bf16x2(v[t * 2], v[t * 2 + 1]);
    if (e.ssq_out != nullptr && m < M) {   // of the rounded values, as the consumer of `out` will see them
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const float2 r = unpack_bf16x2(w[t]);
        ssq += r.x * r.x + r.y * r.y;
      }
    }
    if (t_out != nullptr) store_rows_tma(stage, lane, w, t_out, n0, m_warp);
    else store_rows_bf16(stage, lane, w, ob, e.out_ld, rows_valid);
  }
  return ssq;
}

// ---------------------------------------------------------------------------------------
// shared prologue / teardown
// ---------------------------------------------------------------------------------------
template <int STAGES, int ACC_STAGES>
__device__ __forceinline__ void pipe_setup(PipeBars* bars, int warp, int lane, uint32_t tmem_cols,
                                           const CUtensorMap* ta, const CUtensorMap* tb) {
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(ta);
    tma_prefetch_desc(tb);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < ACC_STAGES; ++a) {
      mbar_init(smem_u32(&bars->tmem_full[a]), 1);
      mbar_init(smem_u32(&bars->tmem_empty[a]), EPI_WARPS);
    }
    for (int w = 0; w < EPI_WARPS; ++w) mbar_init(smem_u32(&bars->aux_full[w]), 1);
    bars->abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
}

__device__ __forceinline__ void pipe_teardown(PipeBars* bars, int warp, uint32_t tmem_cols) {
  tc_fence_before_sync();
  __syncthreads();
  if (aborted(bars)) {
    // give bulk copies that are still in flight time to land before the CTA's shared
    // memory is handed to another CTA (bounded: ~100 us)
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(bars->tmem_base, tmem_cols);
  }
}

// ---------------------------------------------------------------------------------------
// lean single-thread loops
// ---------------------------------------------------------------------------------------
// The producer and the MMA issuer are single threads: their loops are bound by the number of
// dependent instructions per K block, so everything that can be computed once is hoisted (barrier
// addresses, descriptor templates) and the time-budgeted wait lives out of line.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity) { return mbar_wait(bar, parity); }

__device__ __forceinline__ bool wait_fast(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity);
}

__device__ __forceinline__ uint64_t desc_at(uint32_t hi, uint32_t lo) {
  return ((uint64_t)hi << 32) | (uint64_t)lo;
}

// ---------------------------------------------------------------------------------------
// bf16 kernel
// ---------------------------------------------------------------------------------------
constexpr int BF16_BN = 256;
constexpr int BF16_BK = 64;
constexpr int BF16_ACC = 2;
constexpr int BF16_AUX_BYTES = EPI_WARPS * 2 * AUX_BOX_BYTES;   // two boxes (128 columns) per epilogue warp
constexpr int BF16_A_BYTES = BM * STAGE_ROW_BYTES;       // 16 KB
constexpr int BF16_B_BYTES = BF16_BN * STAGE_ROW_BYTES;  // 32 KB
constexpr int BF16_STAGE_BYTES = BF16_A_BYTES + BF16_B_BYTES;

// AUX = the epilogue reads an auxiliary matrix: one pipeline stage is given up for the per-warp prefetch buffers.
template <bool AUX>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_aux, const GemmShape g, const GemmEpilogue e, Status* status) {
  constexpr int BF16_STAGES = AUX ? 3 : 4;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_all = smem + BF16_STAGES * BF16_STAGE_BYTES;
  uint8_t* aux_all = stage_all + EPI_STAGE_BYTES;
  PipeBars* bars = reinterpret_cast<PipeBars*>(aux_all + (AUX ? BF16_AUX_BYTES : 0));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pipe_setup<BF16_STAGES, BF16_ACC>(bars, warp, lane, BF16_ACC * BF16_BN, &tmap_a, &tmap_b);
  pdl_enter();
  const uint32_t tmem_base = bars->tmem_base;

  const int n_tiles_n = (g.N + BF16_BN - 1) / BF16_BN;
  const int n_tiles_m = (g.M + BM - 1) / BM;
  const int n_tiles = n_tiles_m * n_tiles_n;
  const int kblocks = (g.K + BF16_BK - 1) / BF16_BK;
  const int kb_per = (kblocks + g.splits - 1) / g.splits;   // K blocks per split-K share
  const int n_work = n_tiles * g.splits;
  const uint32_t smem0 = smem_u32(smem);
  const uint32_t full0 = smem_u32(&bars->full[0]), empty0 = smem_u32(&bars->empty[0]);
  const uint32_t tfull0 = smem_u32(&bars->tmem_full[0]), tempty0 = smem_u32(&bars->tmem_empty[0]);

  if (warp == 0) {
    {   // all 32 lanes run the loop; one elected lane issues the loads (see elect_one)
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < n_work && ok; work += gridDim.x) {
        const int tile = work % n_tiles, kb0 = (work / n_tiles) * kb_per, kb1 = min(kblocks, kb0 + kb_per);
        int mb_, nb_;
        tile_coords(tile, n_tiles_m, n_tiles_n, mb_, nb_);
        const int m0 = mb_ * BM, n0 = nb_ * BF16_BN;
        int kx = kb0 * BF16_BK;
        for (int kb = kb0; kb < kb1; ++kb, kx += BF16_BK) {
          if (!__all_sync(0xffffffffu, wait_fast(empty0 + 8 * s, ph ^ 1))) {
            if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_SMEM_EMPTY, 10, s);
            ok = false;
            break;
          }
          const uint32_t full = full0 + 8 * s;
          const uint32_t a_dst = smem0 + s * BF16_STAGE_BYTES;
          const uint32_t b_dst = a_dst + BF16_A_BYTES;
          if (elect_one()) {
            mbar_arrive_expect_tx(full, BF16_STAGE_BYTES);
            if (!g.a_mn) {
              tma_load_2d(a_dst, &tmap_a, full, kx, m0);
            } else {
#pragma unroll
              for (int i = 0; i < BM / 64; ++i)
                tma_load_2d(a_dst + i * (BF16_BK * STAGE_ROW_BYTES), &tmap_a, full, m0 + i * 64, kx);
            }
            if (!g.b_mn) {
              tma_load_2d(b_dst, &tmap_b, full, kx, n0);
            } else {
#pragma unroll
              for (int i = 0; i < BF16_BN / 64; ++i)
                tma_load_2d(b_dst + i * (BF16_BK * STAGE_ROW_BYTES), &tmap_b, full, n0 + i * 64, kx);
            }
          }
          __syncwarp();
          if (++s == BF16_STAGES) { s = 0; ph ^= 1; }
        }
        if (aborted(bars)) break;
      }
    }
  } else if (warp == 1) {
    {   // warp-wide loop, one elected lane issues
      const uint32_t idesc = make_instr_desc(1, 1, g.a_mn ? 1 : 0, g.b_mn ? 1 : 0, BM, BF16_BN);
      const uint32_t a_lbo = g.a_mn ? BF16_BK * STAGE_ROW_BYTES : 16, b_lbo = g.b_mn ? BF16_BK * STAGE_ROW_BYTES : 16;
      // K advance per MMA (UMMA_K = 16 elements): 32 B inside the swizzle row when K-major,
      // 16 rows of 128 B when MN-major; in 16-byte units.
      const uint32_t a_step = g.a_mn ? (16 * STAGE_ROW_BYTES) >> 4 : 2, b_step = g.b_mn ? (16 * STAGE_ROW_BYTES) >> 4 : 2;
      const uint64_t a_tmpl = make_smem_desc(smem0, a_lbo, 1024), b_tmpl = make_smem_desc(smem0 + BF16_A_BYTES, b_lbo, 1024);
      const uint32_t a_hi = (uint32_t)(a_tmpl >> 32), a_lo0 = (uint32_t)a_tmpl;
      const uint32_t b_hi = (uint32_t)(b_tmpl >> 32), b_lo0 = (uint32_t)b_tmpl;
      int s = 0, acc = 0;
      uint32_t ph = 0, acc_ph = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < n_work && ok; work += gridDim.x) {
        const int nkb = min(kblocks, (work / n_tiles) * kb_per + kb_per) - (work / n_tiles) * kb_per;
        if (!__all_sync(0xffffffffu, wait_fast(tempty0 + 8 * acc, acc_ph ^ 1))) {
          if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_TMEM_EMPTY, 11, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BF16_BN;
        uint32_t accumulate = 0;
        for (int i = 0; i < nkb; ++i) {
          if (!__all_sync(0xffffffffu, wait_fast(full0 + 8 * s, ph))) {
            if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_SMEM_FULL, 12, s);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_lo = a_lo0 + s * (BF16_STAGE_BYTES >> 4), b_lo = b_lo0 + s * (BF16_STAGE_BYTES >> 4);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BF16_BK / 16; ++k)
              mma_bf16(d_tmem, desc_at(a_hi, a_lo + k * a_step), desc_at(b_hi, b_lo + k * b_step), idesc,
                       (k == 0) ? accumulate : 1u);
            mma_commit(empty0 + 8 * s);
          }
          __syncwarp();
          accumulate = 1;
          if (++s == BF16_STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok || aborted(bars)) break;
        if (elect_one()) mma_commit(tfull0 + 8 * acc);
        __syncwarp();
        if (++acc == BF16_ACC) { acc = 0; acc_ph ^= 1; }
      }
    }
  } else {
    const int ew = warp - 2;
    uint8_t* stage = stage_all + ew * EPI_STAGE_BYTES_PER_WARP;
    const int quarter = warp & 3;        // TMEM lane quarter this warp may access
    const int col_half = ew >> 2;        // which 128 of the tile's 256 columns
    int acc = 0;
    uint32_t acc_ph = 0;
    uint8_t* aux_buf = aux_all + ew * (2 * AUX_BOX_BYTES);
    const uint32_t aux_bar = smem_u32(&bars->aux_full[ew]);
    uint32_t aux_ph = 0;
    bool aux_pending = false;
    if (AUX && blockIdx.x < n_work) {
      int mb_, nb_;
      tile_coords(blockIdx.x % n_tiles, n_tiles_m, n_tiles_n, mb_, nb_);
      aux_pending = aux_prefetch(&tmap_aux, g.M, g.N, mb_ * BM + quarter * 32, lane, nb_ * BF16_BN + col_half * 128, 2,
                                 smem_u32(aux_buf), aux_bar);
    }
    for (int work = blockIdx.x; work < n_work && !aborted(bars); work += gridDim.x) {
      const int tile = work % n_tiles;
      int mb_, nb_;
      tile_coords(tile, n_tiles_m, n_tiles_n, mb_, nb_);
      const int m0 = mb_ * BM, n0 = nb_ * BF16_BN;
      const int m = m0 + quarter * 32 + lane;
      const float rs = (m < g.M) ? row_scale_for(e, m) : 1.0f;
      const float rc = (e.rowcoef != nullptr && m < g.M) ? e.rowcoef[m] : 0.0f;
      float bias_c[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) bias_c[c] = load_bias(e, n0 + col_half * 128 + c * 32 + lane, g.N);
      if (!mbar_wait_warp(tfull0 + 8 * acc, acc_ph)) {
        raise_abort(bars, status, STATUS_TIMEOUT_TMEM_FULL, 13, acc);
        break;
      }
      if (AUX && aux_pending) {
        if (!mbar_wait_warp(aux_bar, aux_ph)) {
          raise_abort(bars, status, STATUS_TIMEOUT_SMEM_FULL, 14, ew);
          break;
        }
        aux_ph ^= 1;
      }
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BF16_BN + col_half * 128;
      float ssq = 0.0f;
      // two chunks are in flight: the TMEM load of the next chunk overlaps the math and stores of this one.
      // The loop body covers two chunks (one per register buffer) and is not unrolled further: the epilogue
      // warps are bound by instruction fetch and issue, so the code has to stay small.
      uint32_t raw0[32], raw1[32];
      auto do_chunk = [&](uint32_t (&raw)[32], int c, float bias) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
        ssq += epilogue_chunk(e, g.M, g.N, m0 + quarter * 32, lane, n0 + col_half * 128 + c * 32, rs, rc, v, stage, bias,
                              AUX ? aux_buf + (c >> 1) * AUX_BOX_BYTES + lane * 128 : nullptr, (c & 1) * 4);
      };
      tmem_ld_32x32(t_row, raw0);
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        tmem_ld_wait();
        tmem_ld_32x32(t_row + (2 * cc + 1) * 32, raw1);
        do_chunk(raw0, 2 * cc, cc ? bias_c[2] : bias_c[0]);
        tmem_ld_wait();
        if (cc == 0) {
          tmem_ld_32x32(t_row + 64, raw0);
        } else {   // everything is in registers: hand the accumulator back before the last chunk's stores
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
        }
        do_chunk(raw1, 2 * cc + 1, cc ? bias_c[3] : bias_c[1]);
      }
      if (AUX) {   // this tile's slice is consumed: fetch the next tile's
        __syncwarp();
        aux_pending = false;
        const int next = work + gridDim.x;
        if (next < n_work) {
          int mb2, nb2;
          tile_coords(next % n_tiles, n_tiles_m, n_tiles_n, mb2, nb2);
          aux_pending = aux_prefetch(&tmap_aux, g.M, g.N, mb2 * BM + quarter * 32, lane,
                                     nb2 * BF16_BN + col_half * 128, 2, smem_u32(aux_buf), aux_bar);
        }
      }
      if (e.ssq_out != nullptr && m < g.M && n0 + col_half * 128 < g.N)
        e.ssq_out[(size_t)m * e.ssq_parts + (n0 / 128 + col_half)] = ssq;
      if (++acc == BF16_ACC) { acc = 0; acc_ph ^= 1; }
    }
  }
  pipe_teardown(bars, warp, BF16_ACC * BF16_BN);
}

// ---------------------------------------------------------------------------------------
// bf16 kernel on CTA pairs
// ---------------------------------------------------------------------------------------
// With a 1024-deep reduction these GEMMs are bound by the traffic from L2 into shared memory, not by the
// tensor cores. A pair of CTAs on neighbouring SMs shares one 256 x 256 tile: each CTA loads its own 128 rows
// of A but only half of B (128 of the 256 N rows), and tcgen05.mma.cta_group::2 reads both halves. Per CTA
// and K block that is 32 KB instead of 48 KB for the same 128 x 256 accumulator.
//
// Barriers: full[s] lives in the rank-0 CTA and counts the bytes of both CTAs' loads; empty[s] and
// tmem_full[a] exist in both CTAs and are signalled together by the commit of the MMA thread (rank 0);
// tmem_empty[a] lives in rank 0 and collects the epilogue warps of both CTAs.
constexpr int PAIR_BN = 256;
constexpr int PAIR_B_ROWS = 128;                               // N rows of B held by each CTA
constexpr int PAIR_A_BYTES = BM * STAGE_ROW_BYTES;            // 16 KB
constexpr int PAIR_B_BYTES = PAIR_B_ROWS * STAGE_ROW_BYTES;   // 16 KB
constexpr int PAIR_STAGE_BYTES = PAIR_A_BYTES + PAIR_B_BYTES;
constexpr int PAIR_TMEM_COLS = BF16_ACC * PAIR_BN;

template <bool AUX>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_aux, const __grid_constant__ CUtensorMap tmap_out,
                      const __grid_constant__ CUtensorMap tmap_pre, const GemmShape g, const GemmEpilogue e,
                      Status* status) {
  constexpr int STAGES = AUX ? 4 : 6;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_all = smem + STAGES * PAIR_STAGE_BYTES;
  uint8_t* aux_all = stage_all + EPI_STAGE_BYTES;
  PipeBars* bars = reinterpret_cast<PipeBars*>(aux_all + (AUX ? BF16_AUX_BYTES : 0));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < BF16_ACC; ++a) {
      mbar_init(smem_u32(&bars->tmem_full[a]), 1);
      mbar_init(smem_u32(&bars->tmem_empty[a]), 2 * EPI_WARPS);
    }
    for (int w = 0; w < 4 * EPI_WARPS; ++w) mbar_init(smem_u32(&bars->aux_full[w]), 1);
    bars->abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&bars->tmem_base), PAIR_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();     // the peer's barriers exist before anything of this CTA can signal them
  tc_fence_after_sync();
  pdl_enter();
  const uint32_t tmem_base = bars->tmem_base;

  const int n_tiles_n = (g.N + PAIR_BN - 1) / PAIR_BN;
  const int n_tiles_m = (g.M + 2 * BM - 1) / (2 * BM);
  const int n_tiles = n_tiles_m * n_tiles_n;
  const int kblocks = (g.K + BF16_BK - 1) / BF16_BK;
  const int kb_per = (kblocks + g.splits - 1) / g.splits;
  const int n_work = n_tiles * g.splits;
  const uint32_t smem0 = smem_u32(smem);
  const uint32_t full0 = smem_u32(&bars->full[0]), empty0 = smem_u32(&bars->empty[0]);
  const uint32_t tfull0 = smem_u32(&bars->tmem_full[0]), tempty0 = smem_u32(&bars->tmem_empty[0]);

  if (warp == 0) {
    {   // all 32 lanes run the loop; one elected lane issues the loads (see elect_one)
      const uint32_t full_lead0 = map_to_cta(full0, 0);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int work = pair; work < n_work && ok; work += n_pairs) {
        const int tile = work % n_tiles, kb0 = (work / n_tiles) * kb_per, kb1 = min(kblocks, kb0 + kb_per);
        int mb_, nb_;
        tile_coords(tile, n_tiles_m, n_tiles_n, mb_, nb_);
        const int m0 = mb_ * 2 * BM + (int)rank * BM, nB = nb_ * PAIR_BN + (int)rank * PAIR_B_ROWS;
        int kx = kb0 * BF16_BK;
        for (int kb = kb0; kb < kb1; ++kb, kx += BF16_BK) {
          if (!__all_sync(0xffffffffu, wait_fast(empty0 + 8 * s, ph ^ 1))) {
            if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_SMEM_EMPTY, 60, s);
            ok = false;
            break;
          }
          const uint32_t full = full_lead0 + 8 * s;
          const uint32_t a_dst = smem0 + s * PAIR_STAGE_BYTES;
          const uint32_t b_dst = a_dst + PAIR_A_BYTES;
          if (elect_one()) {
            if (rank == 0) mbar_arrive_expect_tx(full0 + 8 * s, 2 * PAIR_STAGE_BYTES);
            if (!g.a_mn) {
              tma_load_2d_pair(a_dst, &tmap_a, full, kx, m0);
            } else {
#pragma unroll
              for (int i = 0; i < BM / 64; ++i)
                tma_load_2d_pair(a_dst + i * (BF16_BK * STAGE_ROW_BYTES), &tmap_a, full, m0 + i * 64, kx);
            }
            if (!g.b_mn) {
              tma_load_2d_pair(b_dst, &tmap_b, full, kx, nB);
            } else {
#pragma unroll
              for (int i = 0; i < PAIR_B_ROWS / 64; ++i)
                tma_load_2d_pair(b_dst + i * (BF16_BK * STAGE_ROW_BYTES), &tmap_b, full, nB + i * 64, kx);
            }
          }
          __syncwarp();
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (aborted(bars)) break;
      }
    }
  } else if (warp == 1) {
    if (rank == 0) {   // the leader's warp runs the loop with all lanes; one elected lane issues
      const uint32_t idesc = make_instr_desc(1, 1, g.a_mn ? 1 : 0, g.b_mn ? 1 : 0, 2 * BM, PAIR_BN);
      const uint32_t a_lbo = g.a_mn ? BF16_BK * STAGE_ROW_BYTES : 16, b_lbo = g.b_mn ? BF16_BK * STAGE_ROW_BYTES : 16;
      const uint32_t a_step = g.a_mn ? (16 * STAGE_ROW_BYTES) >> 4 : 2, b_step = g.b_mn ? (16 * STAGE_ROW_BYTES) >> 4 : 2;
      const uint64_t a_tmpl = make_smem_desc(smem0, a_lbo, 1024), b_tmpl = make_smem_desc(smem0 + PAIR_A_BYTES, b_lbo, 1024);
      const uint32_t a_hi = (uint32_t)(a_tmpl >> 32), a_lo0 = (uint32_t)a_tmpl;
      const uint32_t b_hi = (uint32_t)(b_tmpl >> 32), b_lo0 = (uint32_t)b_tmpl;
      int s = 0, acc = 0;
      uint32_t ph = 0, acc_ph = 0;
      bool ok = true;
      for (int work = pair; work < n_work && ok; work += n_pairs) {
        const int nkb = min(kblocks, (work / n_tiles) * kb_per + kb_per) - (work / n_tiles) * kb_per;
        if (!__all_sync(0xffffffffu, wait_fast(tempty0 + 8 * acc, acc_ph ^ 1))) {
          if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_TMEM_EMPTY, 61, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * PAIR_BN;
        uint32_t accumulate = 0;
        for (int i = 0; i < nkb; ++i) {
          if (!__all_sync(0xffffffffu, wait_fast(full0 + 8 * s, ph))) {
            if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_SMEM_FULL, 62, s);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_lo = a_lo0 + s * (PAIR_STAGE_BYTES >> 4), b_lo = b_lo0 + s * (PAIR_STAGE_BYTES >> 4);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BF16_BK / 16; ++k)
              mma_bf16_pair(d_tmem, desc_at(a_hi, a_lo + k * a_step), desc_at(b_hi, b_lo + k * b_step), idesc,
                            (k == 0) ? accumulate : 1u);
            mma_commit_pair(empty0 + 8 * s);
          }
          __syncwarp();
          accumulate = 1;
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok || aborted(bars)) break;
        if (elect_one()) mma_commit_pair(tfull0 + 8 * acc);
        __syncwarp();
        if (++acc == BF16_ACC) { acc = 0; acc_ph ^= 1; }
      }
    } else if (g.jobs != nullptr) {
      // the second CTA's warp 1 issues no MMAs: it pulls parameter ranges from their owner ranks
      run_gather_jobs(g.jobs, g.n_jobs, pair, n_pairs, lane);
    }
  } else {
    const int ew = warp - 2;
    uint8_t* stage = stage_all + ew * EPI_STAGE_BYTES_PER_WARP;
    const int quarter = warp & 3;        // TMEM lane quarter this warp may access
    const int col_half = ew >> 2;        // which 128 of the tile's 256 columns
    const uint32_t tempty_lead0 = map_to_cta(tempty0, 0);
    int acc = 0;
    uint32_t acc_ph = 0;
    const uint32_t aux_slot0 = smem_u32(aux_all + ew * (4 * AUX_CHUNK_BYTES));   // four chunk slots per warp
    const uint8_t* aux_mine = aux_all + ew * (4 * AUX_CHUNK_BYTES) + lane * 64;
    const uint32_t aux_bar0 = smem_u32(&bars->aux_full[ew * 4]);
    uint32_t aux_ph = 0;
    bool aux_ok = true;
    if (AUX && pair < n_work) {
      int mb_, nb_;
      tile_coords(pair % n_tiles, n_tiles_m, n_tiles_n, mb_, nb_);
      for (int c = 0; c < 4; ++c)
        aux_request(&tmap_aux, mb_ * 2 * BM + (int)rank * BM + quarter * 32, nb_ * PAIR_BN + col_half * 128 + c * 32,
                    aux_slot0 + c * AUX_CHUNK_BYTES, aux_bar0 + 8 * c);
    }
    for (int work = pair; work < n_work && !aborted(bars); work += n_pairs) {
      const int tile = work % n_tiles;
      int mb_, nb_;
      tile_coords(tile, n_tiles_m, n_tiles_n, mb_, nb_);
      const int m0 = mb_ * 2 * BM + (int)rank * BM, n0 = nb_ * PAIR_BN;
      const int m = m0 + quarter * 32 + lane;
      const float rs = (m < g.M) ? row_scale_for(e, m) : 1.0f;
      const float rc = (e.rowcoef != nullptr && m < g.M) ? e.rowcoef[m] : 0.0f;
      float bias_c[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) bias_c[c] = load_bias(e, n0 + col_half * 128 + c * 32 + lane, g.N);
      if (!mbar_wait_warp(tfull0 + 8 * acc, acc_ph)) {
        raise_abort(bars, status, STATUS_TIMEOUT_TMEM_FULL, 63, acc);
        break;
      }
      // where the next tile's chunks go (a slot is asked for again as soon as its chunk has been read)
      const int next = work + n_pairs;
      int m_next = 0, n_next = 0;
      if (AUX && next < n_work) {
        int mb2, nb2;
        tile_coords(next % n_tiles, n_tiles_m, n_tiles_n, mb2, nb2);
        m_next = mb2 * 2 * BM + (int)rank * BM + quarter * 32;
        n_next = nb2 * PAIR_BN + col_half * 128;
      }
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * PAIR_BN + col_half * 128;
      float ssq = 0.0f;
      // two chunks are in flight: the TMEM load of the next chunk overlaps the math and stores of this one.
      // The loop body covers two chunks (one per register buffer) and is not unrolled further: the epilogue
      // warps are bound by instruction fetch and issue, so the code has to stay small.
      uint32_t raw0[32], raw1[32];
      auto do_chunk = [&](uint32_t (&raw)[32], int c, float bias) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
        if (AUX && aux_ok && !mbar_wait_warp(aux_bar0 + 8 * c, aux_ph)) {
          raise_abort(bars, status, STATUS_TIMEOUT_SMEM_FULL, 64, ew);
          aux_ok = false;
        }
        ssq += epilogue_chunk(e, g.M, g.N, m0 + quarter * 32, lane, n0 + col_half * 128 + c * 32, rs, rc, v, stage, bias,
                              AUX ? aux_mine + c * AUX_CHUNK_BYTES : nullptr, 0, true,
                              (e.tma_mask & 1) ? &tmap_out : nullptr, (e.tma_mask & 2) ? &tmap_pre : nullptr);
        if (AUX && aux_ok && next < n_work) {
          __syncwarp();
          aux_request(&tmap_aux, m_next, n_next + c * 32, aux_slot0 + c * AUX_CHUNK_BYTES, aux_bar0 + 8 * c);
        }
      };
      tmem_ld_32x32(t_row, raw0);
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        tmem_ld_wait();
        tmem_ld_32x32(t_row + (2 * cc + 1) * 32, raw1);
        do_chunk(raw0, 2 * cc, cc ? bias_c[2] : bias_c[0]);
        tmem_ld_wait();
        if (cc == 0) {
          tmem_ld_32x32(t_row + 64, raw0);
        } else {   // everything is in registers: hand the accumulator back before the last chunk's stores
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tempty_lead0 + 8 * acc);
        }
        do_chunk(raw1, 2 * cc + 1, cc ? bias_c[3] : bias_c[1]);
      }
      aux_ph ^= 1;
      if (!aux_ok) break;
      if (e.ssq_out != nullptr && m < g.M && n0 + col_half * 128 < g.N)
        e.ssq_out[(size_t)m * e.ssq_parts + (n0 / 128 + col_half)] = ssq;
      if (++acc == BF16_ACC) { acc = 0; acc_ph ^= 1; }
    }
    stage_acquire();   // the last bulk stores have read the staging area
  }

  // teardown: neither CTA may leave (or free its TMEM) while the other can still read its shared memory,
  // write its TMEM or signal its barriers
  tc_fence_before_sync();
  __syncthreads();
  if (aborted(bars)) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, PAIR_TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// block-scaled FP8 kernel
// ---------------------------------------------------------------------------------------
constexpr int FP8_BN = 128;
constexpr int FP8_BK = 128;
constexpr int FP8_STAGES = 6;
constexpr int FP8_ACC = 4;
constexpr int FP8_A_BYTES = BM * STAGE_ROW_BYTES;
constexpr int FP8_B_BYTES = FP8_BN * STAGE_ROW_BYTES;
constexpr int FP8_STAGE_BYTES = FP8_A_BYTES + FP8_B_BYTES;

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const GemmShape g, const GemmEpilogue e, Status* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_all = smem + FP8_STAGES * FP8_STAGE_BYTES;
  PipeBars* bars = reinterpret_cast<PipeBars*>(stage_all + EPI_STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pipe_setup<FP8_STAGES, FP8_ACC>(bars, warp, lane, FP8_ACC * FP8_BN, &tmap_a, &tmap_b);
  const uint32_t tmem_base = bars->tmem_base;

  const int n_tiles_n = (g.N + FP8_BN - 1) / FP8_BN;
  const int n_tiles_m = (g.M + BM - 1) / BM;
  const int n_tiles = n_tiles_m * n_tiles_n;
  const int kblocks = (g.K + FP8_BK - 1) / FP8_BK;
  const int kb_per = (kblocks + g.splits - 1) / g.splits;
  const int n_work = n_tiles * g.splits;
  const uint32_t smem0 = smem_u32(smem);
  const uint32_t full0 = smem_u32(&bars->full[0]), empty0 = smem_u32(&bars->empty[0]);
  const uint32_t tfull0 = smem_u32(&bars->tmem_full[0]), tempty0 = smem_u32(&bars->tmem_empty[0]);

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < n_work && ok; work += gridDim.x) {
        const int tile = work % n_tiles, kb0 = (work / n_tiles) * kb_per, kb1 = min(kblocks, kb0 + kb_per);
        int mb_, nb_;
        tile_coords(tile, n_tiles_m, n_tiles_n, mb_, nb_);
        const int m0 = mb_ * BM, n0 = nb_ * FP8_BN;
        int kx = kb0 * FP8_BK;
        for (int kb = kb0; kb < kb1; ++kb, kx += FP8_BK) {
          if (!wait_fast(empty0 + 8 * s, ph ^ 1)) {
            raise_abort(bars, status, STATUS_TIMEOUT_SMEM_EMPTY, 20, s);
            ok = false;
            break;
          }
          const uint32_t full = full0 + 8 * s;
          const uint32_t a_dst = smem0 + s * FP8_STAGE_BYTES;
          mbar_arrive_expect_tx(full, FP8_STAGE_BYTES);
          tma_load_2d(a_dst, &tmap_a, full, kx, m0);
          tma_load_2d(a_dst + FP8_A_BYTES, &tmap_b, full, kx, n0);
          if (++s == FP8_STAGES) { s = 0; ph ^= 1; }
        }
        if (aborted(bars)) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_instr_desc(0, 0, 0, 0, BM, FP8_BN);
      const uint64_t a_tmpl = make_smem_desc(smem0, 16, 1024), b_tmpl = make_smem_desc(smem0 + FP8_A_BYTES, 16, 1024);
      const uint32_t a_hi = (uint32_t)(a_tmpl >> 32), a_lo0 = (uint32_t)a_tmpl;
      const uint32_t b_hi = (uint32_t)(b_tmpl >> 32), b_lo0 = (uint32_t)b_tmpl;
      int s = 0, acc = 0;
      uint32_t ph = 0, acc_ph = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < n_work && ok; work += gridDim.x) {
        const int nkb = min(kblocks, (work / n_tiles) * kb_per + kb_per) - (work / n_tiles) * kb_per;
        for (int i = 0; i < nkb; ++i) {
          if (!wait_fast(tempty0 + 8 * acc, acc_ph ^ 1)) {
            raise_abort(bars, status, STATUS_TIMEOUT_TMEM_EMPTY, 21, acc);
            ok = false;
            break;
          }
          if (!wait_fast(full0 + 8 * s, ph)) {
            raise_abort(bars, status, STATUS_TIMEOUT_SMEM_FULL, 22, s);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_lo = a_lo0 + s * (FP8_STAGE_BYTES >> 4), b_lo = b_lo0 + s * (FP8_STAGE_BYTES >> 4);
          const uint32_t d_tmem = tmem_base + acc * FP8_BN;
#pragma unroll
          for (int k = 0; k < FP8_BK / 32; ++k)
            mma_fp8(d_tmem, desc_at(a_hi, a_lo + k * 2), desc_at(b_hi, b_lo + k * 2), idesc, k != 0);
          mma_commit(empty0 + 8 * s);
          mma_commit(tfull0 + 8 * acc);
          if (++s == FP8_STAGES) { s = 0; ph ^= 1; }
          if (++acc == FP8_ACC) { acc = 0; acc_ph ^= 1; }
        }
        if (aborted(bars)) break;
      }
    }
  } else {
    const int ew = warp - 2;
    uint8_t* stage = stage_all + ew * EPI_STAGE_BYTES_PER_WARP;
    const int quarter = warp & 3;
    const int col_half = ew >> 2;  // which 64 of the tile's 128 columns
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + col_half * 64;
    for (int work = blockIdx.x; work < n_work && ok; work += gridDim.x) {
      const int tile = work % n_tiles, kb0 = (work / n_tiles) * kb_per, kb1 = min(kblocks, kb0 + kb_per);
      int mb_, nb_;
      tile_coords(tile, n_tiles_m, n_tiles_n, mb_, nb_);
      const int m0 = mb_ * BM, n0 = nb_ * FP8_BN;
      const int m = m0 + quarter * 32 + lane;
      const int m_ld = (m < g.M) ? m : (g.M - 1);
      const float* sa_row = g.sa + m_ld;
      const float* sb_row = g.sb + (size_t)nb_ * kblocks;
      float accum[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) accum[j] = 0.0f;
      // scales are fetched four K blocks ahead so their global-memory latency never sits on the
      // accumulate path
      float sq[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        sq[i] = (kb0 + i < kb1) ? sa_row[(size_t)(kb0 + i) * g.sa_ld] * sb_row[kb0 + i] : 0.0f;
      for (int kb = kb0; kb < kb1; ++kb) {
        const float scale = sq[0];
        sq[0] = sq[1]; sq[1] = sq[2]; sq[2] = sq[3];
        sq[3] = (kb + 4 < kb1) ? sa_row[(size_t)(kb + 4) * g.sa_ld] * sb_row[kb + 4] : 0.0f;
        if (!wait_fast(tfull0 + 8 * acc, acc_ph)) {
          raise_abort(bars, status, STATUS_TIMEOUT_TMEM_FULL, 23, acc);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t t_row = t_lane + acc * FP8_BN;
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(t_row, r0);
        tmem_ld_32x32(t_row + 32, r1);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          accum[j] = fmaf(scale, __uint_as_float(r0[j]), accum[j]);
          accum[32 + j] = fmaf(scale, __uint_as_float(r1[j]), accum[32 + j]);
        }
        if (++acc == FP8_ACC) { acc = 0; acc_ph ^= 1; }
      }
      if (!ok || aborted(bars)) break;
      const float rs = (m < g.M) ? row_scale_for(e, m) : 1.0f;
      const float rc = (e.rowcoef != nullptr && m < g.M) ? e.rowcoef[m] : 0.0f;
      float ssq = 0.0f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = accum[c * 32 + j];
        const int nc = n0 + col_half * 64 + c * 32;
        ssq += epilogue_chunk(e, g.M, g.N, m0 + quarter * 32, lane, nc, rs, rc, v, stage, load_bias(e, nc + lane, g.N),
                              nullptr, 0);
      }
      if (e.ssq_out != nullptr && m < g.M)
        e.ssq_out[(size_t)m * e.ssq_parts + (n0 / 64 + col_half)] = ssq;
    }
  }
  pipe_teardown(bars, warp, FP8_ACC * FP8_BN);
}

// ---------------------------------------------------------------------------------------
// hardware block-scaled FP8 kernel (UE8M0 scales applied by the tensor core)
// ---------------------------------------------------------------------------------------
// Same pipeline as the bf16 kernel (whole-K accumulation in TMEM, two accumulator stages). Each stage
// also carries the two 512-byte packed scale chunks of its K block; the MMA thread copies them into
// TMEM (tcgen05.cp) in front of the four MMAs that use them. Scales must be powers of two. A chunk holds four
// bytes per row, one per 32-element K step; K step k of a stage reads byte k of both operands' scale words
// (operands with 1x128 / 128x128 blocks repeat one byte four times, the epilogue's quantised copy has 1x64 blocks).
constexpr int MX_BN = 128;
constexpr int MX_BK = 128;
constexpr int MX_ACC = 2;
constexpr int MX_AUX_BYTES = EPI_WARPS * AUX_BOX_BYTES;        // one box (64 columns) per epilogue warp
constexpr int MX_A_BYTES = BM * STAGE_ROW_BYTES;
constexpr int MX_B_BYTES = MX_BN * STAGE_ROW_BYTES;
constexpr int MX_SF_BYTES = 512;
constexpr int MX_STAGE_BYTES = MX_A_BYTES + MX_B_BYTES + 2 * MX_SF_BYTES;   // 33 KB, a multiple of 1024
constexpr int MX_TMEM_COLS = 512;
constexpr int MX_SF_COL0 = MX_ACC * MX_BN;                                   // scale columns follow the accumulators

// e4m3 copy of one epilogue warp's 32 rows x 64 columns (va: columns nq..nq+31 of row m_warp + lane, vb: the next
// 32), one power-of-two scale per row, for the GEMM that consumes this output as its A operand. The values are
// the bf16-rounded outputs (after silu when q8_silu is set). Warp-collective.
__device__ __forceinline__ void mx_emit_q8(const GemmEpilogue& e, int M, int m_warp, int nq, int lane, int col_half,
                                           float (&va)[32], float (&vb)[32], uint8_t* stage,
                                           const CUtensorMap* t_q8 = nullptr) {
  const int m = m_warp + lane;
  float amax = 0.0f;
  if (e.q8_silu) {   // tested once, not per element (see the auxiliary modes in epilogue_chunk)
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      va[j] = siluf_(__bfloat162float(__float2bfloat16(va[j])));
      vb[j] = siluf_(__bfloat162float(__float2bfloat16(vb[j])));
    }
  }
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const float x0 = __bfloat162float(__float2bfloat16(va[j])), x1 = __bfloat162float(__float2bfloat16(vb[j]));
    va[j] = x0;
    vb[j] = x1;
    amax = fmaxf(amax, fmaxf(fabsf(x0), fabsf(x1)));
  }
  const float sc = block_scale(amax, 1);
  const float inv = 1.0f / sc;
  uint32_t w[16];
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    w[t] = pack4_e4m3(va[4 * t] * inv, va[4 * t + 1] * inv, va[4 * t + 2] * inv, va[4 * t + 3] * inv);
    w[8 + t] = pack4_e4m3(vb[4 * t] * inv, vb[4 * t + 1] * inv, vb[4 * t + 2] * inv, vb[4 * t + 3] * inv);
  }
  // 32 rows x 64 bytes through the staging area (same shape as a 32-column bf16 chunk)
  if (t_q8 != nullptr)
    store_rows_tma(stage, lane, w, t_q8, nq, m_warp);
  else
    store_rows_bf16(stage, lane, w, reinterpret_cast<__nv_bfloat16*>(e.q8 + (size_t)m_warp * e.q8_ld + nq),
                    e.q8_ld / 2, min(32, M - m_warp));
  if (m < M) {
    uint8_t* chunk = e.q8_p + ((int64_t)(m >> 7) * e.q8_p_stride + (nq >> 7)) * 512;
    *reinterpret_cast<uint16_t*>(chunk + (m & 31) * 16 + ((m >> 5) & 3) * 4 + col_half * 2) =
        (uint16_t)(ue8m0_word(sc) & 0xFFFFu);
  }
}

template <bool AUX>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_mx_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_aux, const GemmShape g, const GemmEpilogue e, Status* status) {
  constexpr int MX_STAGES = AUX ? 5 : 6;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_all = smem + MX_STAGES * MX_STAGE_BYTES;
  uint8_t* aux_all = stage_all + EPI_STAGE_BYTES;
  PipeBars* bars = reinterpret_cast<PipeBars*>(aux_all + (AUX ? MX_AUX_BYTES : 0));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pipe_setup<MX_STAGES, MX_ACC>(bars, warp, lane, MX_TMEM_COLS, &tmap_a, &tmap_b);
  pdl_enter();
  const uint32_t tmem_base = bars->tmem_base;

  const int n_tiles_n = (g.N + MX_BN - 1) / MX_BN;
  const int n_tiles_m = (g.M + BM - 1) / BM;
  const int n_tiles = n_tiles_m * n_tiles_n;
  const int kblocks = (g.K + MX_BK - 1) / MX_BK;
  const int kb_per = (kblocks + g.splits - 1) / g.splits;
  const int n_work = n_tiles * g.splits;
  const uint32_t smem0 = smem_u32(smem);
  const uint32_t full0 = smem_u32(&bars->full[0]), empty0 = smem_u32(&bars->empty[0]);
  const uint32_t tfull0 = smem_u32(&bars->tmem_full[0]), tempty0 = smem_u32(&bars->tmem_empty[0]);

  if (warp == 0) {
    {   // all 32 lanes run the loop; one elected lane issues the loads (see elect_one)
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < n_work && ok; work += gridDim.x) {
        const int tile = work % n_tiles, kb0 = (work / n_tiles) * kb_per, kb1 = min(kblocks, kb0 + kb_per);
        int mb_, nb_;
        tile_coords(tile, n_tiles_m, n_tiles_n, mb_, nb_);
        const int m0 = mb_ * BM, n0 = nb_ * MX_BN;
        const uint8_t* sfa = g.sfa_packed + ((size_t)mb_ * kblocks + kb0) * MX_SF_BYTES;
        const uint8_t* sfb = g.sfb_packed + ((size_t)nb_ * kblocks + kb0) * MX_SF_BYTES;
        int kx = kb0 * MX_BK;
        for (int kb = kb0; kb < kb1; ++kb, kx += MX_BK, sfa += MX_SF_BYTES, sfb += MX_SF_BYTES) {
          if (!__all_sync(0xffffffffu, wait_fast(empty0 + 8 * s, ph ^ 1))) {
            if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_SMEM_EMPTY, 50, s);
            ok = false;
            break;
          }
          const uint32_t full = full0 + 8 * s;
          const uint32_t a_dst = smem0 + s * MX_STAGE_BYTES;
          if (elect_one()) {
            mbar_arrive_expect_tx(full, MX_STAGE_BYTES);
            tma_load_2d(a_dst, &tmap_a, full, kx, m0);
            tma_load_2d(a_dst + MX_A_BYTES, &tmap_b, full, kx, n0);
            bulk_load(a_dst + MX_A_BYTES + MX_B_BYTES, sfa, MX_SF_BYTES, full);
            bulk_load(a_dst + MX_A_BYTES + MX_B_BYTES + MX_SF_BYTES, sfb, MX_SF_BYTES, full);
          }
          __syncwarp();
          if (++s == MX_STAGES) { s = 0; ph ^= 1; }
        }
        if (aborted(bars)) break;
      }
    }
  } else if (warp == 1) {
    {   // warp-wide loop, one elected lane issues
      const uint32_t idesc = make_instr_desc_mx(BM, MX_BN, 0, 0);
      const uint64_t a_tmpl = make_smem_desc(smem0, 16, 1024), b_tmpl = make_smem_desc(smem0 + MX_A_BYTES, 16, 1024);
      const uint64_t sfa_tmpl = make_smem_desc_noswizzle(smem0 + MX_A_BYTES + MX_B_BYTES, 16, 128);
      const uint32_t a_hi = (uint32_t)(a_tmpl >> 32), a_lo0 = (uint32_t)a_tmpl;
      const uint32_t b_hi = (uint32_t)(b_tmpl >> 32), b_lo0 = (uint32_t)b_tmpl;
      const uint32_t sf_hi = (uint32_t)(sfa_tmpl >> 32), sf_lo0 = (uint32_t)sfa_tmpl;
      int s = 0, acc = 0, slot = 0;
      uint32_t ph = 0, acc_ph = 0;
      bool ok = true;
      for (int work = blockIdx.x; work < n_work && ok; work += gridDim.x) {
        const int nkb = min(kblocks, (work / n_tiles) * kb_per + kb_per) - (work / n_tiles) * kb_per;
        if (!__all_sync(0xffffffffu, wait_fast(tempty0 + 8 * acc, acc_ph ^ 1))) {
          if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_TMEM_EMPTY, 51, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * MX_BN;
        uint32_t accumulate = 0;
        for (int i = 0; i < nkb; ++i) {
          if (!__all_sync(0xffffffffu, wait_fast(full0 + 8 * s, ph))) {
            if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_SMEM_FULL, 52, s);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t off = s * (MX_STAGE_BYTES >> 4);
          const uint32_t sfa_t = tmem_base + MX_SF_COL0 + slot * 8, sfb_t = sfa_t + 4;
          if (elect_one()) {
            tmem_cp_scales(sfa_t, desc_at(sf_hi, sf_lo0 + off));
            tmem_cp_scales(sfb_t, desc_at(sf_hi, sf_lo0 + off + (MX_SF_BYTES >> 4)));
#pragma unroll
            for (int k = 0; k < MX_BK / 32; ++k)
              mma_mxfp8(d_tmem, desc_at(a_hi, a_lo0 + off + k * 2), desc_at(b_hi, b_lo0 + off + k * 2),
                        idesc | mx_sf_ids(k), (k == 0) ? accumulate : 1u, sfa_t, sfb_t);
            mma_commit(empty0 + 8 * s);
          }
          __syncwarp();
          accumulate = 1;
          slot ^= 1;
          if (++s == MX_STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok || aborted(bars)) break;
        if (elect_one()) mma_commit(tfull0 + 8 * acc);
        __syncwarp();
        if (++acc == MX_ACC) { acc = 0; acc_ph ^= 1; }
      }
    }
  } else {
    const int ew = warp - 2;
    uint8_t* stage = stage_all + ew * EPI_STAGE_BYTES_PER_WARP;
    const int quarter = warp & 3;
    const int col_half = ew >> 2;        // which 64 of the tile's 128 columns
    int acc = 0;
    uint32_t acc_ph = 0;
    uint8_t* aux_buf = aux_all + ew * AUX_BOX_BYTES;
    const uint32_t aux_bar = smem_u32(&bars->aux_full[ew]);
    uint32_t aux_ph = 0;
    bool aux_pending = false;
    if (AUX && blockIdx.x < n_work) {
      int mb_, nb_;
      tile_coords(blockIdx.x % n_tiles, n_tiles_m, n_tiles_n, mb_, nb_);
      aux_pending = aux_prefetch(&tmap_aux, g.M, g.N, mb_ * BM + quarter * 32, lane, nb_ * MX_BN + col_half * 64, 1,
                                 smem_u32(aux_buf), aux_bar);
    }
    for (int work = blockIdx.x; work < n_work && !aborted(bars); work += gridDim.x) {
      const int tile = work % n_tiles;
      int mb_, nb_;
      tile_coords(tile, n_tiles_m, n_tiles_n, mb_, nb_);
      const int m0 = mb_ * BM, n0 = nb_ * MX_BN;
      const int m = m0 + quarter * 32 + lane;
      const float rs = (m < g.M) ? row_scale_for(e, m) : 1.0f;
      const float rc = (e.rowcoef != nullptr && m < g.M) ? e.rowcoef[m] : 0.0f;
      const float bias0 = load_bias(e, n0 + col_half * 64 + lane, g.N);
      const float bias1 = load_bias(e, n0 + col_half * 64 + 32 + lane, g.N);
      if (!mbar_wait_warp(tfull0 + 8 * acc, acc_ph)) {
        raise_abort(bars, status, STATUS_TIMEOUT_TMEM_FULL, 53, acc);
        break;
      }
      if (AUX && aux_pending) {
        if (!mbar_wait_warp(aux_bar, aux_ph)) {
          raise_abort(bars, status, STATUS_TIMEOUT_SMEM_FULL, 54, ew);
          break;
        }
        aux_ph ^= 1;
      }
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * MX_BN + col_half * 64;
      uint32_t r0[32], r1[32];
      tmem_ld_32x32(t_row, r0);
      tmem_ld_32x32(t_row + 32, r1);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
      float va[32], vb[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        va[j] = __uint_as_float(r0[j]);
        vb[j] = __uint_as_float(r1[j]);
      }
      const uint8_t* aux_row = AUX ? aux_buf + lane * 128 : nullptr;
      float ssq = epilogue_chunk(e, g.M, g.N, m0 + quarter * 32, lane, n0 + col_half * 64, rs, rc, va, stage, bias0,
                                 aux_row, 0);
      ssq += epilogue_chunk(e, g.M, g.N, m0 + quarter * 32, lane, n0 + col_half * 64 + 32, rs, rc, vb, stage, bias1,
                            aux_row, 4);
      if (e.q8 != nullptr && m0 + quarter * 32 < g.M && n0 + col_half * 64 < g.N)
        mx_emit_q8(e, g.M, m0 + quarter * 32, n0 + col_half * 64, lane, col_half, va, vb, stage);
      if (e.ssq_out != nullptr && m < g.M)
        e.ssq_out[(size_t)m * e.ssq_parts + (n0 / 64 + col_half)] = ssq;
      if (AUX) {   // this tile's slice is consumed: fetch the next tile's
        __syncwarp();
        aux_pending = false;
        const int next = work + gridDim.x;
        if (next < n_work) {
          int mb2, nb2;
          tile_coords(next % n_tiles, n_tiles_m, n_tiles_n, mb2, nb2);
          aux_pending = aux_prefetch(&tmap_aux, g.M, g.N, mb2 * BM + quarter * 32, lane, nb2 * MX_BN + col_half * 64, 1,
                                     smem_u32(aux_buf), aux_bar);
        }
      }
      if (++acc == MX_ACC) { acc = 0; acc_ph ^= 1; }
    }
  }
  pipe_teardown(bars, warp, MX_TMEM_COLS);
}

// ---------------------------------------------------------------------------------------
// hardware block-scaled FP8 kernel on CTA pairs
// ---------------------------------------------------------------------------------------
// The single-CTA kernel above is bound by the shared-memory fill: a 128 x 128 tile needs 32 KB of operands per
// 128-deep K block, the ring holds about 200 KB, and at the latency of a loaded L2 that caps the rate at which
// stages turn over. Here one MMA spans two CTAs (tcgen05 cta_group::2, 256 x 128 pair tile): each CTA loads its
// own 128 rows of A and 64 of the 128 rows of B, 24 KB per K block for the same 128 x 128 of output, so a ring
// of the same size feeds a third more math. Every CTA needs the scale factors of its own A rows and of all 128
// B rows in its own TMEM; both load the B chunk, and the leader's tcgen05.cp copies them in both CTAs. All
// loads count their bytes on the leader's barrier (the cta_group::2 form of the tiled load, which no
// plain bulk copy has: the scale chunks are therefore fetched through a tensor map over 256-byte rows).
constexpr int MXP_B_ROWS = MX_BN / 2;
constexpr int MXP_B_BYTES = MXP_B_ROWS * STAGE_ROW_BYTES;
constexpr int MXP_STAGE_BYTES = MX_A_BYTES + MXP_B_BYTES + 2 * MX_SF_BYTES;   // 25 KB, a multiple of 1024
constexpr int MXP_STAGES_PLAIN = 8;
constexpr int MXP_STAGES_AUX = 7;

template <bool AUX>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_mx_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                        const __grid_constant__ CUtensorMap tmap_aux, const __grid_constant__ CUtensorMap tmap_out,
                        const __grid_constant__ CUtensorMap tmap_pre, const __grid_constant__ CUtensorMap tmap_q8,
                        const GemmShape g, const GemmEpilogue e, Status* status) {
  constexpr int STAGES = AUX ? MXP_STAGES_AUX : MXP_STAGES_PLAIN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_all = smem + STAGES * MXP_STAGE_BYTES;
  uint8_t* aux_all = stage_all + EPI_STAGE_BYTES;
  PipeBars* bars = reinterpret_cast<PipeBars*>(aux_all + (AUX ? MX_AUX_BYTES : 0));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_sfa);
    tma_prefetch_desc(&tmap_sfb);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < MX_ACC; ++a) {
      mbar_init(smem_u32(&bars->tmem_full[a]), 1);
      mbar_init(smem_u32(&bars->tmem_empty[a]), 2 * EPI_WARPS);
    }
    for (int w = 0; w < 4 * EPI_WARPS; ++w) mbar_init(smem_u32(&bars->aux_full[w]), 1);
    bars->abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&bars->tmem_base), MX_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();     // the peer's barriers exist before anything of this CTA can signal them
  tc_fence_after_sync();
  pdl_enter();
  const uint32_t tmem_base = bars->tmem_base;

  const int n_tiles_n = g.N / MX_BN;
  const int n_tiles_m = g.M / (2 * BM);
  const int n_tiles = n_tiles_m * n_tiles_n;
  const int kblocks = g.K / MX_BK;
  const uint32_t smem0 = smem_u32(smem);
  const uint32_t full0 = smem_u32(&bars->full[0]), empty0 = smem_u32(&bars->empty[0]);
  const uint32_t tfull0 = smem_u32(&bars->tmem_full[0]), tempty0 = smem_u32(&bars->tmem_empty[0]);

  if (warp == 0) {
    {   // all 32 lanes run the loop; one elected lane issues the loads
      const uint32_t full_lead0 = map_to_cta(full0, 0);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
        int mb_, nb_;
        tile_coords(tile, n_tiles_m, n_tiles_n, mb_, nb_);
        const int mblk = mb_ * 2 + (int)rank;                       // this CTA's 128-row block of A
        const int m0 = mblk * BM, nB = nb_ * MX_BN + (int)rank * MXP_B_ROWS;
        int sfa_row = mblk * kblocks * 2, sfb_row = nb_ * kblocks * 2;   // 256-byte rows of the packed scale arrays
        if (g.b_ready != nullptr) {
          // this launch gathers its own B: column block nb_ must have landed in the staging area
          uint32_t there = 1;
          if (lane == 0)
            there = wait_flag_ge_gpu(g.b_ready + nb_, g.b_target, GD_WAIT_BUDGET_NS) &&
                    wait_flag_ge_gpu(g.sfb_ready + nb_, g.sfb_target, GD_WAIT_BUDGET_NS);
          there = __shfl_sync(0xffffffffu, there, 0);
          if (!there) {
            if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_PEER_FLAG, 75, nb_);
            ok = false;
            break;
          }
          fence_proxy_async_global();
        }
        int kx = 0;
        for (int kb = 0; kb < kblocks; ++kb, kx += MX_BK, sfa_row += 2, sfb_row += 2) {
          if (!__all_sync(0xffffffffu, wait_fast(empty0 + 8 * s, ph ^ 1))) {
            if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_SMEM_EMPTY, 70, s);
            ok = false;
            break;
          }
          const uint32_t full = full_lead0 + 8 * s;
          const uint32_t a_dst = smem0 + s * MXP_STAGE_BYTES;
          if (elect_one()) {
            if (rank == 0) mbar_arrive_expect_tx(full0 + 8 * s, 2 * MXP_STAGE_BYTES);
            tma_load_2d_pair(a_dst, &tmap_a, full, kx, m0);
            tma_load_2d_pair(a_dst + MX_A_BYTES, &tmap_b, full, kx, nB);
            tma_load_2d_pair(a_dst + MX_A_BYTES + MXP_B_BYTES, &tmap_sfa, full, 0, sfa_row);
            tma_load_2d_pair(a_dst + MX_A_BYTES + MXP_B_BYTES + MX_SF_BYTES, &tmap_sfb, full, 0, sfb_row);
          }
          __syncwarp();
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (aborted(bars)) break;
      }
    }
  } else if (warp == 1) {
    if (rank == 0) {   // the leader's warp runs the loop with all lanes; one elected lane issues
      const uint32_t idesc = make_instr_desc_mx(2 * BM, MX_BN, 0, 0);
      const uint64_t a_tmpl = make_smem_desc(smem0, 16, 1024), b_tmpl = make_smem_desc(smem0 + MX_A_BYTES, 16, 1024);
      const uint64_t sfa_tmpl = make_smem_desc_noswizzle(smem0 + MX_A_BYTES + MXP_B_BYTES, 16, 128);
      const uint32_t a_hi = (uint32_t)(a_tmpl >> 32), a_lo0 = (uint32_t)a_tmpl;
      const uint32_t b_hi = (uint32_t)(b_tmpl >> 32), b_lo0 = (uint32_t)b_tmpl;
      const uint32_t sf_hi = (uint32_t)(sfa_tmpl >> 32), sf_lo0 = (uint32_t)sfa_tmpl;
      int s = 0, acc = 0, slot = 0;
      uint32_t ph = 0, acc_ph = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
        if (!__all_sync(0xffffffffu, wait_fast(tempty0 + 8 * acc, acc_ph ^ 1))) {
          if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_TMEM_EMPTY, 71, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * MX_BN;
        uint32_t accumulate = 0;
        for (int i = 0; i < kblocks; ++i) {
          if (!__all_sync(0xffffffffu, wait_fast(full0 + 8 * s, ph))) {
            if (lane == 0) raise_abort(bars, status, STATUS_TIMEOUT_SMEM_FULL, 72, s);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t off = s * (MXP_STAGE_BYTES >> 4);
          const uint32_t sfa_t = tmem_base + MX_SF_COL0 + slot * 8, sfb_t = sfa_t + 4;
          if (elect_one()) {
            tmem_cp_scales_pair(sfa_t, desc_at(sf_hi, sf_lo0 + off));
            tmem_cp_scales_pair(sfb_t, desc_at(sf_hi, sf_lo0 + off + (MX_SF_BYTES >> 4)));
#pragma unroll
            for (int k = 0; k < MX_BK / 32; ++k)
              mma_mxfp8_pair(d_tmem, desc_at(a_hi, a_lo0 + off + k * 2), desc_at(b_hi, b_lo0 + off + k * 2),
                             idesc | mx_sf_ids(k), (k == 0) ? accumulate : 1u, sfa_t, sfb_t);
            mma_commit_pair(empty0 + 8 * s);
          }
          __syncwarp();
          accumulate = 1;
          slot ^= 1;
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok || aborted(bars)) break;
        if (elect_one()) mma_commit_pair(tfull0 + 8 * acc);
        __syncwarp();
        if (++acc == MX_ACC) { acc = 0; acc_ph ^= 1; }
      }
    } else if (g.jobs != nullptr) {
      // the second CTA's warp 1 issues no MMAs: it pulls parameter ranges from their owner ranks
      run_gather_jobs(g.jobs, g.n_jobs, pair, n_pairs, lane);
    }
  } else {
    const int ew = warp - 2;
    uint8_t* stage = stage_all + ew * EPI_STAGE_BYTES_PER_WARP;
    const int quarter = warp & 3;
    const int col_half = ew >> 2;        // which 64 of the tile's 128 columns
    const uint32_t tempty_lead0 = map_to_cta(tempty0, 0);
    int acc = 0;
    uint32_t acc_ph = 0;
    const uint32_t aux_slot0 = smem_u32(aux_all + ew * (2 * AUX_CHUNK_BYTES));   // two chunk slots per warp
    const uint8_t* aux_mine = aux_all + ew * (2 * AUX_CHUNK_BYTES) + lane * 64;
    const uint32_t aux_bar0 = smem_u32(&bars->aux_full[ew * 4]);
    uint32_t aux_ph = 0;
    if (AUX && pair < n_tiles) {
      int mb_, nb_;
      tile_coords(pair, n_tiles_m, n_tiles_n, mb_, nb_);
      for (int c = 0; c < 2; ++c)
        aux_request(&tmap_aux, (mb_ * 2 + (int)rank) * BM + quarter * 32, nb_ * MX_BN + col_half * 64 + c * 32,
                    aux_slot0 + c * AUX_CHUNK_BYTES, aux_bar0 + 8 * c);
    }
    for (int tile = pair; tile < n_tiles && !aborted(bars); tile += n_pairs) {
      int mb_, nb_;
      tile_coords(tile, n_tiles_m, n_tiles_n, mb_, nb_);
      const int m0 = (mb_ * 2 + (int)rank) * BM, n0 = nb_ * MX_BN;
      const int m = m0 + quarter * 32 + lane;
      const float rs = (m < g.M) ? row_scale_for(e, m) : 1.0f;
      const float rc = (e.rowcoef != nullptr && m < g.M) ? e.rowcoef[m] : 0.0f;
      const float bias0 = load_bias(e, n0 + col_half * 64 + lane, g.N);
      const float bias1 = load_bias(e, n0 + col_half * 64 + 32 + lane, g.N);
      if (!mbar_wait_warp(tfull0 + 8 * acc, acc_ph)) {
        raise_abort(bars, status, STATUS_TIMEOUT_TMEM_FULL, 73, acc);
        break;
      }
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * MX_BN + col_half * 64;
      uint32_t r0[32], r1[32];
      tmem_ld_32x32(t_row, r0);
      tmem_ld_32x32(t_row + 32, r1);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_lead0 + 8 * acc);
      float va[32], vb[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        va[j] = __uint_as_float(r0[j]);
        vb[j] = __uint_as_float(r1[j]);
      }
      // where the next tile's chunks go (the slots are asked for again as soon as they have been read)
      const int next = tile + n_pairs;
      int m_next = 0, n_next = 0;
      if (AUX && next < n_tiles) {
        int mb2, nb2;
        tile_coords(next, n_tiles_m, n_tiles_n, mb2, nb2);
        m_next = (mb2 * 2 + (int)rank) * BM + quarter * 32;
        n_next = nb2 * MX_BN + col_half * 64;
      }
      float ssq = 0.0f;
      bool aux_ok = true;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        if (AUX) {
          if (!mbar_wait_warp(aux_bar0 + 8 * c, aux_ph)) {
            raise_abort(bars, status, STATUS_TIMEOUT_SMEM_FULL, 74, ew);
            aux_ok = false;
            break;
          }
        }
        ssq += epilogue_chunk(e, g.M, g.N, m0 + quarter * 32, lane, n0 + col_half * 64 + c * 32, rs, rc, c ? vb : va, stage,
                              c ? bias1 : bias0, AUX ? aux_mine + c * AUX_CHUNK_BYTES : nullptr, 0, true,
                              (e.tma_mask & 1) ? &tmap_out : nullptr, (e.tma_mask & 2) ? &tmap_pre : nullptr);
        if (AUX && next < n_tiles) {
          __syncwarp();
          aux_request(&tmap_aux, m_next, n_next + c * 32, aux_slot0 + c * AUX_CHUNK_BYTES, aux_bar0 + 8 * c);
        }
      }
      if (!aux_ok) break;
      aux_ph ^= 1;
      if (e.q8 != nullptr)
        mx_emit_q8(e, g.M, m0 + quarter * 32, n0 + col_half * 64, lane, col_half, va, vb, stage,
                   (e.tma_mask & 4) ? &tmap_q8 : nullptr);
      if (e.ssq_out != nullptr && m < g.M)
        e.ssq_out[(size_t)m * e.ssq_parts + (n0 / 64 + col_half)] = ssq;
      if (++acc == MX_ACC) { acc = 0; acc_ph ^= 1; }
    }
    stage_acquire();   // the last bulk stores have read the staging area
  }

  // teardown: neither CTA may leave (or free its TMEM) while the other can still read its shared memory,
  // write its TMEM or signal its barriers
  tc_fence_before_sync();
  __syncthreads();
  if (aborted(bars)) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, MX_TMEM_COLS);
  }
}

// Stand-alone gather: four warps per block, every warp a worker of run_gather_jobs.
__global__ void __launch_bounds__(128)
gather_jobs_kernel(const int64_t* __restrict__ jobs, int n_jobs) {
  run_gather_jobs(jobs, n_jobs, (int)(blockIdx.x * 4 + (threadIdx.x >> 5)), (int)(gridDim.x * 4), (int)(threadIdx.x & 31));
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows][cols] with a row pitch of ld elements; box = box_rows x (128 bytes of cols).
const char* make_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, int64_t rows, int64_t cols,
                               int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return "cuTensorMapEncodeTiled entry point not found";
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return "tensor base is not 16-byte aligned";
  if ((ld * elem_bytes) % 16 != 0) return "row pitch is not a multiple of 16 bytes";
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld * elem_bytes)};
  cuuint32_t box[2] = {(cuuint32_t)(STAGE_ROW_BYTES / elem_bytes), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? nullptr : "cuTensorMapEncodeTiled failed";
}

// A row-major matrix [rows][cols] (bf16, or bytes with elem_bytes = 1) as boxes of 32 rows x 64 bytes with the 64-byte
// swizzle: the unit of the epilogue's auxiliary loads (aux_request) and bulk stores (store_rows_tma).
static const char* make_tensor_map_box64(CUtensorMap* out, const void* base, int elem_bytes, int64_t rows, int64_t cols,
                                         int64_t ld) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return "cuTensorMapEncodeTiled entry point not found";
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return "matrix is not 16-byte aligned";
  if ((ld * elem_bytes) % 16 != 0) return "row pitch is not a multiple of 16 bytes";
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld * elem_bytes)};
  cuuint32_t box[2] = {(cuuint32_t)(64 / elem_bytes), 32};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? nullptr : "cuTensorMapEncodeTiled failed (64-byte boxes)";
}

static const char* make_tensor_map_aux64(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld) {
  return make_tensor_map_box64(out, base, 2, rows, cols, ld);
}

// Tensor maps for the outputs that can leave through bulk stores (bf16 out without accumulation, pre_out, q8);
// sets es.tma_mask. An output whose base or pitch does not meet the 16-byte rules simply keeps the plain stores.
static void make_store_maps(const GemmShape& g, GemmEpilogue& es, CUtensorMap* t_out, CUtensorMap* t_pre, CUtensorMap* t_q8) {
  es.tma_mask = 0;
  static int on = -1;
  if (on < 0) {
    const char* v = getenv("GDNET_TMA_STORE");
    on = (v == nullptr || v[0] != '0') ? 1 : 0;
  }
  if (!on) return;
  if (es.out != nullptr && !es.out_f32 && !es.accumulate &&
      make_tensor_map_box64(t_out, es.out, 2, g.M, g.N, es.out_ld) == nullptr)
    es.tma_mask |= 1;
  if (es.pre_out != nullptr && make_tensor_map_box64(t_pre, es.pre_out, 2, g.M, g.N, es.pre_ld) == nullptr)
    es.tma_mask |= 2;
  if (es.q8 != nullptr && make_tensor_map_box64(t_q8, es.q8, 1, g.M, g.N, es.q8_ld) == nullptr) es.tma_mask |= 4;
}

// Packed UE8M0 scale chunks (512 bytes each, n_chunks of them back to back) as a tensor of 256-byte rows: a box
// of two rows is one chunk and lands in shared memory exactly as it lies in global memory (no swizzle).
static const char* make_tensor_map_chunks(CUtensorMap* out, const void* base, int64_t n_chunks) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return "cuTensorMapEncodeTiled entry point not found";
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return "packed scales are not 16-byte aligned";
  cuuint64_t dims[2] = {256, (cuuint64_t)(n_chunks * 2)};
  cuuint64_t strides[1] = {256};
  cuuint32_t box[2] = {256, 2};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? nullptr : "cuTensorMapEncodeTiled failed (scale chunks)";
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

// Split the reduction over several CTAs when the output has too few tiles to fill the GPU (weight
// gradients: small output, reduction over all tokens). Only for a plain fp32 "out += acc" epilogue,
// whose additions can be done with atomics in any order.
static int pick_splits(int tiles, int kblocks, const GemmEpilogue& e) {
  const bool plain = e.out_f32 && e.accumulate && e.bias == nullptr && e.aux == nullptr && e.pre_out == nullptr &&
                     e.act == ACT_NONE && e.row_scale == nullptr && e.ssq_in == nullptr && e.ssq_out == nullptr;
  if (!plain || tiles * 2 > sm_count()) return 1;
  // (more shares per tile, chosen so that the rounds of work items fill the CTA pairs evenly, were measured slower:
  // 61.1 against 57.7 us for the 1024 x 1024 weight gradient; the extra atomics cost more than the idle pairs)
  int s = sm_count() / tiles;
  if (s > kblocks / 4) s = kblocks / 4;   // keep at least four K blocks per share
  if (s < 1) return 1;
  const int per = (kblocks + s - 1) / s;
  return (kblocks + per - 1) / per;       // no share may be empty: an empty one would publish a stale accumulator
}

// CTA pairs that can be resident at once (a pair needs two free SMs of one TPC; fewer than sm_count / 2 when a
// GPC has an odd number of usable SMs). 0 = cluster launch not possible, use the single-CTA kernel.
template <typename KernelT>
static int max_active_pairs(KernelT kernel, int smem) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(sm_count() & ~1));
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = (size_t)smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

static bool pair_kernels_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* v = getenv("GDNET_GEMM_PAIR");
    on = (v == nullptr || v[0] != '0') ? 1 : 0;
  }
  return on == 1;
}

static const char* launch_gemm_bf16_pair(const GemmOperands& op, const GemmShape& g, const GemmEpilogue& e,
                                         Status* status, cudaStream_t stream, bool* launched) {
  *launched = false;
  static int pairs_plain = -1, pairs_aux = -1;
  const bool aux = e.aux != nullptr;
  const int smem_plain = 6 * PAIR_STAGE_BYTES + EPI_STAGE_BYTES + (int)sizeof(PipeBars) + 1024;
  const int smem_aux = 4 * PAIR_STAGE_BYTES + EPI_STAGE_BYTES + BF16_AUX_BYTES + (int)sizeof(PipeBars) + 1024;
  if (pairs_plain < 0) {
    pairs_plain = pairs_aux = 0;
    if (cudaFuncSetAttribute(gemm_bf16_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_plain) == cudaSuccess &&
        cudaFuncSetAttribute(gemm_bf16_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_aux) == cudaSuccess) {
      pairs_plain = max_active_pairs(gemm_bf16_pair_kernel<false>, smem_plain);
      pairs_aux = max_active_pairs(gemm_bf16_pair_kernel<true>, smem_aux);
    } else {
      (void)cudaGetLastError();
    }
  }
  const int max_pairs = aux ? pairs_aux : pairs_plain;
  if (max_pairs < 1) return nullptr;
  CUtensorMap ta, tb, tx;
  const char* err;
  if (!g.a_mn) err = make_tensor_map_2d(&ta, op.a, 2, g.M, g.K, op.a_ld, BM);
  else err = make_tensor_map_2d(&ta, op.a, 2, g.K, g.M, op.a_ld, BF16_BK);
  if (err) return err;
  if (!g.b_mn) err = make_tensor_map_2d(&tb, op.b, 2, g.N, g.K, op.b_ld, PAIR_B_ROWS);
  else err = make_tensor_map_2d(&tb, op.b, 2, g.K, g.N, op.b_ld, BF16_BK);
  if (err) return err;
  const int tiles = ((g.M + 2 * BM - 1) / (2 * BM)) * ((g.N + PAIR_BN - 1) / PAIR_BN);
  GemmShape gs = g;
  GemmEpilogue es = e;
  gs.splits = pick_splits(tiles * 2, (g.K + BF16_BK - 1) / BF16_BK, e);
  es.atomic = gs.splits > 1;
  CUtensorMap to = ta, tp = ta, tq = ta;
  make_store_maps(g, es, &to, &tp, &tq);
  const int work = tiles * gs.splits;
  const int grid = 2 * (work < max_pairs ? work : max_pairs);
  if (aux) {
    if ((err = make_tensor_map_aux64(&tx, e.aux, g.M, g.N, e.aux_ld)) != nullptr) return err;
    launch_pdl(gemm_bf16_pair_kernel<true>, dim3(grid), dim3(NUM_THREADS), smem_aux, stream, ta, tb, tx, to, tp, gs, es, status);
  } else {
    launch_pdl(gemm_bf16_pair_kernel<false>, dim3(grid), dim3(NUM_THREADS), smem_plain, stream, ta, tb, ta, to, tp, gs, es, status);
  }
  *launched = true;
  return cudaGetLastError() == cudaSuccess ? nullptr : "gemm_bf16_pair_kernel launch failed";
}

int gemm_pair_capacity() {
  const int smem_plain = 6 * PAIR_STAGE_BYTES + EPI_STAGE_BYTES + (int)sizeof(PipeBars) + 1024;
  if (cudaFuncSetAttribute(gemm_bf16_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_plain) != cudaSuccess) {
    (void)cudaGetLastError();
    return -1;
  }
  return max_active_pairs(gemm_bf16_pair_kernel<false>, smem_plain);
}

const char* launch_gemm_bf16(const GemmOperands& op, const GemmShape& g, const GemmEpilogue& e, Status* status,
                             cudaStream_t stream) {
  if (g.K % 8 != 0 || g.N % 32 != 0) return "bf16 GEMM needs K % 8 == 0 and N % 32 == 0";
  if (pair_kernels_enabled() && g.M >= 2 * BM && g.N >= PAIR_BN / 2) {
    bool launched = false;
    const char* perr = launch_gemm_bf16_pair(op, g, e, status, stream, &launched);
    if (perr != nullptr || launched) return perr;
  }
  CUtensorMap ta, tb;
  const char* err;
  if (g.jobs != nullptr && (err = launch_gather_jobs(g.jobs, g.n_jobs, stream)) != nullptr) return err;
  if (!g.a_mn) err = make_tensor_map_2d(&ta, op.a, 2, g.M, g.K, op.a_ld, BM);
  else err = make_tensor_map_2d(&ta, op.a, 2, g.K, g.M, op.a_ld, BF16_BK);   // rows = reduction, cols = M
  if (err) return err;
  if (!g.b_mn) err = make_tensor_map_2d(&tb, op.b, 2, g.N, g.K, op.b_ld, BF16_BN);
  else err = make_tensor_map_2d(&tb, op.b, 2, g.K, g.N, op.b_ld, BF16_BK);
  if (err) return err;
  static bool attr_set = false;
  const bool aux = e.aux != nullptr;
  const int smem_plain = 4 * BF16_STAGE_BYTES + EPI_STAGE_BYTES + (int)sizeof(PipeBars) + 1024;
  const int smem_aux = 3 * BF16_STAGE_BYTES + EPI_STAGE_BYTES + BF16_AUX_BYTES + (int)sizeof(PipeBars) + 1024;
  const int smem = aux ? smem_aux : smem_plain;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_bf16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_plain) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_bf16_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_aux) != cudaSuccess)
      return "cudaFuncSetAttribute(gemm_bf16_kernel) failed";
    attr_set = true;
  }
  const int tiles = ((g.M + BM - 1) / BM) * ((g.N + BF16_BN - 1) / BF16_BN);
  GemmShape gs = g;
  GemmEpilogue es = e;
  gs.splits = pick_splits(tiles, (g.K + BF16_BK - 1) / BF16_BK, e);
  es.atomic = gs.splits > 1;
  const int work = tiles * gs.splits;
  const int grid = work < sm_count() ? work : sm_count();
  if (aux) {
    CUtensorMap tx;
    if ((err = make_tensor_map_2d(&tx, e.aux, 2, g.M, g.N, e.aux_ld, 32)) != nullptr) return err;
    launch_pdl(gemm_bf16_kernel<true>, dim3(grid), dim3(NUM_THREADS), smem, stream, ta, tb, tx, gs, es, status);
  } else {
    launch_pdl(gemm_bf16_kernel<false>, dim3(grid), dim3(NUM_THREADS), smem, stream, ta, tb, ta, gs, es, status);
  }
  return cudaGetLastError() == cudaSuccess ? nullptr : "gemm_bf16_kernel launch failed";
}

const char* launch_gemm_fp8(const GemmOperands& op, const GemmShape& g, const GemmEpilogue& e, Status* status,
                            cudaStream_t stream) {
  if (g.K % 128 != 0 || g.N % 64 != 0) return "fp8 GEMM needs K % 128 == 0 and N % 64 == 0";
  if (g.sa == nullptr || g.sb == nullptr) return "fp8 GEMM needs block scales";
  CUtensorMap ta, tb;
  const char* err = make_tensor_map_2d(&ta, op.a, 1, g.M, g.K, op.a_ld, BM);
  if (err) return err;
  err = make_tensor_map_2d(&tb, op.b, 1, g.N, g.K, op.b_ld, FP8_BN);
  if (err) return err;
  static bool attr_set = false;
  const int smem = FP8_STAGES * FP8_STAGE_BYTES + EPI_STAGE_BYTES + (int)sizeof(PipeBars) + 1024;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return "cudaFuncSetAttribute(gemm_fp8_kernel) failed";
    attr_set = true;
  }
  const int tiles = ((g.M + BM - 1) / BM) * ((g.N + FP8_BN - 1) / FP8_BN);
  GemmShape gs = g;
  GemmEpilogue es = e;
  gs.splits = pick_splits(tiles, (g.K + FP8_BK - 1) / FP8_BK, e);
  es.atomic = gs.splits > 1;
  const int work = tiles * gs.splits;
  const int grid = work < sm_count() ? work : sm_count();
  gemm_fp8_kernel<<<grid, NUM_THREADS, smem, stream>>>(ta, tb, gs, es, status);
  return cudaGetLastError() == cudaSuccess ? nullptr : "gemm_fp8_kernel launch failed";
}

const char* launch_gather_jobs(const int64_t* jobs, int n_jobs, cudaStream_t stream) {
  if (n_jobs <= 0) return nullptr;
  int blocks = (n_jobs + 3) / 4;
  if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
  gather_jobs_kernel<<<blocks, 128, 0, stream>>>(jobs, n_jobs);
  return cudaGetLastError() == cudaSuccess ? nullptr : "gather_jobs_kernel launch failed";
}

static int g_mx_pair = -1;   // -1: take GDNET_MX_PAIR from the environment on first use

void gemm_set_mx_pair(int on) { g_mx_pair = on ? 1 : 0; }

static bool mx_pair_enabled() {
  if (g_mx_pair < 0) {
    const char* v = getenv("GDNET_MX_PAIR");
    g_mx_pair = (v == nullptr || v[0] != '0') ? 1 : 0;
  }
  return g_mx_pair == 1 && pair_kernels_enabled();
}

// CTA-pair form of the hardware-scaled FP8 GEMM (256 x 128 pair tiles). *launched stays false when pairs cannot
// be launched on this device; the caller then uses the single-CTA kernel.
static const char* launch_gemm_fp8_mx_pair(const GemmOperands& op, const GemmShape& g, const GemmEpilogue& e,
                                           Status* status, cudaStream_t stream, bool* launched) {
  *launched = false;
  static int pairs_plain = -1, pairs_aux = -1;
  const bool aux = e.aux != nullptr;
  const int smem_plain = MXP_STAGES_PLAIN * MXP_STAGE_BYTES + EPI_STAGE_BYTES + (int)sizeof(PipeBars) + 1024;
  const int smem_aux = MXP_STAGES_AUX * MXP_STAGE_BYTES + EPI_STAGE_BYTES + MX_AUX_BYTES + (int)sizeof(PipeBars) + 1024;
  if (pairs_plain < 0) {
    pairs_plain = pairs_aux = 0;
    if (cudaFuncSetAttribute(gemm_fp8_mx_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_plain) == cudaSuccess &&
        cudaFuncSetAttribute(gemm_fp8_mx_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_aux) == cudaSuccess) {
      pairs_plain = max_active_pairs(gemm_fp8_mx_pair_kernel<false>, smem_plain);
      pairs_aux = max_active_pairs(gemm_fp8_mx_pair_kernel<true>, smem_aux);
    } else {
      (void)cudaGetLastError();
    }
  }
  const int max_pairs = aux ? pairs_aux : pairs_plain;
  if (max_pairs < 1) return nullptr;
  CUtensorMap ta, tb, tsa, tsb, tx;
  const char* err;
  if ((err = make_tensor_map_2d(&ta, op.a, 1, g.M, g.K, op.a_ld, BM)) != nullptr) return err;
  if ((err = make_tensor_map_2d(&tb, op.b, 1, g.N, g.K, op.b_ld, MXP_B_ROWS)) != nullptr) return err;
  const int64_t kblocks = g.K / MX_BK;
  if ((err = make_tensor_map_chunks(&tsa, g.sfa_packed, (g.M / BM) * kblocks)) != nullptr) return err;
  if ((err = make_tensor_map_chunks(&tsb, g.sfb_packed, (g.N / MX_BN) * kblocks)) != nullptr) return err;
  const int tiles = (g.M / (2 * BM)) * (g.N / MX_BN);
  GemmShape gs = g;
  GemmEpilogue es = e;
  gs.splits = 1;
  es.atomic = 0;
  CUtensorMap to = ta, tp = ta, tq = ta;
  make_store_maps(g, es, &to, &tp, &tq);
  const int grid = 2 * (tiles < max_pairs ? tiles : max_pairs);
  if (aux) {
    if ((err = make_tensor_map_aux64(&tx, e.aux, g.M, g.N, e.aux_ld)) != nullptr) return err;
    launch_pdl(gemm_fp8_mx_pair_kernel<true>, dim3(grid), dim3(NUM_THREADS), smem_aux, stream, ta, tb, tsa, tsb, tx, to, tp, tq, gs,
               es, status);
  } else {
    launch_pdl(gemm_fp8_mx_pair_kernel<false>, dim3(grid), dim3(NUM_THREADS), smem_plain, stream, ta, tb, tsa, tsb, ta, to, tp, tq,
               gs, es, status);
  }
  *launched = true;
  return cudaGetLastError() == cudaSuccess ? nullptr : "gemm_fp8_mx_pair_kernel launch failed";
}

const char* launch_gemm_fp8_mx(const GemmOperands& op, const GemmShape& g, const GemmEpilogue& e, Status* status,
                               cudaStream_t stream) {
  if (g.K % 128 != 0 || g.N % 128 != 0 || g.M % 128 != 0) return "hardware-scaled fp8 GEMM needs M, N, K % 128 == 0";
  if (g.sfa_packed == nullptr || g.sfb_packed == nullptr) return "hardware-scaled fp8 GEMM needs packed scales";
  if (mx_pair_enabled() && g.M % (2 * BM) == 0 && pick_splits((g.M / BM) * (g.N / MX_BN), g.K / MX_BK, e) == 1) {
    bool launched = false;
    const char* perr = launch_gemm_fp8_mx_pair(op, g, e, status, stream, &launched);
    if (perr != nullptr || launched) return perr;
  }
  CUtensorMap ta, tb;
  const char* err;
  // the single-CTA kernel carries no gather jobs: copy first, in stream order (its B is then complete)
  if (g.jobs != nullptr && (err = launch_gather_jobs(g.jobs, g.n_jobs, stream)) != nullptr) return err;
  err = make_tensor_map_2d(&ta, op.a, 1, g.M, g.K, op.a_ld, BM);
  if (err) return err;
  err = make_tensor_map_2d(&tb, op.b, 1, g.N, g.K, op.b_ld, MX_BN);
  if (err) return err;
  static bool attr_set = false;
  const bool aux = e.aux != nullptr;
  const int smem_plain = 6 * MX_STAGE_BYTES + EPI_STAGE_BYTES + (int)sizeof(PipeBars) + 1024;
  const int smem_aux = 5 * MX_STAGE_BYTES + EPI_STAGE_BYTES + MX_AUX_BYTES + (int)sizeof(PipeBars) + 1024;
  const int smem = aux ? smem_aux : smem_plain;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_fp8_mx_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_plain) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_fp8_mx_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_aux) != cudaSuccess)
      return "cudaFuncSetAttribute(gemm_fp8_mx_kernel) failed";
    attr_set = true;
  }
  const int tiles = (g.M / BM) * (g.N / MX_BN);
  GemmShape gs = g;
  GemmEpilogue es = e;
  gs.splits = pick_splits(tiles, g.K / MX_BK, e);
  es.atomic = gs.splits > 1;
  const int work = tiles * gs.splits;
  const int grid = work < sm_count() ? work : sm_count();
  if (aux) {
    CUtensorMap tx;
    if ((err = make_tensor_map_2d(&tx, e.aux, 2, g.M, g.N, e.aux_ld, 32)) != nullptr) return err;
    launch_pdl(gemm_fp8_mx_kernel<true>, dim3(grid), dim3(NUM_THREADS), smem, stream, ta, tb, tx, gs, es, status);
  } else {
    launch_pdl(gemm_fp8_mx_kernel<false>, dim3(grid), dim3(NUM_THREADS), smem, stream, ta, tb, ta, gs, es, status);
  }
  return cudaGetLastError() == cudaSuccess ? nullptr : "gemm_fp8_mx_kernel launch failed";
}

}  // namespace gd
