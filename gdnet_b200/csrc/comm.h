// Kernels that fuse compute with communication over NVLink peer memory (comm.cu).
//
// Peer buffers are ordinary device pointers into other GPUs' memory (CUDA VMM mappings made
// by torch's symmetric-memory allocator). The kernels read and write them with plain
// vectorised loads and stores plus system-scope release/acquire flags; there is no bulk
// tensor copy with a cluster-wide broadcast anywhere in this file.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gd {

struct Status;

// Gradient all-reduce (as reduce-scatter over peer memory) fused with the gradient projection,
// the AdamW update of this rank's shard and the all-gather of the updated parameters.
//
//   phase 0: everything in one launch (no gradient clipping)
//   phase 1: barrier, reduce this rank's shard of both gradients in place, shard dot products
//   phase 2: AdamW on the shard (scalars now hold the clip factor), write the new parameters
//            into every rank's parameter buffer, closing barrier
//
// When the producers have already added their gradients into the owner's shard (weight-gradient GEMM
// epilogues and peer_add, i.e. the reduce-scatter happened tile by tile during backward):
//   phase 3: barrier, shard dot products of the mean gradients
//   phase 4: AdamW on the shard, all-gather of the parameters, shard cleared, closing barrier
//   phase 5: 3 and 4 in one launch (scalars known beforehand)
//
// Overlap with backward: the task gradient is final after the first backward pass of a step, so
//   phase 6: barrier (its own flag slot), reduce this rank's shard of the TASK gradient only, mean into t_red
// runs on a side stream while the second backward pass computes the information gradient. Phases 0-2 then take
// the reduced task shard from t_red and pull only the information gradient: half the bytes after backward.
struct FusedReduceAdamWArgs {
  float* const* gt;        // [world] task-gradient buffers (fp32, n elements each)
  float* const* gi;        // [world] info-gradient buffers
  void* const* p;          // [world] parameter buffers (bf16 or fp32, n elements each)
  uint32_t* const* signals;  // [world] flag words: signals[r][phase_slot * world + writer]
  float* m;                // AdamW moments of the local shard (shard_len elements)
  float* v;
  const float* scalars;    // [coef, grad_scale]
  float* shard_sums;       // [3] += sum GT^2, sum GT*GI, sum GI^2 over the reduced shard; [4] block counter
  float* t_red;            // shard_len floats or null: the reduced task gradient of this rank's shard (see phase 6)
  const float* gt_mc;      // null, or the NVLink multicast address of the task-gradient buffers (every rank's buffer
  const float* gi_mc;      // bound at the same offset): the sum over ranks is then one multimem.ld_reduce per vector,
  void* p_mc;              // added inside the switch, and the updated shard reaches every rank by one multimem.st
  unsigned long long* timing;  // null or 4 words of %globaltimer (ns): kernel start, opening barrier passed,
                               // last block done with its elements, closing barrier passed
  int64_t n;
  int rank, world;
  uint32_t seq;            // strictly increasing per call pair
  int p_is_bf16;
  int gather_params;       // 1: store the updated shard into every rank's parameter buffer; 0: this rank's only
                           // (parameters sharded over the ranks: p[rank] is the shard base minus the shard offset)
  int phase;
  float beta_proj, lr, beta1, beta2, eps, weight_decay, bc1, bc2;
  Status* status;
};
const char* launch_fused_reduce_adamw(const FusedReduceAdamWArgs& a, cudaStream_t st);

// dst_flat[flat_off + i] += src[i] for i < n, where dst_flat is the flat gradient buffer spread over the
// ranks: element idx lives in table[idx / shard_elems] (vector atomics, local or over NVLink).
struct PeerAddArgs {
  const void* src;          // n contiguous fp32 or bf16 values
  int src_bf16;
  float* const* table;      // [world] flat fp32 gradient buffers
  int64_t flat_off, n, shard_elems;
};
const char* launch_peer_add(const PeerAddArgs& a, cudaStream_t st);

// One-shot MAX all-reduce of a small fp32 vector (the amax windows of the per-tensor FP8 recipe): every rank
// stores its vector into its slot of every rank's exchange area, raises a flag there, waits (bounded) for all
// flags and takes the element-wise maximum. One launch, one block.
struct MaxAllReduceArgs {
  float* vec;               // n values, in place
  int n;
  float* const* areas;      // [world] exchange areas: 2 * world slots of `slot_elems` floats each
  uint32_t* const* flags;   // [world] flag words: flags[r][writer]
  int slot_elems;
  int rank, world;
  uint32_t seq;             // strictly increasing per call
  uint64_t budget_ns;       // time limit of the wait for the peers' flags; 0 = the library default (2 s)
  float* gather_out;        // null: element-wise MAX into vec. Else an all-gather: gather_out[r * n + i] = rank r's vec[i]
  Status* status;
};
const char* launch_max_allreduce(const MaxAllReduceArgs& a, cudaStream_t st);

// Sequence-parallel neighbour exchange: store `tail` into the next rank's slot, raise its flag,
// wait (bounded) for this rank's own flag from the previous rank, copy the slot out.
// reverse = true exchanges in the other direction (halo gradients).
struct HaloArgs {
  const void* tail;
  void* halo_out;
  int64_t nbytes;
  uint8_t* const* slots;   // [world] base of every rank's slot area
  uint32_t* const* flags;  // [world] base of every rank's flag area
  int64_t slot_offset;     // byte offset of this exchange's slot
  int flag_index;
  int rank, world;
  uint32_t seq;
  int reverse;
  uint64_t budget_ns;      // time limit of the wait for the neighbour's flag; 0 = the library default (2 s)
  Status* status;
};
const char* launch_halo_push_wait(const HaloArgs& a, cudaStream_t st);

}  // namespace gd
