// torch.ops.gdnet_b200.* : thin, checked bindings from tensors to the kernel launchers.
// Every op validates device, dtype, contiguity of the innermost dimension and alignment on the
// host, launches on the current CUDA stream and never synchronises.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <nvtx3/nvToolsExt.h>

#include <cstdlib>

#include "comm.h"
#include "gemm_sm100.h"
#include "kernels.h"

namespace {

using at::Tensor;
using OptT = const std::optional<Tensor>&;

// NVTX range around every op (named after the binding), for timeline tools; on with GDNET_NVTX=1.
struct OpRange {
  bool on;
  explicit OpRange(const char* name) : on(enabled()) {
    if (on) nvtxRangePushA(name);
  }
  ~OpRange() {
    if (on) nvtxRangePop();
  }
  static bool enabled() {
    static int v = -1;
    if (v < 0) {
      const char* e = std::getenv("GDNET_NVTX");
      v = (e != nullptr && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
  }
};

#define GD_LAUNCH(expr)                                             \
  do {                                                              \
    const char* gd_err_ = (expr);                                   \
    TORCH_CHECK(gd_err_ == nullptr, "gdnet_b200: ", gd_err_);       \
  } while (0)

cudaStream_t stream_of(const Tensor& t) { return c10::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

void check_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.dim() == 0 || t.stride(-1) == 1 || t.size(-1) == 1, name, " must be contiguous in its last dim");
}

const __nv_bfloat16* bf16_ptr(const Tensor& t, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name, " must be 16-byte aligned");
  return reinterpret_cast<const __nv_bfloat16*>(t.data_ptr());
}
__nv_bfloat16* bf16_mut(const Tensor& t, const char* name) { return const_cast<__nv_bfloat16*>(bf16_ptr(t, name)); }

const float* f32_ptr(const Tensor& t, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == at::kFloat, name, " must be float32");
  return t.data_ptr<float>();
}
float* f32_mut(const Tensor& t, const char* name) { return const_cast<float*>(f32_ptr(t, name)); }

const float* opt_f32(OptT t, const char* name) { return t.has_value() ? f32_ptr(*t, name) : nullptr; }
const __nv_bfloat16* opt_bf16(OptT t, const char* name) { return t.has_value() ? bf16_ptr(*t, name) : nullptr; }

uint8_t* fp8_mut(const Tensor& t, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.element_size() == 1, name, " must be an 8-bit tensor");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name, " must be 16-byte aligned");
  return reinterpret_cast<uint8_t*>(t.data_ptr());
}

Tensor& status_tensor(int device) {
  static std::vector<Tensor> per_device(64);
  TORCH_CHECK(device >= 0 && device < 64, "bad device index");
  if (!per_device[device].defined())
    per_device[device] = at::zeros({4}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
  return per_device[device];
}

gd::Status* status_ptr(const Tensor& like) {
  return reinterpret_cast<gd::Status*>(status_tensor(like.get_device()).data_ptr());
}

Tensor kernel_status(const Tensor& like) { return status_tensor(like.get_device()); }

// Flat gradient buffers whose contents are spread over the ranks ("grad sinks"): a weight-gradient GEMM or a
// peer_add whose destination lies inside a registered buffer adds into the owner rank's copy instead.
struct GradSink {
  uintptr_t base;
  int64_t elems;    // > 0: a local full-size buffer starts at `base`; < 0: virtual (|elems| flat elements, no local buffer)
  Tensor table;     // int64 device tensor: the buffer's address on every rank
  int64_t shard_elems;
  int64_t id;
};

std::vector<GradSink>& grad_sinks() {
  static std::vector<GradSink> sinks;
  return sinks;
}

int64_t next_sink_id() {
  static int64_t next = 0;
  return next++;
}

const GradSink* find_sink(const void* p) {
  const uintptr_t u = reinterpret_cast<uintptr_t>(p);
  for (const GradSink& s : grad_sinks())
    if (s.elems > 0 && u >= s.base && u < s.base + (uintptr_t)s.elems * 4) return &s;
  return nullptr;
}

// Every training engine registers the buffers it spreads over the ranks and removes them again when it is closed, so
// several engines can live in one process. Returns the handle for unregister_grad_sink.
int64_t register_grad_sink(const Tensor& flat, const Tensor& ptr_table, int64_t shard_elems) {
  TORCH_CHECK(flat.is_cuda() && flat.scalar_type() == at::kFloat && flat.is_contiguous(), "grad sink must be flat fp32");
  TORCH_CHECK(ptr_table.is_cuda() && ptr_table.scalar_type() == at::kLong, "ptr_table must be an int64 CUDA tensor");
  TORCH_CHECK(shard_elems > 0 && shard_elems % 128 == 0, "shard_elems must be a positive multiple of 128");
  TORCH_CHECK(flat.numel() <= shard_elems * ptr_table.numel(), "shards do not cover the buffer");
  const int64_t id = next_sink_id();
  grad_sinks().push_back({reinterpret_cast<uintptr_t>(flat.data_ptr()), flat.numel(), ptr_table, shard_elems, id});
  return id;
}

// A sink without a local full-size buffer (parameters sharded over the ranks: every rank holds only its own
// shard of the flat gradient). Gradients are addressed by (sink handle, flat element offset); ptr_table[r] is
// rank r's shard base minus r * shard_elems elements, so that table[idx / shard_elems] + idx is element idx.
int64_t register_virtual_grad_sink(const Tensor& ptr_table, int64_t total_elems, int64_t shard_elems) {
  TORCH_CHECK(ptr_table.is_cuda() && ptr_table.scalar_type() == at::kLong, "ptr_table must be an int64 CUDA tensor");
  TORCH_CHECK(shard_elems > 0 && shard_elems % 128 == 0, "shard_elems must be a positive multiple of 128");
  TORCH_CHECK(total_elems <= shard_elems * ptr_table.numel(), "shards do not cover the buffer");
  const int64_t id = next_sink_id();
  grad_sinks().push_back({0, -total_elems, ptr_table, shard_elems, id});     // elems < 0: never matched by address
  return id;
}

void unregister_grad_sink(int64_t id) {
  auto& v = grad_sinks();
  for (size_t i = 0; i < v.size(); ++i)
    if (v[i].id == id) {
      v.erase(v.begin() + (long)i);
      return;
    }
}

const GradSink& sink_at(int64_t id) {
  for (const GradSink& s : grad_sinks())
    if (s.id == id) return s;
  TORCH_CHECK(false, "unknown gradient sink ", id);
}

bool is_spread(const Tensor& t) { return t.is_cuda() && find_sink(t.data_ptr()) != nullptr; }

// One-shot attachments for the next tensor-core GEMM launched from this thread: a list of peer -> local gather
// jobs that the launch carries, and the counters that tell the hardware-scaled fp8 GEMM when its own B has landed.
struct PendingGather {
  std::optional<Tensor> jobs, b_ready, sfb_ready;
  int64_t b_target = 0, sfb_target = 0;
};
PendingGather& pending_gather() {
  static thread_local PendingGather p;
  return p;
}

void attach_gather_jobs(const Tensor& jobs) {
  TORCH_CHECK(jobs.is_cuda() && jobs.scalar_type() == at::kLong && jobs.is_contiguous() && jobs.dim() == 2 && jobs.size(1) == 4,
              "gather jobs must be a contiguous int64 CUDA tensor (n, 4): src, dst, counter, 16-byte vectors");
  pending_gather().jobs = jobs;
}

void attach_b_ready(const Tensor& b_ready, const Tensor& sfb_ready, int64_t b_target, int64_t sfb_target) {
  TORCH_CHECK(b_ready.is_cuda() && sfb_ready.is_cuda() && b_ready.scalar_type() == at::kInt &&
              sfb_ready.scalar_type() == at::kInt && b_ready.is_contiguous() && sfb_ready.is_contiguous(),
              "ready counters must be contiguous int32 CUDA tensors");
  PendingGather& p = pending_gather();
  p.b_ready = b_ready;
  p.sfb_ready = sfb_ready;
  p.b_target = b_target;
  p.sfb_target = sfb_target;
}

void take_pending_gather(gd::GemmShape& g, int64_t n_blocks, bool may_wait) {
  PendingGather& p = pending_gather();
  if (p.jobs.has_value()) {
    g.jobs = p.jobs->data_ptr<int64_t>();
    g.n_jobs = (int)p.jobs->size(0);
    p.jobs.reset();
  }
  if (p.b_ready.has_value()) {
    TORCH_CHECK(may_wait, "only the hardware-scaled fp8 GEMM can wait for a gathered B operand");
    TORCH_CHECK(p.b_ready->numel() >= n_blocks && p.sfb_ready->numel() >= n_blocks, "one ready counter per 128 rows of B");
    g.b_ready = reinterpret_cast<const uint32_t*>(p.b_ready->data_ptr<int>());
    g.sfb_ready = reinterpret_cast<const uint32_t*>(p.sfb_ready->data_ptr<int>());
    g.b_target = (uint32_t)p.b_target;
    g.sfb_target = (uint32_t)p.sfb_target;
    p.b_ready.reset();
    p.sfb_ready.reset();
  }
}

void clear_grad_sinks() { grad_sinks().clear(); }

void gather_jobs(const Tensor& jobs) {
  c10::cuda::CUDAGuard guard(jobs.device());
  TORCH_CHECK(jobs.is_cuda() && jobs.scalar_type() == at::kLong && jobs.is_contiguous() && jobs.dim() == 2 && jobs.size(1) == 4,
              "gather jobs must be a contiguous int64 CUDA tensor (n, 4)");
  GD_LAUNCH(gd::launch_gather_jobs(jobs.data_ptr<int64_t>(), (int)jobs.size(0), stream_of(jobs)));
}

// Optional fused 1x128 FP8 copy of a (rows, cols) output: q (rows, cols) e4m3 (may be a column range of a wider
// buffer), s (cols/128, rows) fp32 (rows of a taller buffer), p (rows/128, cols/128, 512) packed chunks.
gd::RowQuantOut row_quant_out(OptT q, OptT s, OptT p, int64_t rows, int64_t cols) {
  gd::RowQuantOut o{};
  if (!q.has_value()) return o;
  TORCH_CHECK(s.has_value() && p.has_value(), "a quantised output needs q, s and p");
  TORCH_CHECK(rows % 128 == 0 && cols % 128 == 0, "a quantised output needs rows and cols to be multiples of 128");
  TORCH_CHECK(q->dim() == 2 && q->size(0) == rows && q->size(1) == cols && q->stride(1) == 1, "q must be (rows, cols)");
  TORCH_CHECK(s->dim() == 2 && s->size(0) == cols / 128 && s->size(1) == rows && s->stride(1) == 1 &&
              s->scalar_type() == at::kFloat, "s must be (cols/128, rows) float32");
  TORCH_CHECK(p->dim() == 3 && p->size(0) == rows / 128 && p->size(1) == cols / 128 && p->size(2) == 512 &&
              p->stride(2) == 1 && p->stride(1) == 512 && p->stride(0) % 512 == 0, "p must be (rows/128, cols/128, 512) bytes");
  o.q = fp8_mut(*q, "q");
  TORCH_CHECK(q->stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(o.q) & 7) == 0, "q rows must be 8-byte aligned");
  o.q_ld = q->stride(0);
  o.s = s->data_ptr<float>();
  o.s_ld = s->stride(0);
  o.p = fp8_mut(*p, "p");
  o.p_stride = p->stride(0) / 512;
  return o;
}

void fill_epilogue(gd::GemmEpilogue& e, const Tensor& out, bool accumulate, OptT bias, OptT row_scale, OptT ssq_in,
                   int64_t norm_dim, double norm_eps, OptT aux, int64_t aux_mode, OptT rowcoef, OptT pre_out,
                   int64_t act, OptT ssq_out, int64_t M, int64_t N) {
  check_cuda(out, "out");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == M && out.size(1) == N, "out must be (M, N)");
  e.out = out.data_ptr();
  e.out_ld = out.stride(0);
  e.out_f32 = out.scalar_type() == at::kFloat;
  TORCH_CHECK(e.out_f32 || out.scalar_type() == at::kBFloat16, "out must be bfloat16 or float32");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0 && (e.out_ld * out.element_size()) % 16 == 0,
              "out rows must be 16-byte aligned");
  e.accumulate = accumulate;
  e.atomic = 0;
  e.peer_out = nullptr;
  e.flat_off = 0;
  e.shard_elems = 1;
  e.q8 = nullptr;
  e.q8_ld = 0;
  e.q8_p = nullptr;
  e.q8_p_stride = 0;
  e.q8_silu = 0;
  if (e.out_f32 && accumulate) {
    if (const GradSink* s = find_sink(out.data_ptr())) {
      TORCH_CHECK(out.stride(1) == 1 && out.stride(0) % 32 == 0 && N % 32 == 0,
                  "a gradient inside a spread flat buffer needs unit column stride and 32-element granularity");
      e.peer_out = reinterpret_cast<float* const*>(s->table.data_ptr<int64_t>());
      e.flat_off = (int64_t)((reinterpret_cast<uintptr_t>(out.data_ptr()) - s->base) / 4);
      e.shard_elems = s->shard_elems;
      TORCH_CHECK(e.flat_off % 32 == 0, "gradient views must start at a multiple of 32 elements");
    }
  }
  e.bias = nullptr;
  e.bias_f32 = 0;
  if (bias.has_value()) {
    check_cuda(*bias, "bias");
    TORCH_CHECK(bias->numel() == N, "bias must have N elements");
    e.bias = bias->data_ptr();
    e.bias_f32 = bias->scalar_type() == at::kFloat;
    TORCH_CHECK(e.bias_f32 || bias->scalar_type() == at::kBFloat16, "bias must be bfloat16 or float32");
  }
  e.row_scale = opt_f32(row_scale, "row_scale");
  if (row_scale.has_value()) TORCH_CHECK(row_scale->numel() == M, "row_scale must have M elements");
  e.ssq_in = opt_f32(ssq_in, "ssq_in");
  e.ssq_parts = 0;
  if (ssq_in.has_value()) {
    TORCH_CHECK(ssq_in->dim() == 2 && ssq_in->size(0) == M && ssq_in->is_contiguous(), "ssq_in must be (M, parts)");
    e.ssq_parts = (int)ssq_in->size(1);
  }
  e.norm_dim = (int)norm_dim;
  e.norm_eps = (float)norm_eps;
  e.aux = opt_bf16(aux, "aux");
  e.aux_ld = 0;
  e.aux_mode = (int)aux_mode;
  if (aux.has_value()) {
    TORCH_CHECK(aux->dim() == 2 && aux->size(0) == M && aux->size(1) == N, "aux must be (M, N)");
    e.aux_ld = aux->stride(0);
    TORCH_CHECK((e.aux_ld * 2) % 16 == 0, "aux rows must be 16-byte aligned");
    TORCH_CHECK(aux_mode >= 1 && aux_mode <= 3, "aux_mode must be 1..3 when aux is given");
  }
  e.rowcoef = opt_f32(rowcoef, "rowcoef");
  if (aux_mode == gd::AUX_RMS_SILU_BWD) TORCH_CHECK(rowcoef.has_value() && rowcoef->numel() == M, "rowcoef (M) needed");
  e.pre_out = nullptr;
  e.pre_ld = 0;
  if (pre_out.has_value()) {
    TORCH_CHECK(pre_out->dim() == 2 && pre_out->size(0) == M && pre_out->size(1) == N, "pre_out must be (M, N)");
    e.pre_out = bf16_mut(*pre_out, "pre_out");
    e.pre_ld = pre_out->stride(0);
    TORCH_CHECK((e.pre_ld * 2) % 16 == 0, "pre_out rows must be 16-byte aligned");
  }
  e.act = (int)act;
  e.tma_mask = 0;   // chosen by the launcher
  e.ssq_out = nullptr;
  if (ssq_out.has_value()) {
    TORCH_CHECK(ssq_out->dim() == 2 && ssq_out->size(0) == M && ssq_out->is_contiguous(), "ssq_out must be (M, parts)");
    TORCH_CHECK(!ssq_in.has_value() || ssq_in->size(1) == ssq_out->size(1), "ssq_in/ssq_out parts differ");
    e.ssq_out = f32_mut(*ssq_out, "ssq_out");
    e.ssq_parts = (int)ssq_out->size(1);
  }
}

// D = A B^T. a: (M,K) [K-major] or (K,M) [a_mn]; b: (N,K) or (K,N) [b_mn].
void gemm_bf16(const Tensor& a, const Tensor& b, bool a_mn, bool b_mn, Tensor out, bool accumulate, OptT bias,
               OptT row_scale, OptT ssq_in, int64_t norm_dim, double norm_eps, OptT aux, int64_t aux_mode,
               OptT rowcoef, OptT pre_out, int64_t act, OptT ssq_out, int64_t sink, int64_t sink_off, int64_t sink_ld) {
  c10::cuda::CUDAGuard guard(a.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "gemm operands must be 2-D");
  const int64_t M = a_mn ? a.size(1) : a.size(0), K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm: reduction sizes differ: ", K, " vs ", Kb);
  gd::GemmOperands op{bf16_ptr(a, "a"), bf16_ptr(b, "b"), a.stride(0), b.stride(0)};
  gd::GemmShape g{(int)M, (int)N, (int)K, a_mn, b_mn, nullptr, nullptr, 0, 1, nullptr, nullptr};
  gd::GemmEpilogue e;
  if (sink >= 0) {
    // fp32 accumulation into a gradient that lives sharded over the ranks: `out` only gives the shape
    const GradSink& gs = sink_at(sink);
    TORCH_CHECK(gs.elems < 0, "explicit gradient offsets need a virtual sink");
    TORCH_CHECK(out.dim() == 2 && out.size(0) == M && out.size(1) == N, "out must be (M, N)");
    TORCH_CHECK(sink_ld >= N && sink_ld % 32 == 0 && N % 32 == 0 && sink_off % 32 == 0 && sink_off >= 0 &&
                sink_off + (M - 1) * sink_ld + N <= -gs.elems, "gradient range outside the sink");
    TORCH_CHECK(!bias.has_value() && !aux.has_value() && !pre_out.has_value() && !row_scale.has_value() &&
                !ssq_in.has_value() && !ssq_out.has_value() && act == 0, "a sharded gradient takes a plain epilogue");
    e = gd::GemmEpilogue{};
    e.out = gs.table.data_ptr();      // non-null, never dereferenced: every chunk goes through peer_out
    e.out_ld = sink_ld;
    e.out_f32 = 1;
    e.accumulate = 1;
    e.peer_out = reinterpret_cast<float* const*>(gs.table.data_ptr<int64_t>());
    e.flat_off = sink_off;
    e.shard_elems = gs.shard_elems;
  } else {
    fill_epilogue(e, out, accumulate, bias, row_scale, ssq_in, norm_dim, norm_eps, aux, aux_mode, rowcoef, pre_out, act,
                  ssq_out, M, N);
  }
  if (ssq_out.has_value()) TORCH_CHECK(ssq_out->size(1) == (N + 127) / 128, "bf16 gemm writes N/128 ssq partials");
  take_pending_gather(g, 0, false);
  GD_LAUNCH(gd::launch_gemm_bf16(op, g, e, status_ptr(a), stream_of(a)));
}

// a8: (M,K) e4m3 with sa (K/128, M); b8: (N,K) e4m3 with sb (N/128, K/128).
void gemm_fp8(const Tensor& a8, const Tensor& sa, const Tensor& b8, const Tensor& sb, Tensor out, bool accumulate,
              OptT bias, OptT row_scale, OptT aux, int64_t aux_mode, OptT pre_out, int64_t act) {
  c10::cuda::CUDAGuard guard(a8.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(a8.dim() == 2 && b8.dim() == 2, "gemm operands must be 2-D");
  const int64_t M = a8.size(0), K = a8.size(1), N = b8.size(0);
  TORCH_CHECK(b8.size(1) == K, "gemm_fp8: reduction sizes differ");
  const int64_t KB = (K + 127) / 128, NB = (N + 127) / 128;
  TORCH_CHECK(sa.dim() == 2 && sa.size(0) == KB && sa.size(1) >= M && sa.stride(1) == 1, "sa must be (K/128, M)");
  TORCH_CHECK(sb.dim() == 2 && sb.size(0) == NB && sb.size(1) == KB && sb.is_contiguous(), "sb must be (N/128, K/128)");
  gd::GemmOperands op{fp8_mut(a8, "a8"), fp8_mut(b8, "b8"), a8.stride(0), b8.stride(0)};
  gd::GemmShape g{(int)M, (int)N, (int)K, 0, 0, f32_ptr(sa, "sa"), f32_ptr(sb, "sb"), sa.stride(0), 1, nullptr, nullptr};
  gd::GemmEpilogue e;
  std::optional<Tensor> none;
  fill_epilogue(e, out, accumulate, bias, row_scale, none, 0, 0.0, aux, aux_mode, none, pre_out, act, none, M, N);
  GD_LAUNCH(gd::launch_gemm_fp8(op, g, e, status_ptr(a8), stream_of(a8)));
}

// a8: (M,K) e4m3 with packed UE8M0 chunks pa (M/128, K/128, 512); b8: (N,K) with pb (N/128, K/128, 512).
void gemm_fp8_mx(const Tensor& a8, const Tensor& pa, const Tensor& b8, const Tensor& pb, Tensor out, bool accumulate,
                 OptT bias, OptT row_scale, OptT aux, int64_t aux_mode, OptT pre_out, int64_t act, OptT q8, OptT q8_p,
                 bool q8_silu, bool store_out) {
  c10::cuda::CUDAGuard guard(a8.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(a8.dim() == 2 && b8.dim() == 2, "gemm operands must be 2-D");
  const int64_t M = a8.size(0), K = a8.size(1), N = b8.size(0);
  TORCH_CHECK(b8.size(1) == K, "gemm_fp8_mx: reduction sizes differ");
  TORCH_CHECK(M % 128 == 0 && N % 128 == 0 && K % 128 == 0, "gemm_fp8_mx: M, N, K must be multiples of 128");
  TORCH_CHECK(pa.is_contiguous() && pa.numel() == (M / 128) * (K / 128) * 512, "pa must hold M/128 * K/128 * 512 bytes");
  TORCH_CHECK(pb.is_contiguous() && pb.numel() == (N / 128) * (K / 128) * 512, "pb must hold N/128 * K/128 * 512 bytes");
  gd::GemmOperands op{fp8_mut(a8, "a8"), fp8_mut(b8, "b8"), a8.stride(0), b8.stride(0)};
  gd::GemmShape g{(int)M, (int)N, (int)K, 0, 0, nullptr, nullptr, 0, 1, fp8_mut(pa, "pa"), fp8_mut(pb, "pb")};
  gd::GemmEpilogue e;
  std::optional<Tensor> none;
  fill_epilogue(e, out, accumulate, bias, row_scale, none, 0, 0.0, aux, aux_mode, none, pre_out, act, none, M, N);
  if (q8.has_value()) {
    TORCH_CHECK(q8_p.has_value(), "q8 needs q8_p");
    TORCH_CHECK(q8->dim() == 2 && q8->size(0) == M && q8->size(1) == N && q8->stride(1) == 1 && q8->stride(0) % 16 == 0,
                "q8 must be (M, N) with 16-byte aligned rows");
    TORCH_CHECK(q8_p->dim() == 3 && q8_p->size(0) == M / 128 && q8_p->size(1) == N / 128 && q8_p->size(2) == 512 &&
                q8_p->stride(2) == 1 && q8_p->stride(1) == 512 && q8_p->stride(0) % 512 == 0,
                "q8_p must be (M/128, N/128, 512) bytes");
    TORCH_CHECK(!e.out_f32 && !accumulate, "a quantised copy needs a plain bf16 epilogue");
    e.q8 = fp8_mut(*q8, "q8");
    e.q8_ld = q8->stride(0);
    e.q8_p = fp8_mut(*q8_p, "q8_p");
    e.q8_p_stride = q8_p->stride(0) / 512;
    e.q8_silu = q8_silu;
  }
  if (!store_out) {
    TORCH_CHECK(q8.has_value() && !pre_out.has_value(), "store_out=False only makes sense with a quantised copy");
    e.out = nullptr;
  }
  take_pending_gather(g, N / 128, true);
  GD_LAUNCH(gd::launch_gemm_fp8_mx(op, g, e, status_ptr(a8), stream_of(a8)));
}

void dwconv_fwd(const Tensor& x, OptT halo, const Tensor& w, Tensor out, OptT q, OptT qs, OptT qp) {
  c10::cuda::CUDAGuard guard(x.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(x.dim() == 3 && out.dim() == 3, "dwconv: x and out must be (B, T, d)");
  const int B = (int)x.size(0), T = (int)x.size(1), d = (int)x.size(2), k = (int)w.size(0);
  TORCH_CHECK(w.dim() == 2 && w.size(1) == d && w.is_contiguous(), "dwconv: taps must be (k, d) contiguous (transposed)");
  TORCH_CHECK(B == 1 || (x.stride(0) == x.stride(1) * T && out.stride(0) == out.stride(1) * T), "dwconv: batch stride must be T rows");
  TORCH_CHECK(out.size(0) == B && out.size(1) == T && out.size(2) == d, "dwconv: out shape");
  if (halo.has_value()) TORCH_CHECK(halo->is_contiguous() && halo->size(0) == B && halo->size(1) == k - 1 && halo->size(2) == d, "dwconv: halo must be (B, k-1, d)");
  TORCH_CHECK((x.stride(1) * 2) % 16 == 0 && (out.stride(1) * 2) % 16 == 0, "dwconv: rows must be 16-byte aligned");
  gd::ConvArgs a{bf16_ptr(x, "x"), opt_bf16(halo, "halo"), f32_ptr(w, "w"), bf16_mut(out, "out"), B, T, d, k,
                 x.stride(1), out.stride(1), row_quant_out(q, qs, qp, (int64_t)B * T, d), {}};
  GD_LAUNCH(gd::launch_dwconv_fwd(a, stream_of(x)));
}

void dwconv_bwd(const Tensor& dc, const Tensor& x, OptT halo, const Tensor& w, OptT tail_add, Tensor dx, OptT dhalo,
                Tensor dw) {
  c10::cuda::CUDAGuard guard(x.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(x.dim() == 3 && dc.dim() == 3 && dx.dim() == 3, "dwconv_bwd: tensors must be (B, T, d)");
  const int B = (int)x.size(0), T = (int)x.size(1), d = (int)x.size(2), k = (int)w.size(0);
  TORCH_CHECK(w.dim() == 2 && w.size(1) == d && w.is_contiguous(), "dwconv_bwd: taps must be (k, d) contiguous (transposed)");
  TORCH_CHECK(dx.is_contiguous() && dw.is_contiguous() && dw.size(0) == d && dw.size(1) == k, "dwconv_bwd: dx/dw layout");
  TORCH_CHECK(B == 1 || (x.stride(0) == x.stride(1) * T && dc.stride(0) == dc.stride(1) * T), "dwconv_bwd: batch stride must be T rows");
  TORCH_CHECK((x.stride(1) * 2) % 16 == 0 && (dc.stride(1) * 2) % 16 == 0, "dwconv_bwd: rows must be 16-byte aligned");
  if (halo.has_value()) TORCH_CHECK(halo->is_contiguous() && halo->size(1) == k - 1, "dwconv_bwd: halo");
  if (tail_add.has_value()) TORCH_CHECK(tail_add->is_contiguous() && tail_add->size(1) == k - 1, "dwconv_bwd: tail_add");
  if (dhalo.has_value()) TORCH_CHECK(dhalo->is_contiguous() && dhalo->size(1) == k - 1, "dwconv_bwd: dhalo");
  gd::ConvBwdArgs a{bf16_ptr(dc, "dc"), bf16_ptr(x, "x"), opt_bf16(halo, "halo"), f32_ptr(w, "w"),
                    opt_bf16(tail_add, "tail_add"), bf16_mut(dx, "dx"),
                    dhalo.has_value() ? bf16_mut(*dhalo, "dhalo") : nullptr, f32_mut(dw, "dw"), B, T, d, k,
                    dc.stride(1), x.stride(1)};
  GD_LAUNCH(gd::launch_dwconv_bwd(a, stream_of(x)));
}

gd::ConvSp conv_sp(const Tensor& slot_ptrs, const Tensor& flag_ptrs, Tensor& counter, int64_t slot_offset, int64_t flag_index,
                   int64_t rank, int64_t world, int64_t seq, int64_t budget_ns, const Tensor& like) {
  TORCH_CHECK(slot_ptrs.is_cuda() && slot_ptrs.scalar_type() == at::kLong && slot_ptrs.numel() == world &&
              flag_ptrs.is_cuda() && flag_ptrs.scalar_type() == at::kLong && flag_ptrs.numel() == world,
              "halo exchange: one slot pointer and one flag pointer per rank");
  TORCH_CHECK(counter.is_cuda() && counter.scalar_type() == at::kInt && counter.numel() >= 1, "halo exchange: counter must be int32");
  TORCH_CHECK(rank >= 0 && rank < world && slot_offset % 16 == 0 && flag_index >= 0, "halo exchange: rank / offsets");
  gd::ConvSp sp{};
  sp.slots = reinterpret_cast<uint8_t* const*>(slot_ptrs.data_ptr<int64_t>());
  sp.flags = reinterpret_cast<uint32_t* const*>(flag_ptrs.data_ptr<int64_t>());
  sp.slot_offset = slot_offset;
  sp.flag_index = (int)flag_index;
  sp.rank = (int)rank;
  sp.world = (int)world;
  sp.seq = (uint32_t)seq;
  sp.counter = reinterpret_cast<uint32_t*>(counter.data_ptr<int>());
  sp.budget_ns = budget_ns > 0 ? (uint64_t)budget_ns : 0;
  sp.halo_out = nullptr;
  sp.status = status_ptr(like);
  return sp;
}

// Causal conv of a sequence shard with the neighbour exchange inside the kernel: the last k-1 input rows go to the
// next rank's slot, the previous rank's rows are waited for (bounded) and read from this rank's slot; they are
// also written to halo_out for the backward pass.
void dwconv_fwd_sp(const Tensor& x, const Tensor& w, Tensor out, Tensor halo_out, const Tensor& slot_ptrs,
                   const Tensor& flag_ptrs, Tensor counter, int64_t slot_offset, int64_t flag_index, int64_t rank,
                   int64_t world, int64_t seq, int64_t budget_ns, OptT q, OptT qs, OptT qp) {
  c10::cuda::CUDAGuard guard(x.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(x.dim() == 3 && out.dim() == 3, "dwconv: x and out must be (B, T, d)");
  const int B = (int)x.size(0), T = (int)x.size(1), d = (int)x.size(2), k = (int)w.size(0);
  TORCH_CHECK(w.dim() == 2 && w.size(1) == d && w.is_contiguous(), "dwconv: taps must be (k, d) contiguous (transposed)");
  TORCH_CHECK(B == 1 || (x.stride(0) == x.stride(1) * T && out.stride(0) == out.stride(1) * T), "dwconv: batch stride must be T rows");
  TORCH_CHECK(out.size(0) == B && out.size(1) == T && out.size(2) == d, "dwconv: out shape");
  TORCH_CHECK((x.stride(1) * 2) % 16 == 0 && (out.stride(1) * 2) % 16 == 0, "dwconv: rows must be 16-byte aligned");
  TORCH_CHECK(k == 4 && T % 8 == 0 && d % 8 == 0, "dwconv_fwd_sp: needs k == 4, T % 8 == 0, d % 8 == 0");
  TORCH_CHECK(halo_out.is_contiguous() && halo_out.dim() == 3 && halo_out.size(0) == B && halo_out.size(1) == k - 1 &&
              halo_out.size(2) == d, "dwconv_fwd_sp: halo_out must be (B, k-1, d)");
  gd::ConvArgs a{bf16_ptr(x, "x"), nullptr, f32_ptr(w, "w"), bf16_mut(out, "out"), B, T, d, k,
                 x.stride(1), out.stride(1), row_quant_out(q, qs, qp, (int64_t)B * T, d), {}};
  a.sp = conv_sp(slot_ptrs, flag_ptrs, counter, slot_offset, flag_index, rank, world, seq, budget_ns, x);
  a.sp.halo_out = bf16_mut(halo_out, "halo_out");
  GD_LAUNCH(gd::launch_dwconv_fwd(a, stream_of(x)));
}

// Backward of dwconv_fwd_sp: the gradient of the received rows goes to the previous rank's slot, the next rank's
// is waited for (bounded) and added to the last k-1 rows of dx inside the kernel; dw as in dwconv_bwd.
void dwconv_bwd_sp(const Tensor& dc, const Tensor& x, const Tensor& halo, const Tensor& w, Tensor dx, Tensor dw,
                   const Tensor& slot_ptrs, const Tensor& flag_ptrs, Tensor counter, int64_t slot_offset,
                   int64_t flag_index, int64_t rank, int64_t world, int64_t seq, int64_t budget_ns) {
  c10::cuda::CUDAGuard guard(x.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(x.dim() == 3 && dc.dim() == 3 && dx.dim() == 3, "dwconv_bwd: tensors must be (B, T, d)");
  const int B = (int)x.size(0), T = (int)x.size(1), d = (int)x.size(2), k = (int)w.size(0);
  TORCH_CHECK(w.dim() == 2 && w.size(1) == d && w.is_contiguous(), "dwconv_bwd: taps must be (k, d) contiguous (transposed)");
  TORCH_CHECK(dx.is_contiguous() && dw.is_contiguous() && dw.size(0) == d && dw.size(1) == k, "dwconv_bwd: dx/dw layout");
  TORCH_CHECK(B == 1 || (x.stride(0) == x.stride(1) * T && dc.stride(0) == dc.stride(1) * T), "dwconv_bwd: batch stride must be T rows");
  TORCH_CHECK((x.stride(1) * 2) % 16 == 0 && (dc.stride(1) * 2) % 16 == 0, "dwconv_bwd: rows must be 16-byte aligned");
  TORCH_CHECK(k == 4 && T % 8 == 0 && d % 8 == 0, "dwconv_bwd_sp: needs k == 4, T % 8 == 0, d % 8 == 0");
  TORCH_CHECK(halo.is_contiguous() && halo.dim() == 3 && halo.size(0) == B && halo.size(1) == k - 1 && halo.size(2) == d,
              "dwconv_bwd_sp: halo must be (B, k-1, d)");
  gd::ConvBwdArgs a{bf16_ptr(dc, "dc"), bf16_ptr(x, "x"), bf16_ptr(halo, "halo"), f32_ptr(w, "w"), nullptr,
                    bf16_mut(dx, "dx"), nullptr, f32_mut(dw, "dw"), B, T, d, k, dc.stride(1), x.stride(1), {}};
  a.sp = conv_sp(slot_ptrs, flag_ptrs, counter, slot_offset, flag_index, rank, world, seq, budget_ns, x);
  GD_LAUNCH(gd::launch_dwconv_bwd(a, stream_of(x)));
}

void gate_update_fwd(const Tensor& g_pre, const Tensor& z, const Tensor& c, const Tensor& s, const Tensor& w_r,
                     Tensor fwd_out, Tensor side_out, OptT gate_out, OptT rstd_out, OptT gate_sum, double eps_r, OptT q,
                     OptT qs, OptT qp) {
  c10::cuda::CUDAGuard guard(c.device());
  OpRange gd_range_(__func__);
  const int64_t rows = g_pre.size(0);
  const int d = (int)g_pre.size(1);
  TORCH_CHECK(g_pre.is_contiguous() && z.is_contiguous() && fwd_out.is_contiguous() && side_out.is_contiguous(),
              "gate_update: g_pre, z and outputs must be contiguous (rows, d)");
  TORCH_CHECK(c.size(0) == rows && s.size(0) == rows && c.size(1) == d && s.size(1) == d && w_r.numel() == d, "gate_update: shapes");
  gd::GateFwdArgs a{bf16_ptr(g_pre, "g_pre"), bf16_ptr(z, "z"), bf16_ptr(c, "c"), bf16_ptr(s, "s"), f32_ptr(w_r, "w_r"),
                    bf16_mut(fwd_out, "fwd_out"), bf16_mut(side_out, "side_out"),
                    gate_out.has_value() ? bf16_mut(*gate_out, "gate_out") : nullptr,
                    rstd_out.has_value() ? f32_mut(*rstd_out, "rstd_out") : nullptr,
                    gate_sum.has_value() ? f32_mut(*gate_sum, "gate_sum") : nullptr,
                    rows, d, c.stride(0), s.stride(0), (float)eps_r, row_quant_out(q, qs, qp, rows, d)};
  GD_LAUNCH(gd::launch_gate_update_fwd(a, stream_of(c)));
}

void gate_only_fwd(const Tensor& g_pre, const Tensor& c, Tensor fwd_out, Tensor side_out, OptT gate_sum, OptT q, OptT qs,
                   OptT qp) {
  c10::cuda::CUDAGuard guard(c.device());
  OpRange gd_range_(__func__);
  const int64_t rows = g_pre.size(0);
  const int d = (int)g_pre.size(1);
  TORCH_CHECK(g_pre.dim() == 2 && c.dim() == 2 && g_pre.is_contiguous() && fwd_out.is_contiguous() && side_out.is_contiguous(),
              "gate_only_fwd: g_pre and outputs must be contiguous (rows, d)");
  TORCH_CHECK(c.size(0) == rows && c.size(1) == d && c.stride(1) == 1 && fwd_out.numel() == rows * d && side_out.numel() == rows * d,
              "gate_only_fwd: shapes");
  gd::GateOnlyFwdArgs a{bf16_ptr(g_pre, "g_pre"), bf16_ptr(c, "c"), bf16_mut(fwd_out, "fwd_out"), bf16_mut(side_out, "side_out"),
                        gate_sum.has_value() ? f32_mut(*gate_sum, "gate_sum") : nullptr, rows, d, c.stride(0),
                        row_quant_out(q, qs, qp, rows, d)};
  GD_LAUNCH(gd::launch_gate_only_fwd(a, stream_of(c)));
}

void gate_only_bwd(const Tensor& dF, const Tensor& dS, const Tensor& g_pre, const Tensor& c, const Tensor& b2g,
                   const Tensor& ssq_g, double eps_g, OptT dgate_mean, Tensor dq, Tensor dc, Tensor rowcoef, Tensor db2g) {
  c10::cuda::CUDAGuard guard(c.device());
  OpRange gd_range_(__func__);
  const int64_t rows = g_pre.size(0);
  const int d = (int)g_pre.size(1);
  TORCH_CHECK(g_pre.dim() == 2 && g_pre.is_contiguous() && dq.is_contiguous() && dc.is_contiguous(), "gate_only_bwd: contiguity");
  for (const Tensor* t : std::initializer_list<const Tensor*>{&dF, &dS, &c})
    TORCH_CHECK(t->dim() == 2 && t->size(0) == rows && t->size(1) == d && t->stride(1) == 1, "gate_only_bwd: shapes");
  TORCH_CHECK(dq.numel() == rows * d && dc.numel() == rows * d, "gate_only_bwd: output shapes");
  TORCH_CHECK(ssq_g.dim() == 2 && ssq_g.size(0) == rows && ssq_g.is_contiguous(), "gate_only_bwd: ssq_g");
  TORCH_CHECK(db2g.numel() == d && b2g.numel() == d && rowcoef.numel() == rows, "gate_only_bwd: sizes");
  gd::GateOnlyBwdArgs a{bf16_ptr(dF, "dF"), bf16_ptr(dS, "dS"), bf16_ptr(g_pre, "g_pre"), bf16_ptr(c, "c"), f32_ptr(b2g, "b2g"),
                        f32_ptr(ssq_g, "ssq_g"), (int)ssq_g.size(1), (float)eps_g, opt_f32(dgate_mean, "dgate_mean"),
                        bf16_mut(dq, "dq"), bf16_mut(dc, "dc"), f32_mut(rowcoef, "rowcoef"), f32_mut(db2g, "db2g"), rows, d,
                        dF.stride(0), dS.stride(0), c.stride(0)};
  GD_LAUNCH(gd::launch_gate_only_bwd(a, stream_of(c)));
}

void gate_update_bwd(const Tensor& dF, const Tensor& dS, const Tensor& g_pre, const Tensor& z, const Tensor& c,
                     const Tensor& s, const Tensor& w_r, const Tensor& b2g, const Tensor& rstd_z, const Tensor& ssq_g,
                     double eps_g, OptT dgate_mean, Tensor dq, Tensor dz, Tensor dsc, Tensor rowcoef, Tensor db2g,
                     Tensor dw_r, Tensor db2r, OptT q, OptT qs, OptT qp) {
  c10::cuda::CUDAGuard guard(c.device());
  OpRange gd_range_(__func__);
  const int64_t rows = g_pre.size(0);
  const int d = (int)g_pre.size(1);
  TORCH_CHECK(g_pre.is_contiguous() && z.is_contiguous() && dq.is_contiguous() && dz.is_contiguous() && dsc.is_contiguous(),
              "gate_update_bwd: contiguity");
  TORCH_CHECK(dsc.size(0) == rows && dsc.size(1) == 2 * d, "gate_update_bwd: dsc must be (rows, 2d)");
  TORCH_CHECK(ssq_g.dim() == 2 && ssq_g.size(0) == rows && ssq_g.is_contiguous(), "gate_update_bwd: ssq_g");
  TORCH_CHECK(db2g.numel() == d && dw_r.numel() == d && db2r.numel() == d && rowcoef.numel() == rows, "gate_update_bwd: sizes");
  gd::GateBwdArgs a{bf16_ptr(dF, "dF"), bf16_ptr(dS, "dS"), bf16_ptr(g_pre, "g_pre"), bf16_ptr(z, "z"), bf16_ptr(c, "c"),
                    bf16_ptr(s, "s"), f32_ptr(w_r, "w_r"), f32_ptr(b2g, "b2g"), 1, f32_ptr(rstd_z, "rstd_z"),
                    f32_ptr(ssq_g, "ssq_g"), (int)ssq_g.size(1), (float)eps_g, opt_f32(dgate_mean, "dgate_mean"),
                    bf16_mut(dq, "dq"), bf16_mut(dz, "dz"), bf16_mut(dsc, "dsc"), f32_mut(rowcoef, "rowcoef"),
                    nullptr, nullptr, f32_mut(db2g, "db2g"), f32_mut(dw_r, "dw_r"), f32_mut(db2r, "db2r"), rows, d,
                    dF.stride(0), dS.stride(0), c.stride(0), s.stride(0), row_quant_out(q, qs, qp, rows, d)};
  GD_LAUNCH(gd::launch_gate_update_bwd(a, stream_of(c)));
}

void rmsnorm_fwd(const Tensor& x, const Tensor& w, Tensor y, OptT rstd, double eps) {
  c10::cuda::CUDAGuard guard(x.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && x.dim() == 2, "rmsnorm: (rows, d) contiguous");
  GD_LAUNCH(gd::launch_rmsnorm_fwd(bf16_ptr(x, "x"), f32_ptr(w, "w"), bf16_mut(y, "y"),
                                   rstd.has_value() ? f32_mut(*rstd, "rstd") : nullptr, x.size(0), (int)x.size(1),
                                   (float)eps, stream_of(x)));
}

void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, Tensor dx, Tensor dw) {
  c10::cuda::CUDAGuard guard(x.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous() && dx.is_contiguous() && x.dim() == 2, "rmsnorm_bwd: contiguity");
  GD_LAUNCH(gd::launch_rmsnorm_bwd(bf16_ptr(dy, "dy"), bf16_ptr(x, "x"), f32_ptr(w, "w"), f32_ptr(rstd, "rstd"),
                                   bf16_mut(dx, "dx"), f32_mut(dw, "dw"), x.size(0), (int)x.size(1), stream_of(x)));
}

void quant_tile(const Tensor& x, bool pre_silu, OptT q_row, OptT s_row, int64_t row_mode, OptT q_col, OptT s_col,
                int64_t col_mode, bool pow2, OptT p_row, OptT p_col, OptT peer_delta) {
  c10::cuda::CUDAGuard guard(x.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(x.dim() == 2, "quantise: x must be 2-D");
  gd::QuantArgs a{};
  a.x = bf16_ptr(x, "x");
  a.rows = x.size(0);
  a.cols = (int)x.size(1);
  a.x_ld = x.stride(0);
  TORCH_CHECK((a.x_ld * 2) % 16 == 0, "quantise: rows must be 16-byte aligned");
  a.pre_silu = pre_silu;
  a.row_mode = (int)row_mode;
  a.col_mode = (int)col_mode;
  const int64_t rb = (a.rows + 127) / 128, cb = (a.cols + 127) / 128;
  if (q_row.has_value()) {
    TORCH_CHECK(s_row.has_value(), "quantise: s_row needed with q_row");
    TORCH_CHECK(q_row->dim() == 2 && q_row->size(0) == a.rows && q_row->size(1) == a.cols, "quantise: q_row shape");
    a.q_row = fp8_mut(*q_row, "q_row");
    a.q_row_ld = q_row->stride(0);
    TORCH_CHECK(a.q_row_ld % 8 == 0, "quantise: q_row pitch must be a multiple of 8");
    a.s_row = f32_mut(*s_row, "s_row");
    if (row_mode == gd::QUANT_ROWS) {
      TORCH_CHECK(s_row->dim() == 2 && s_row->size(0) == cb && s_row->size(1) >= a.rows && s_row->stride(1) == 1, "quantise: s_row must be (cols/128, rows)");
      a.s_row_ld = s_row->stride(0);
    } else {
      TORCH_CHECK(row_mode == gd::QUANT_BLOCK && s_row->is_contiguous() && s_row->numel() == rb * cb, "quantise: s_row must be (rows/128, cols/128)");
    }
  }
  if (q_col.has_value()) {
    TORCH_CHECK(s_col.has_value(), "quantise: s_col needed with q_col");
    TORCH_CHECK(q_col->dim() == 2 && q_col->size(0) == a.cols && q_col->size(1) == a.rows, "quantise: q_col shape");
    a.q_col = fp8_mut(*q_col, "q_col");
    a.q_col_ld = q_col->stride(0);
    TORCH_CHECK(a.q_col_ld % 16 == 0, "quantise: q_col pitch must be a multiple of 16");
    a.s_col = f32_mut(*s_col, "s_col");
    if (col_mode == gd::QUANT_COLS) {
      TORCH_CHECK(s_col->dim() == 2 && s_col->size(0) == rb && s_col->size(1) >= a.cols && s_col->stride(1) == 1, "quantise: s_col must be (rows/128, cols)");
      a.s_col_ld = s_col->stride(0);
    } else {
      TORCH_CHECK(col_mode == gd::QUANT_BLOCK && s_col->is_contiguous() && s_col->numel() == rb * cb, "quantise: s_col must be (cols/128, rows/128)");
    }
  }
  a.pow2 = pow2;
  if (p_row.has_value() || p_col.has_value()) {
    TORCH_CHECK(pow2 && a.rows % 128 == 0 && a.cols % 128 == 0, "packed scales need pow2 scales and 128-multiples");
    if (p_row.has_value()) {
      TORCH_CHECK(q_row.has_value() && p_row->dim() == 3 && p_row->size(0) == rb && p_row->size(1) == cb && p_row->size(2) == 512 &&
                  p_row->stride(2) == 1 && p_row->stride(1) == 512 && p_row->stride(0) % 512 == 0,
                  "p_row must be (rows/128, cols/128, 512) bytes, dense in its last two dims");
      a.p_row = fp8_mut(*p_row, "p_row");
      a.p_row_stride = p_row->stride(0) / 512;
    }
    if (p_col.has_value()) {
      TORCH_CHECK(q_col.has_value() && p_col->is_contiguous() && p_col->numel() == rb * cb * 512, "p_col must hold cols/128 * rows/128 * 512 bytes");
      a.p_col = fp8_mut(*p_col, "p_col");
    }
  }
  if (peer_delta.has_value() && peer_delta->numel() > 0) {
    TORCH_CHECK(peer_delta->is_cuda() && peer_delta->scalar_type() == at::kLong && peer_delta->is_contiguous(),
                "peer_delta must be an int64 CUDA tensor");
    a.peer_delta = peer_delta->data_ptr<int64_t>();
    a.n_peer = (int)peer_delta->numel();
  }
  GD_LAUNCH(gd::launch_quant_tile(a, stream_of(x)));
}

void quant_tensor(const Tensor& x, const Tensor& scale, Tensor q_row, OptT q_col, OptT amax) {
  c10::cuda::CUDAGuard guard(x.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && q_row.is_contiguous(), "quant_tensor: contiguous 2-D");
  if (q_col.has_value()) TORCH_CHECK(q_col->is_contiguous(), "quant_tensor: q_col contiguous");
  GD_LAUNCH(gd::launch_quant_tensor(bf16_ptr(x, "x"), f32_ptr(scale, "scale"), fp8_mut(q_row, "q_row"),
                                    q_col.has_value() ? fp8_mut(*q_col, "q_col") : nullptr,
                                    amax.has_value() ? f32_mut(*amax, "amax") : nullptr, x.size(0), (int)x.size(1),
                                    stream_of(x)));
}

gd::GateMixArgs gate_mix_common(const Tensor& g_pre, const Tensor& c, const Tensor& s, const Tensor& R) {
  TORCH_CHECK(g_pre.dim() == 2 && g_pre.is_contiguous(), "gate_mix: g_pre must be contiguous (rows, d)");
  const int64_t rows = g_pre.size(0), d = g_pre.size(1);
  for (const Tensor* t : std::initializer_list<const Tensor*>{&c, &s, &R}) {
    TORCH_CHECK(t->dim() == 2 && t->size(0) == rows && t->size(1) == d && t->stride(1) == 1 && (t->stride(0) * 2) % 16 == 0,
                "gate_mix: c, s and R must be (rows, d) with unit column stride and 16-byte aligned rows");
  }
  gd::GateMixArgs a{};
  a.g_pre = bf16_ptr(g_pre, "g_pre");
  a.c = bf16_ptr(c, "c");
  a.s = bf16_ptr(s, "s");
  a.R = bf16_ptr(R, "R");
  a.rows = rows;
  a.d = (int)d;
  a.c_ld = c.stride(0);
  a.s_ld = s.stride(0);
  a.r_ld = R.stride(0);
  return a;
}

void gate_mix_fwd(const Tensor& g_pre, const Tensor& c, const Tensor& s, const Tensor& R, Tensor fwd_out, Tensor side_out) {
  c10::cuda::CUDAGuard guard(c.device());
  OpRange gd_range_(__func__);
  gd::GateMixArgs a = gate_mix_common(g_pre, c, s, R);
  TORCH_CHECK(fwd_out.is_contiguous() && side_out.is_contiguous() && fwd_out.numel() == g_pre.numel() &&
              side_out.numel() == g_pre.numel(), "gate_mix: outputs must be contiguous (rows, d)");
  a.fwd_out = bf16_mut(fwd_out, "fwd_out");
  a.side_out = bf16_mut(side_out, "side_out");
  GD_LAUNCH(gd::launch_gate_mix_fwd(a, stream_of(c)));
}

void gate_mix_bwd(const Tensor& dF, const Tensor& dS, const Tensor& g_pre, const Tensor& c, const Tensor& s, const Tensor& R,
                  OptT ssq, OptT b2, double eps, Tensor dgp, OptT dq, Tensor dc, Tensor ds, Tensor dR, OptT rowcoef) {
  c10::cuda::CUDAGuard guard(c.device());
  OpRange gd_range_(__func__);
  gd::GateMixArgs a = gate_mix_common(g_pre, c, s, R);
  for (const Tensor* t : std::initializer_list<const Tensor*>{&dF, &dS, &dgp, &dc, &ds, &dR})
    TORCH_CHECK(t->is_contiguous() && t->numel() == g_pre.numel(), "gate_mix_bwd: gradients must be contiguous (rows, d)");
  a.dF = bf16_ptr(dF, "dF");
  a.dS = bf16_ptr(dS, "dS");
  if (ssq.has_value()) {
    TORCH_CHECK(ssq->dim() == 2 && ssq->size(0) == a.rows && ssq->is_contiguous(), "gate_mix_bwd: ssq must be (rows, parts)");
    a.ssq = f32_ptr(*ssq, "ssq");
    a.ssq_parts = (int)ssq->size(1);
  }
  if (b2.has_value()) {
    TORCH_CHECK(b2->numel() == a.d, "gate_mix_bwd: b2 must have d elements");
    a.b2 = f32_ptr(*b2, "b2");
  }
  a.eps = (float)eps;
  a.dgp = bf16_mut(dgp, "dgp");
  if (dq.has_value()) {
    TORCH_CHECK(dq->is_contiguous() && dq->numel() == g_pre.numel(), "gate_mix_bwd: dq must be contiguous (rows, d)");
    a.dq = bf16_mut(*dq, "dq");
  }
  a.dc = bf16_mut(dc, "dc");
  a.ds = bf16_mut(ds, "ds");
  a.dR = bf16_mut(dR, "dR");
  if (rowcoef.has_value()) {
    TORCH_CHECK(rowcoef->numel() == a.rows, "gate_mix_bwd: rowcoef must have one value per row");
    a.rowcoef = f32_mut(*rowcoef, "rowcoef");
  }
  GD_LAUNCH(gd::launch_gate_mix_bwd(a, stream_of(c)));
}

gd::CamBlendArgs cam_blend_common(const Tensor& z, const Tensor& fwd, const Tensor& retr, const Tensor& w, int64_t T, double eps) {
  TORCH_CHECK(z.dim() == 2 && z.is_contiguous() && fwd.is_contiguous() && fwd.numel() == z.numel(), "cam_blend: z and fwd must be contiguous (rows, d)");
  const int64_t rows = z.size(0), d = z.size(1);
  TORCH_CHECK(T >= 1 && rows % T == 0 && retr.is_contiguous() && retr.numel() == (rows / T) * d, "cam_blend: retrieved must be (rows / T, d)");
  TORCH_CHECK(w.numel() == d, "cam_blend: one norm weight per column");
  gd::CamBlendArgs a{};
  a.z = bf16_ptr(z, "z");
  a.fwd = bf16_ptr(fwd, "fwd");
  a.retr = bf16_ptr(retr, "retrieved");
  a.w = f32_ptr(w, "w");
  a.rows = rows;
  a.T = (int)T;
  a.d = (int)d;
  a.eps = (float)eps;
  return a;
}

void cam_blend_fwd(const Tensor& z, const Tensor& fwd, const Tensor& retr, const Tensor& w, int64_t T, double eps,
                   Tensor out, Tensor rstd) {
  c10::cuda::CUDAGuard guard(z.device());
  OpRange gd_range_(__func__);
  gd::CamBlendArgs a = cam_blend_common(z, fwd, retr, w, T, eps);
  TORCH_CHECK(out.is_contiguous() && out.numel() == z.numel() && rstd.numel() == z.size(0), "cam_blend: outputs");
  a.out = bf16_mut(out, "out");
  a.rstd = f32_mut(rstd, "rstd");
  GD_LAUNCH(gd::launch_cam_blend_fwd(a, stream_of(z)));
}

void cam_blend_bwd(const Tensor& dout, const Tensor& z, const Tensor& fwd, const Tensor& retr, const Tensor& w,
                   const Tensor& rstd, int64_t T, double eps, Tensor dz, Tensor dfwd, Tensor dretr, Tensor dw) {
  c10::cuda::CUDAGuard guard(z.device());
  OpRange gd_range_(__func__);
  gd::CamBlendArgs a = cam_blend_common(z, fwd, retr, w, T, eps);
  TORCH_CHECK(dout.is_contiguous() && dz.is_contiguous() && dfwd.is_contiguous() && dout.numel() == z.numel() &&
              dz.numel() == z.numel() && dfwd.numel() == z.numel(), "cam_blend_bwd: gradients must be contiguous (rows, d)");
  TORCH_CHECK(dretr.is_contiguous() && dretr.numel() == retr.numel() && dw.numel() == z.size(1) && rstd.numel() == z.size(0),
              "cam_blend_bwd: dretr (B, d), dw (d), rstd (rows)");
  a.rstd = const_cast<float*>(f32_ptr(rstd, "rstd"));
  a.dout = bf16_ptr(dout, "dout");
  a.dz = bf16_mut(dz, "dz");
  a.dfwd = bf16_mut(dfwd, "dfwd");
  a.dretr = f32_mut(dretr, "dretr");
  a.dw = f32_mut(dw, "dw");
  GD_LAUNCH(gd::launch_cam_blend_bwd(a, stream_of(z)));
}

void colsum(const Tensor& x, Tensor out) {
  c10::cuda::CUDAGuard guard(x.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(x.dim() == 2 && out.numel() == x.size(1), "colsum: shapes");
  TORCH_CHECK((x.stride(0) * 2) % 16 == 0, "colsum: rows must be 16-byte aligned");
  GD_LAUNCH(gd::launch_colsum(bf16_ptr(x, "x"), f32_mut(out, "out"), x.size(0), (int)x.size(1), x.stride(0), stream_of(x)));
}

void segment_add(const Tensor& src, const Tensor& dst_addr, const Tensor& seg_off) {
  c10::cuda::CUDAGuard guard(src.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(src.is_contiguous() && dst_addr.is_cuda() && dst_addr.scalar_type() == at::kLong && dst_addr.is_contiguous(),
              "segment_add: src contiguous, dst_addr int64 on the device");
  TORCH_CHECK(seg_off.is_cuda() && seg_off.scalar_type() == at::kInt && seg_off.numel() == dst_addr.numel(),
              "segment_add: one int32 offset per segment");
  GD_LAUNCH(gd::launch_segment_add(f32_ptr(src, "src"), dst_addr.data_ptr<int64_t>(), seg_off.data_ptr<int>(),
                                   (int)dst_addr.numel(), (int)src.numel(), stream_of(src)));
}

void scale_cols(const Tensor& w, const Tensor& colw, Tensor out) {
  c10::cuda::CUDAGuard guard(w.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(w.is_contiguous() && out.is_contiguous() && w.dim() == 2 && colw.numel() == w.size(1), "scale_cols: shapes");
  GD_LAUNCH(gd::launch_scale_cols(bf16_ptr(w, "w"), f32_ptr(colw, "colw"), bf16_mut(out, "out"), w.size(0), (int)w.size(1), stream_of(w)));
}

void unscale_cols_bwd(const Tensor& dW2w, const Tensor& W2, const Tensor& colw, Tensor dW2, Tensor dcolw) {
  c10::cuda::CUDAGuard guard(W2.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(dW2w.is_contiguous() && W2.is_contiguous() && dW2.is_contiguous(), "unscale_cols_bwd: contiguity");
  GD_LAUNCH(gd::launch_unscale_cols_bwd(f32_ptr(dW2w, "dW2w"), bf16_ptr(W2, "W2"), f32_ptr(colw, "colw"),
                                        f32_mut(dW2, "dW2"), f32_mut(dcolw, "dcolw"), (int)W2.size(0), (int)W2.size(1),
                                        stream_of(W2)));
}

void cross_entropy(Tensor logits, const Tensor& targets, Tensor row_loss, const Tensor& inv_count, int64_t vocab,
                   int64_t ignore_index, double grad_scale, bool write_grad) {
  c10::cuda::CUDAGuard guard(logits.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(logits.dim() == 2 && targets.scalar_type() == at::kLong && targets.is_contiguous(), "cross_entropy: inputs");
  TORCH_CHECK(targets.numel() == logits.size(0) && row_loss.numel() == logits.size(0) && vocab <= logits.size(1), "cross_entropy: sizes");
  GD_LAUNCH(gd::launch_cross_entropy(bf16_mut(logits, "logits"), targets.data_ptr<int64_t>(), f32_mut(row_loss, "row_loss"),
                                     f32_ptr(inv_count, "inv_count"), logits.size(0), (int)vocab, logits.stride(0),
                                     (int)ignore_index, (float)grad_scale, write_grad, status_ptr(logits),
                                     stream_of(logits)));
}

void mem_read_fwd(const Tensor& q, const Tensor& gamma, const Tensor& e, const Tensor& tags, const Tensor& vals,
                  const Tensor& alpha, Tensor w, Tensor out) {
  c10::cuda::CUDAGuard guard(q.device());
  OpRange gd_range_(__func__);
  for (const Tensor* t : std::initializer_list<const Tensor*>{&q, &gamma, &e, &tags, &vals, &w, &out}) TORCH_CHECK(t->is_contiguous(), "mem_read: contiguous inputs");
  const int B = (int)tags.size(0), S = (int)tags.size(1), dsig = (int)tags.size(2), dc = (int)vals.size(2);
  GD_LAUNCH(gd::launch_mem_read_fwd(f32_ptr(q, "q"), f32_ptr(gamma, "gamma"), f32_ptr(e, "e"), f32_ptr(tags, "tags"),
                                    f32_ptr(vals, "vals"), f32_ptr(alpha, "alpha"), f32_mut(w, "w"), f32_mut(out, "out"),
                                    B, S, dsig, dc, stream_of(q)));
}

void mem_read_bwd(const Tensor& d_out, const Tensor& q, const Tensor& gamma, const Tensor& e, const Tensor& tags,
                  const Tensor& vals, const Tensor& w, const Tensor& alpha, Tensor d_q, Tensor d_gamma, Tensor d_e,
                  Tensor d_tags, Tensor d_vals, Tensor d_alpha) {
  c10::cuda::CUDAGuard guard(q.device());
  OpRange gd_range_(__func__);
  for (const Tensor* t : std::initializer_list<const Tensor*>{&d_out, &q, &gamma, &e, &tags, &vals, &w, &d_q, &d_gamma, &d_e, &d_tags, &d_vals})
    TORCH_CHECK(t->is_contiguous(), "mem_read_bwd: contiguous tensors");
  const int B = (int)tags.size(0), S = (int)tags.size(1), dsig = (int)tags.size(2), dc = (int)vals.size(2);
  GD_LAUNCH(gd::launch_mem_read_bwd(f32_ptr(d_out, "d_out"), f32_ptr(q, "q"), f32_ptr(gamma, "gamma"), f32_ptr(e, "e"),
                                    f32_ptr(tags, "tags"), f32_ptr(vals, "vals"), f32_ptr(w, "w"), f32_ptr(alpha, "alpha"),
                                    f32_mut(d_q, "d_q"), f32_mut(d_gamma, "d_gamma"), f32_mut(d_e, "d_e"),
                                    f32_mut(d_tags, "d_tags"), f32_mut(d_vals, "d_vals"), f32_mut(d_alpha, "d_alpha"),
                                    B, S, dsig, dc, stream_of(q)));
}

void grad_dots(const Tensor& gt, OptT gi, Tensor sums) {
  c10::cuda::CUDAGuard guard(gt.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(gt.is_contiguous() && sums.numel() >= 3, "grad_dots: inputs");
  if (gi.has_value()) TORCH_CHECK(gi->is_contiguous() && gi->numel() == gt.numel(), "grad_dots: gi size");
  GD_LAUNCH(gd::launch_grad_dots(f32_ptr(gt, "gt"), opt_f32(gi, "gi"), f32_mut(sums, "sums"), gt.numel(), stream_of(gt)));
}

void projected_adamw(Tensor p, const Tensor& gt, OptT gi, Tensor m, Tensor v, const Tensor& scalars, double beta_proj,
                     double lr, double beta1, double beta2, double eps, double weight_decay, int64_t step) {
  c10::cuda::CUDAGuard guard(p.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(p.is_contiguous() && gt.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "adamw: contiguity");
  TORCH_CHECK(gt.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel() && scalars.numel() >= 2, "adamw: sizes");
  gd::AdamWArgs a{};
  if (p.scalar_type() == at::kBFloat16) a.p_bf16 = reinterpret_cast<__nv_bfloat16*>(p.data_ptr());
  else { TORCH_CHECK(p.scalar_type() == at::kFloat, "adamw: params must be bf16 or fp32"); a.p_f32 = p.data_ptr<float>(); }
  a.gt = f32_ptr(gt, "gt");
  a.gi = opt_f32(gi, "gi");
  a.m = f32_mut(m, "m");
  a.v = f32_mut(v, "v");
  a.scalars = f32_ptr(scalars, "scalars");
  a.n = p.numel();
  a.beta_proj = (float)beta_proj; a.lr = (float)lr; a.beta1 = (float)beta1; a.beta2 = (float)beta2;
  a.eps = (float)eps; a.weight_decay = (float)weight_decay;
  a.bc1 = (float)(1.0 - std::pow(beta1, (double)step));
  a.bc2 = (float)(1.0 - std::pow(beta2, (double)step));
  GD_LAUNCH(gd::launch_projected_adamw(a, stream_of(p)));
}

// tables: int64 device tensors of pointers (mats, vecs, outs) and int32 (rows, cols, is_bf16)
void batched_outer_add(const Tensor& dsts, const Tensor& ys, const Tensor& vecs, const Tensor& coef, const Tensor& rows,
                       const Tensor& cols, int64_t max_rows) {
  c10::cuda::CUDAGuard guard(dsts.device());
  OpRange gd_range_(__func__);
  const int n = (int)dsts.numel();
  TORCH_CHECK(ys.numel() == n && vecs.numel() == n && coef.numel() == n && rows.numel() == n && cols.numel() == n,
              "batched_outer_add: one entry per matrix");
  TORCH_CHECK(coef.is_contiguous() && coef.scalar_type() == at::kFloat, "batched_outer_add: coef must be fp32");
  GD_LAUNCH(gd::launch_batched_outer_add(reinterpret_cast<float* const*>(dsts.data_ptr<int64_t>()),
                                         reinterpret_cast<const float* const*>(ys.data_ptr<int64_t>()),
                                         reinterpret_cast<const float* const*>(vecs.data_ptr<int64_t>()),
                                         coef.data_ptr<float>(), rows.data_ptr<int>(), cols.data_ptr<int>(), n,
                                         (int)max_rows, stream_of(dsts)));
}

void batched_gemv(const Tensor& mats, const Tensor& vecs, const Tensor& outs, const Tensor& rows, const Tensor& cols,
                  const Tensor& is_bf16, int64_t max_rows) {
  c10::cuda::CUDAGuard guard(mats.device());
  OpRange gd_range_(__func__);
  const int n = (int)mats.numel();
  GD_LAUNCH(gd::launch_batched_gemv(reinterpret_cast<const void* const*>(mats.data_ptr<int64_t>()),
                                    reinterpret_cast<const float* const*>(vecs.data_ptr<int64_t>()),
                                    reinterpret_cast<float* const*>(outs.data_ptr<int64_t>()), rows.data_ptr<int>(),
                                    cols.data_ptr<int>(), is_bf16.data_ptr<int>(), n, (int)max_rows, stream_of(mats)));
}

void sn_power_iter(const Tensor& W, Tensor u, Tensor v, Tensor sigma, bool do_iter, double eps) {
  c10::cuda::CUDAGuard guard(W.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(W.is_cuda() && W.dim() == 2 && W.is_contiguous(), "sn_power_iter: W must be a contiguous CUDA matrix");
  TORCH_CHECK(W.scalar_type() == at::kBFloat16 || W.scalar_type() == at::kFloat, "sn_power_iter: W must be bf16 or fp32");
  TORCH_CHECK(u.is_contiguous() && v.is_contiguous() && u.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat &&
              u.numel() == W.size(0) && v.numel() == W.size(1) && sigma.scalar_type() == at::kFloat && sigma.numel() >= 1,
              "sn_power_iter: u (rows), v (cols), sigma (1) must be contiguous fp32");
  Tensor t = at::empty({W.size(0)}, u.options());
  GD_LAUNCH(gd::launch_sn_power_iter(W.data_ptr(), W.scalar_type() == at::kBFloat16, u.data_ptr<float>(), v.data_ptr<float>(),
                                     t.data_ptr<float>(), sigma.data_ptr<float>(), (int)W.size(0), (int)W.size(1), do_iter,
                                     (float)eps, stream_of(W)));
}

// ---- communication kernels over peer memory (comm.cu) -----------------------------------------
void allreduce_adamw(const Tensor& ptr_table_gt, const Tensor& ptr_table_gi, const Tensor& ptr_table_p,
                     const Tensor& signal_table, Tensor m, Tensor v, const Tensor& scalars, int64_t n, int64_t rank,
                     int64_t world, int64_t seq, int64_t phase, bool p_is_bf16, double beta_proj, double lr, double beta1,
                     double beta2, double eps, double weight_decay, int64_t step, Tensor shard_sums, bool gather_params,
                     OptT t_red, OptT timing, int64_t mc_gt, int64_t mc_gi, int64_t mc_p) {
  c10::cuda::CUDAGuard guard(m.device());
  OpRange gd_range_(__func__);
  gd::FusedReduceAdamWArgs a{};
  a.gt = reinterpret_cast<float* const*>(ptr_table_gt.data_ptr<int64_t>());
  a.gi = reinterpret_cast<float* const*>(ptr_table_gi.data_ptr<int64_t>());
  a.p = reinterpret_cast<void* const*>(ptr_table_p.data_ptr<int64_t>());
  a.signals = reinterpret_cast<uint32_t* const*>(signal_table.data_ptr<int64_t>());
  a.m = f32_mut(m, "m");
  a.v = f32_mut(v, "v");
  a.scalars = f32_ptr(scalars, "scalars");
  a.shard_sums = f32_mut(shard_sums, "shard_sums");
  a.n = n; a.rank = (int)rank; a.world = (int)world; a.seq = (uint32_t)seq; a.phase = (int)phase; a.p_is_bf16 = p_is_bf16;
  a.gather_params = gather_params;
  a.t_red = nullptr;
  if (t_red.has_value()) a.t_red = f32_mut(*t_red, "t_red");
  TORCH_CHECK(mc_gt % 16 == 0 && mc_gi % 16 == 0 && mc_p % 16 == 0, "multicast addresses must be 16-byte aligned");
  a.gt_mc = reinterpret_cast<const float*>(mc_gt);
  a.gi_mc = reinterpret_cast<const float*>(mc_gi);
  a.p_mc = reinterpret_cast<void*>(mc_p);
  a.timing = nullptr;
  if (timing.has_value()) {
    TORCH_CHECK(timing->is_cuda() && timing->scalar_type() == at::kLong && timing->numel() >= 4 && timing->is_contiguous(),
                "timing must be 4 int64 words on the device");
    a.timing = reinterpret_cast<unsigned long long*>(timing->data_ptr<int64_t>());
  }
  a.beta_proj = (float)beta_proj; a.lr = (float)lr; a.beta1 = (float)beta1; a.beta2 = (float)beta2;
  a.eps = (float)eps; a.weight_decay = (float)weight_decay;
  a.bc1 = (float)(1.0 - std::pow(beta1, (double)step));
  a.bc2 = (float)(1.0 - std::pow(beta2, (double)step));
  a.status = status_ptr(m);
  GD_LAUNCH(gd::launch_fused_reduce_adamw(a, stream_of(m)));
}

// dst += src where dst is a view into a registered spread gradient buffer (else a plain local add)
void peer_add(Tensor dst, const Tensor& src) {
  c10::cuda::CUDAGuard guard(dst.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(dst.is_cuda() && dst.scalar_type() == at::kFloat && dst.is_contiguous(), "peer_add: dst must be contiguous fp32");
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && src.numel() == dst.numel(), "peer_add: src must match dst");
  TORCH_CHECK(src.scalar_type() == at::kFloat || src.scalar_type() == at::kBFloat16, "peer_add: src must be fp32 or bf16");
  const GradSink* s = find_sink(dst.data_ptr());
  if (s == nullptr) {
    dst.add_(src.view_as(dst));
    return;
  }
  gd::PeerAddArgs a{};
  a.src = src.data_ptr();
  a.src_bf16 = src.scalar_type() == at::kBFloat16;
  a.table = reinterpret_cast<float* const*>(s->table.data_ptr<int64_t>());
  a.flat_off = (int64_t)((reinterpret_cast<uintptr_t>(dst.data_ptr()) - s->base) / 4);
  a.n = dst.numel();
  a.shard_elems = s->shard_elems;
  GD_LAUNCH(gd::launch_peer_add(a, stream_of(dst)));
}

// sink[off : off + n] += src for a gradient that lives sharded over the ranks (see register_virtual_grad_sink)
void peer_add_at(int64_t sink, int64_t off, const Tensor& src) {
  c10::cuda::CUDAGuard guard(src.device());
  OpRange gd_range_(__func__);
  const GradSink& s = sink_at(sink);
  TORCH_CHECK(s.elems < 0, "peer_add_at needs a virtual sink");
  TORCH_CHECK(src.is_cuda() && src.is_contiguous(), "peer_add_at: src must be a contiguous CUDA tensor");
  TORCH_CHECK(src.scalar_type() == at::kFloat || src.scalar_type() == at::kBFloat16, "peer_add_at: src must be fp32 or bf16");
  TORCH_CHECK(off >= 0 && off % 4 == 0 && off + src.numel() <= -s.elems, "peer_add_at: range outside the sink");
  gd::PeerAddArgs a{};
  a.src = src.data_ptr();
  a.src_bf16 = src.scalar_type() == at::kBFloat16;
  a.table = reinterpret_cast<float* const*>(s.table.data_ptr<int64_t>());
  a.flat_off = off;
  a.n = src.numel();
  a.shard_elems = s.shard_elems;
  GD_LAUNCH(gd::launch_peer_add(a, stream_of(src)));
}

void max_allreduce(Tensor vec, const Tensor& area_ptrs, const Tensor& flag_ptrs, int64_t slot_elems, int64_t rank,
                   int64_t world, int64_t seq, int64_t budget_ns, OptT gather_out) {
  c10::cuda::CUDAGuard guard(vec.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(vec.is_contiguous() && vec.scalar_type() == at::kFloat, "max_allreduce: vec must be contiguous fp32");
  TORCH_CHECK(area_ptrs.numel() == world && flag_ptrs.numel() == world, "max_allreduce: one pointer per rank");
  gd::MaxAllReduceArgs a{};
  a.vec = vec.data_ptr<float>();
  a.n = (int)vec.numel();
  a.areas = reinterpret_cast<float* const*>(area_ptrs.data_ptr<int64_t>());
  a.flags = reinterpret_cast<uint32_t* const*>(flag_ptrs.data_ptr<int64_t>());
  a.slot_elems = (int)slot_elems;
  a.rank = (int)rank; a.world = (int)world; a.seq = (uint32_t)seq;
  a.budget_ns = budget_ns > 0 ? (uint64_t)budget_ns : 0;
  a.gather_out = nullptr;
  if (gather_out.has_value()) {
    TORCH_CHECK(gather_out->is_contiguous() && gather_out->scalar_type() == at::kFloat && gather_out->numel() == world * vec.numel(),
                "max_allreduce: gather_out must be contiguous fp32 (world, n)");
    a.gather_out = gather_out->data_ptr<float>();
  }
  a.status = status_ptr(vec);
  GD_LAUNCH(gd::launch_max_allreduce(a, stream_of(vec)));
}

void halo_push_wait(const Tensor& tail, Tensor halo_out, const Tensor& slot_ptrs, const Tensor& flag_ptrs,
                    int64_t slot_offset_bytes, int64_t flag_index, int64_t rank, int64_t world, int64_t seq,
                    bool reverse, int64_t budget_ns) {
  c10::cuda::CUDAGuard guard(tail.device());
  OpRange gd_range_(__func__);
  TORCH_CHECK(tail.is_contiguous() && halo_out.is_contiguous() && tail.numel() == halo_out.numel(), "halo: shapes");
  TORCH_CHECK((tail.numel() * tail.element_size()) % 16 == 0, "halo: message must be a multiple of 16 bytes");
  gd::HaloArgs a{};
  a.tail = tail.data_ptr();
  a.halo_out = halo_out.data_ptr();
  a.nbytes = tail.numel() * tail.element_size();
  a.slots = reinterpret_cast<uint8_t* const*>(slot_ptrs.data_ptr<int64_t>());
  a.flags = reinterpret_cast<uint32_t* const*>(flag_ptrs.data_ptr<int64_t>());
  a.slot_offset = slot_offset_bytes;
  a.flag_index = (int)flag_index;
  a.rank = (int)rank; a.world = (int)world; a.seq = (uint32_t)seq; a.reverse = reverse;
  a.budget_ns = budget_ns > 0 ? (uint64_t)budget_ns : 0;
  a.status = status_ptr(tail);
  GD_LAUNCH(gd::launch_halo_push_wait(a, stream_of(tail)));
}

}  // namespace

TORCH_LIBRARY(gdnet_b200, m) {
  m.def("kernel_status(Tensor like) -> Tensor", &kernel_status);
  m.def("gemm_bf16(Tensor a, Tensor b, bool a_mn, bool b_mn, Tensor(a!) out, bool accumulate, Tensor? bias, Tensor? row_scale, Tensor? ssq_in, int norm_dim, float norm_eps, Tensor? aux, int aux_mode, Tensor? rowcoef, Tensor(b!)? pre_out, int act, Tensor(c!)? ssq_out, int sink=-1, int sink_off=0, int sink_ld=0) -> ()", &gemm_bf16);
  m.def("gemm_fp8(Tensor a8, Tensor sa, Tensor b8, Tensor sb, Tensor(a!) out, bool accumulate, Tensor? bias, Tensor? row_scale, Tensor? aux, int aux_mode, Tensor(b!)? pre_out, int act) -> ()", &gemm_fp8);
  m.def("gemm_fp8_mx(Tensor a8, Tensor pa, Tensor b8, Tensor pb, Tensor(a!) out, bool accumulate, Tensor? bias, Tensor? row_scale, Tensor? aux, int aux_mode, Tensor(b!)? pre_out, int act, Tensor(c!)? q8=None, Tensor(d!)? q8_p=None, bool q8_silu=False, bool store_out=True) -> ()", &gemm_fp8_mx);
  m.def("dwconv_fwd(Tensor x, Tensor? halo, Tensor w, Tensor(a!) out, Tensor(b!)? q=None, Tensor(c!)? qs=None, Tensor(d!)? qp=None) -> ()", &dwconv_fwd);
  m.def("dwconv_bwd(Tensor dc, Tensor x, Tensor? halo, Tensor w, Tensor? tail_add, Tensor(a!) dx, Tensor(b!)? dhalo, Tensor(c!) dw) -> ()", &dwconv_bwd);
  m.def("dwconv_fwd_sp(Tensor x, Tensor w, Tensor(a!) out, Tensor(b!) halo_out, Tensor slot_ptrs, Tensor flag_ptrs, Tensor(c!) counter, int slot_offset, int flag_index, int rank, int world, int seq, int budget_ns=0, Tensor(d!)? q=None, Tensor(e!)? qs=None, Tensor(f!)? qp=None) -> ()", &dwconv_fwd_sp);
  m.def("dwconv_bwd_sp(Tensor dc, Tensor x, Tensor halo, Tensor w, Tensor(a!) dx, Tensor(b!) dw, Tensor slot_ptrs, Tensor flag_ptrs, Tensor(c!) counter, int slot_offset, int flag_index, int rank, int world, int seq, int budget_ns=0) -> ()", &dwconv_bwd_sp);
  m.def("gate_update_fwd(Tensor g_pre, Tensor z, Tensor c, Tensor s, Tensor w_r, Tensor(a!) fwd_out, Tensor(b!) side_out, Tensor(c!)? gate_out, Tensor(d!)? rstd_out, Tensor(e!)? gate_sum, float eps_r, Tensor(f!)? q=None, Tensor(g!)? qs=None, Tensor(h!)? qp=None) -> ()", &gate_update_fwd);
  m.def("gate_only_fwd(Tensor g_pre, Tensor c, Tensor(a!) fwd_out, Tensor(b!) side_out, Tensor(c!)? gate_sum, Tensor(d!)? q=None, Tensor(e!)? qs=None, Tensor(f!)? qp=None) -> ()", &gate_only_fwd);
  m.def("gate_only_bwd(Tensor dF, Tensor dS, Tensor g_pre, Tensor c, Tensor b2g, Tensor ssq_g, float eps_g, Tensor? dgate_mean, Tensor(a!) dq, Tensor(b!) dc, Tensor(c!) rowcoef, Tensor(d!) db2g) -> ()", &gate_only_bwd);
  m.def("gate_update_bwd(Tensor dF, Tensor dS, Tensor g_pre, Tensor z, Tensor c, Tensor s, Tensor w_r, Tensor b2g, Tensor rstd_z, Tensor ssq_g, float eps_g, Tensor? dgate_mean, Tensor(a!) dq, Tensor(b!) dz, Tensor(c!) dsc, Tensor(d!) rowcoef, Tensor(e!) db2g, Tensor(f!) dw_r, Tensor(g!) db2r, Tensor(h!)? q=None, Tensor(i!)? qs=None, Tensor(j!)? qp=None) -> ()", &gate_update_bwd);
  m.def("gate_mix_fwd(Tensor g_pre, Tensor c, Tensor s, Tensor R, Tensor(a!) fwd_out, Tensor(b!) side_out) -> ()", &gate_mix_fwd);
  m.def("gate_mix_bwd(Tensor dF, Tensor dS, Tensor g_pre, Tensor c, Tensor s, Tensor R, Tensor? ssq, Tensor? b2, float eps, Tensor(a!) dgp, Tensor(b!)? dq, Tensor(c!) dc, Tensor(d!) ds, Tensor(e!) dR, Tensor(f!)? rowcoef) -> ()", &gate_mix_bwd);
  m.def("cam_blend_fwd(Tensor z, Tensor fwd, Tensor retr, Tensor w, int T, float eps, Tensor(a!) out, Tensor(b!) rstd) -> ()", &cam_blend_fwd);
  m.def("cam_blend_bwd(Tensor dout, Tensor z, Tensor fwd, Tensor retr, Tensor w, Tensor rstd, int T, float eps, Tensor(a!) dz, Tensor(b!) dfwd, Tensor(c!) dretr, Tensor(d!) dw) -> ()", &cam_blend_bwd);
  m.def("rmsnorm_fwd(Tensor x, Tensor w, Tensor(a!) y, Tensor(b!)? rstd, float eps) -> ()", &rmsnorm_fwd);
  m.def("rmsnorm_bwd(Tensor dy, Tensor x, Tensor w, Tensor rstd, Tensor(a!) dx, Tensor(b!) dw) -> ()", &rmsnorm_bwd);
  m.def("quant_tile(Tensor x, bool pre_silu, Tensor(a!)? q_row, Tensor(b!)? s_row, int row_mode, Tensor(c!)? q_col, Tensor(d!)? s_col, int col_mode, bool pow2=False, Tensor(e!)? p_row=None, Tensor(f!)? p_col=None, Tensor? peer_delta=None) -> ()", &quant_tile);
  m.def("quant_tensor(Tensor x, Tensor scale, Tensor(a!) q_row, Tensor(b!)? q_col, Tensor(c!)? amax) -> ()", &quant_tensor);
  m.def("colsum(Tensor x, Tensor(a!) out) -> ()", &colsum);
  m.def("segment_add(Tensor src, Tensor dst_addr, Tensor seg_off) -> ()", &segment_add);
  m.def("scale_cols(Tensor w, Tensor colw, Tensor(a!) out) -> ()", &scale_cols);
  m.def("unscale_cols_bwd(Tensor dW2w, Tensor W2, Tensor colw, Tensor(a!) dW2, Tensor(b!) dcolw) -> ()", &unscale_cols_bwd);
  m.def("cross_entropy(Tensor(a!) logits, Tensor targets, Tensor(b!) row_loss, Tensor inv_count, int vocab, int ignore_index, float grad_scale, bool write_grad) -> ()", &cross_entropy);
  m.def("mem_read_fwd(Tensor q, Tensor gamma, Tensor e, Tensor tags, Tensor vals, Tensor alpha, Tensor(a!) w, Tensor(b!) out) -> ()", &mem_read_fwd);
  m.def("mem_read_bwd(Tensor d_out, Tensor q, Tensor gamma, Tensor e, Tensor tags, Tensor vals, Tensor w, Tensor alpha, Tensor(a!) d_q, Tensor(b!) d_gamma, Tensor(c!) d_e, Tensor(d!) d_tags, Tensor(e!) d_vals, Tensor(f!) d_alpha) -> ()", &mem_read_bwd);
  m.def("grad_dots(Tensor gt, Tensor? gi, Tensor(a!) sums) -> ()", &grad_dots);
  m.def("projected_adamw(Tensor(a!) p, Tensor gt, Tensor? gi, Tensor(b!) m, Tensor(c!) v, Tensor scalars, float beta_proj, float lr, float beta1, float beta2, float eps, float weight_decay, int step) -> ()", &projected_adamw);
  m.def("batched_outer_add(Tensor dsts, Tensor ys, Tensor vecs, Tensor coef, Tensor rows, Tensor cols, int max_rows) -> ()", &batched_outer_add);
  m.def("sn_power_iter(Tensor W, Tensor(a!) u, Tensor(b!) v, Tensor(c!) sigma, bool do_iter, float eps) -> ()", &sn_power_iter);
  m.def("batched_gemv(Tensor mats, Tensor vecs, Tensor outs, Tensor rows, Tensor cols, Tensor is_bf16, int max_rows) -> ()", &batched_gemv);
  m.def("allreduce_adamw(Tensor ptr_table_gt, Tensor ptr_table_gi, Tensor ptr_table_p, Tensor signal_table, Tensor(a!) m, Tensor(b!) v, Tensor scalars, int n, int rank, int world, int seq, int phase, bool p_is_bf16, float beta_proj, float lr, float beta1, float beta2, float eps, float weight_decay, int step, Tensor(c!) shard_sums, bool gather_params=True, Tensor(d!)? t_red=None, Tensor(e!)? timing=None, int mc_gt=0, int mc_gi=0, int mc_p=0) -> ()", &allreduce_adamw);
  m.def("gemm_pair_capacity() -> int", []() -> int64_t { return gd::gemm_pair_capacity(); });
  m.def("gemm_set_mx_pair(int on) -> ()", [](int64_t on) { gd::gemm_set_mx_pair((int)on); });
  m.def("register_grad_sink(Tensor flat, Tensor ptr_table, int shard_elems) -> int", &register_grad_sink);
  m.def("unregister_grad_sink(int id) -> ()", &unregister_grad_sink);
  m.def("is_spread(Tensor t) -> bool", &is_spread);
  m.def("clear_grad_sinks() -> ()", &clear_grad_sinks);
  m.def("register_virtual_grad_sink(Tensor ptr_table, int total_elems, int shard_elems) -> int", &register_virtual_grad_sink);
  m.def("peer_add_at(int sink, int off, Tensor src) -> ()", &peer_add_at);
  m.def("attach_gather_jobs(Tensor jobs) -> ()", &attach_gather_jobs);
  m.def("attach_b_ready(Tensor b_ready, Tensor sfb_ready, int b_target, int sfb_target) -> ()", &attach_b_ready);
  m.def("gather_jobs(Tensor jobs) -> ()", &gather_jobs);
  m.def("peer_add(Tensor(a!) dst, Tensor src) -> ()", &peer_add);
  m.def("max_allreduce(Tensor(a!) vec, Tensor area_ptrs, Tensor flag_ptrs, int slot_elems, int rank, int world, int seq, int budget_ns=0, Tensor(b!)? gather_out=None) -> ()", &max_allreduce);
  m.def("halo_push_wait(Tensor tail, Tensor(a!) halo_out, Tensor slot_ptrs, Tensor flag_ptrs, int slot_offset_bytes, int flag_index, int rank, int world, int seq, bool reverse, int budget_ns=0) -> ()", &halo_push_wait);
}
