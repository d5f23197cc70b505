"""CUDA (sm_100a) implementations of the GDNet ops and their autograd wiring.

Everything here runs hand-written kernels from ``gdnet_b200/_C.so`` through
``torch.ops.gdnet_b200``. The module refuses to import without the library. Layout:

* thin wrappers that allocate outputs and call one kernel (``gemm``, ``quantize_*``, ...)
* autograd Functions: ``causal_dwconv``, ``rmsnorm``, ``fused_mem_read``, ``cross_entropy``,
  ``bf16_linear``, ``fp8_linear`` and the fused ``layer_step``
* gradients of weights go to ``param.main_grad`` (fp32, accumulated by the GEMM epilogue)
  when the training engine has installed it, else they are returned to autograd.

Activations are bf16. Small vectors (biases, norm weights, conv taps) are read as fp32
copies cached per parameter version.
"""

from __future__ import annotations

import os
import weakref

import torch

from .. import _ext
from . import reference as ref

_ext.load()


class _CountingOps:
    """Proxy of ``torch.ops.gdnet_b200`` that counts kernel launches (every op launches exactly one
    kernel of this library), so benchmarks can report how many of them ran."""

    def __init__(self, ns):
        self._ns = ns
        self.launches = 0
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            op = getattr(self._ns, name)

            def fn(*args, _op=op, **kw):
                self.launches += 1
                return _op(*args, **kw)

            self._cache[name] = fn
        return fn


K = _CountingOps(torch.ops.gdnet_b200)


def launch_count() -> int:
    return K.launches

AUX_ADD, AUX_MUL_SILU_GRAD, AUX_RMS_SILU_BWD = 1, 2, 3
ACT_NONE, ACT_SILU = 0, 1
Q_ROWS, Q_COLS, Q_BLOCK = 0, 1, 2
BF16, F32, FP8 = torch.bfloat16, torch.float32, torch.float8_e4m3fn


# --------------------------------------------------------------------------------------
# caches keyed on (tensor identity, version): fp32 copies of small vectors and FP8 weights
# --------------------------------------------------------------------------------------
_f32_cache: dict[int, tuple] = {}
_param_epoch = 0


def invalidate_param_caches() -> None:
    """Tell the caches that parameters changed behind autograd's back (the engine's fused
    optimizer writes the flat buffer, which does not bump the version of the parameter views)."""
    global _param_epoch
    _param_epoch += 1


def f32(t: torch.Tensor) -> torch.Tensor:
    """fp32 contiguous copy of a small parameter, refreshed when the parameter changes."""
    if t.dtype == F32 and t.is_contiguous():
        return t.detach()
    key = (t.data_ptr(), t.numel(), t.dtype)      # views of a parameter are new objects every time: key on storage
    hit = _f32_cache.get(key)
    if hit is not None and hit[0] == (t._version, t.data_ptr(), _param_epoch):
        return hit[1]
    out = t.detach().to(F32).contiguous()
    # the entry keeps `t` alive, so its storage address cannot be handed to another tensor while cached
    _f32_cache[key] = ((t._version, t.data_ptr(), _param_epoch), out, t)
    return out


_taps_cache: dict[int, tuple] = {}


def taps_t(w: torch.Tensor) -> torch.Tensor:
    """Conv taps ``(d, k)`` as an fp32 ``(k, d)`` table (what the conv kernels read), cached per version."""
    key = (w.data_ptr(), w.numel(), w.dtype)
    stamp = (w._version, w.data_ptr(), _param_epoch)
    hit = _taps_cache.get(key)
    if hit is not None and hit[0] == stamp:
        return hit[1]
    out = w.detach().to(F32).t().contiguous()
    _taps_cache[key] = (stamp, out, w)
    return out


class QuantizedWeight:
    """e4m3 copies of a weight ``(N, K)`` with 128x128 block scales: ``q`` / ``s`` for the
    forward GEMM and ``qt`` / ``st`` (the transposed matrix ``(K, N)``) for the data gradient."""

    __slots__ = ("q", "s", "qt", "st", "p", "pt", "version", "ptr", "source")


_wq_cache: dict[int, QuantizedWeight] = {}


class SharedWeights:
    """FP8 copies of the weights in symmetric memory, each weight quantised by ONE rank per parameter update.

    The owner's quantisation kernel stores every output byte into the same place of every rank's arena (peer
    stores over NVLink from inside ``quant_tile_kernel``), so the all-gather of the e4m3 weights is part of the
    kernel that produces them and moves half the bytes of a bf16 gather; the GEMMs then read their local copy
    through TMA. One bounded flag exchange per update tells every rank that all copies have landed.
    """

    ALIGN = 1024

    def __init__(self, weights, group, device):
        import torch.distributed as dist

        from ..parallel.symm import SymmBuffer

        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        plan, off = [], 0

        def take(nbytes):
            nonlocal off
            o = off
            off += -(-nbytes // self.ALIGN) * self.ALIGN
            return o

        for w in weights:
            N, Kd = w.shape
            nb, kb = N // 128, Kd // 128
            plan.append((w, take(N * Kd), take(nb * kb * 4), take(N * Kd), take(nb * kb * 4), take(nb * kb * 512),
                         take(nb * kb * 512)))
        self.arena = SymmBuffer(max(off, self.ALIGN), group, device)
        base = self.arena.ptrs[self.rank]
        self.peer_delta = torch.tensor([p - base for r, p in enumerate(self.arena.ptrs) if r != self.rank],
                                       dtype=torch.int64, device=device)
        self.entries: dict = {}
        self.owned = []
        loc = self.arena.local
        for i, (w, oq, os_, oqt, ost, op, opt) in enumerate(plan):
            N, Kd = w.shape
            nb, kb = N // 128, Kd // 128
            qw = QuantizedWeight()
            qw.q = loc[oq : oq + N * Kd].view(FP8).view(N, Kd)
            qw.s = loc[os_ : os_ + nb * kb * 4].view(F32).view(nb, kb)
            qw.qt = loc[oqt : oqt + N * Kd].view(FP8).view(Kd, N)
            qw.st = loc[ost : ost + nb * kb * 4].view(F32).view(kb, nb)
            qw.p = loc[op : op + nb * kb * 512].view(nb, kb, 512)
            qw.pt = loc[opt : opt + nb * kb * 512].view(kb, nb, 512)
            qw.version, qw.ptr, qw.source = None, w.data_ptr(), w
            self.entries[(w.data_ptr(), w.numel(), w.dtype)] = qw
            if i % self.world == self.rank:
                self.owned.append((w, qw))
        self.epoch = -1
        self._token = torch.zeros(1, dtype=F32, device=device)
        self.arena.barrier()

    def refresh(self) -> None:
        """Collective: every rank quantises the weights it owns into all arenas, then waits for the others."""
        from ..parallel.symm import max_allreduce_

        for w, qw in self.owned:
            K.quant_tile(w.detach(), False, qw.q, qw.s, Q_BLOCK, qw.qt, qw.st, Q_BLOCK, True, qw.p, qw.pt, self.peer_delta)
        max_allreduce_(self._token, self.group)      # flags + bounded waits: all peers' stores are complete and visible
        self.epoch = _param_epoch


# Providers installed by training engines (each engine owns its own and removes it when it is closed, so several
# engines can live in one process): shared FP8 weight caches and the weight streams of fully sharded engines.
_shared_list: list = []
_weight_streams: list = []


def share_fp8_weights(weights, group, device) -> SharedWeights:
    """Install a shared FP8 weight cache for ``weights`` (2-D bf16, both dims multiples of 128)."""
    sw = SharedWeights(list(weights), group, device)
    _shared_list.append(sw)
    return sw


def remove_provider(obj) -> None:
    for lst in (_shared_list, _weight_streams):
        if obj in lst:
            lst.remove(obj)


def refresh_shared_weights(sw=None) -> None:
    """Collective: bring a shared FP8 weight cache (default: all installed) up to date now. The training engine
    calls this right after every optimizer update, where all ranks are in lockstep, so that a later forward on one
    rank only (an evaluation on rank 0) never reaches the collective refresh by itself."""
    for s_ in ([sw] if sw is not None else list(_shared_list)):
        if s_.epoch != _param_epoch:
            s_.refresh()


def quantize_weight(w: torch.Tensor) -> QuantizedWeight:
    key = (w.data_ptr(), w.numel(), w.dtype)
    for sw in _shared_list:
        ent = sw.entries.get(key)
        if ent is not None:
            if sw.epoch != _param_epoch:
                sw.refresh()
            return ent
    hit = _wq_cache.get(key)
    stamp = (w._version, _param_epoch)
    if hit is not None and hit.version == stamp and hit.ptr == w.data_ptr():
        return hit
    N, Kd = w.shape
    nb, kb = (N + 127) // 128, (Kd + 127) // 128
    qw = hit if hit is not None and hit.q.shape == w.shape else QuantizedWeight()
    if hit is None or hit.q.shape != w.shape:
        qw.q = torch.empty(N, Kd, dtype=FP8, device=w.device)
        qw.s = torch.empty(nb, kb, dtype=F32, device=w.device)
        qw.qt = torch.empty(Kd, N, dtype=FP8, device=w.device)
        qw.st = torch.empty(kb, nb, dtype=F32, device=w.device)
        mx = N % 128 == 0 and Kd % 128 == 0
        qw.p = packed_buffer(N, Kd, w.device) if mx else None
        qw.pt = packed_buffer(Kd, N, w.device) if mx else None
    # power-of-two scales: the same copies serve the hardware-scaled and the software-scaled GEMM
    K.quant_tile(w.detach(), False, qw.q, qw.s, Q_BLOCK, qw.qt, qw.st, Q_BLOCK, True, qw.p, qw.pt)
    qw.version, qw.ptr, qw.source = stamp, w.data_ptr(), w   # `source` pins the storage address
    _wq_cache[key] = qw
    return qw


def clear_caches() -> None:
    """Drop every derived copy (they are rebuilt on demand). Providers installed by engines stay."""
    _f32_cache.clear()
    _wq_cache.clear()
    _taps_cache.clear()
    _w2w_cache.clear()
    _side_offers.clear()
    _seg_tables.clear()
    _sigma_plans.clear()


# --------------------------------------------------------------------------------------
# fully sharded parameters: gradient handles and the weight stream
# --------------------------------------------------------------------------------------
class GradRef:
    """Handle of a gradient that lives sharded over the ranks (no local full-size buffer): a registered virtual
    sink, the flat element offset of the matrix in it, its shape and row pitch. Stands where a ``main_grad``
    tensor would; the weight-gradient GEMM epilogue and ``peer_add_at`` add into the owner rank's shard."""

    __slots__ = ("sink", "off", "rows", "cols", "ld")

    def __init__(self, sink, off, rows, cols, ld=None):
        self.sink, self.off, self.rows, self.cols, self.ld = int(sink), int(off), int(rows), int(cols), int(ld or cols)

    def col_range(self, c0, n):
        return GradRef(self.sink, self.off + c0, self.rows, n, self.ld)

    @property
    def shape(self):
        return (self.rows, self.cols)


_shape_dummies: dict = {}


def _shape_only(device, M, N):
    """A (M, N) fp32 tensor without storage of its own (one element, stride 0): carries a shape to a binding."""
    d = _shape_dummies.get(device)
    if d is None:
        d = torch.zeros(1, dtype=F32, device=device)
        _shape_dummies[device] = d
    return d.expand(M, N)


def add_weight_stream(ws) -> None:
    """Install the provider of an engine's fully sharded layer weights
    (:class:`gdnet_b200.parallel.weight_stream.WeightStream`); ``remove_provider`` takes it out again."""
    _weight_streams.append(ws)


def _stream_for(rW1):
    """The weight stream that owns the layer step whose first recovery matrix is ``rW1``, or None."""
    for ws in _weight_streams:
        if ws.owns(rW1):
            return ws
    return None


def _attach_gather() -> None:
    for ws in _weight_streams:
        if ws.pending:
            ws.attach()
            return


# --------------------------------------------------------------------------------------
# GEMM wrappers
# --------------------------------------------------------------------------------------
def gemm_bf16(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=BF16, accumulate=False, bias=None,
              row_scale=None, ssq_in=None, norm_dim=0, norm_eps=0.0, aux=None, aux_mode=0, rowcoef=None,
              pre_out=None, act=ACT_NONE, ssq_out=None):
    """``D = A B^T`` on the tcgen05 tensor cores, bf16 operands, fp32 accumulation.

    ``a`` is ``(M, K)`` (or ``(K, M)`` with ``a_mn``), ``b`` is ``(N, K)`` (or ``(K, N)`` with
    ``b_mn``). See ``csrc/gemm_sm100.h`` for the epilogue order.
    """
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    _attach_gather()
    if isinstance(out, GradRef):
        # fp32 accumulation into the owner rank's shard of a gradient (the tensor only carries the shape)
        K.gemm_bf16(a, b, a_mn, b_mn, _shape_only(a.device, M, N), True, None, None, None, 0, 0.0, None, 0, None, None, 0,
                    None, out.sink, out.off, out.ld)
        return out
    if out is None:
        if out_dtype == F32:
            # a fresh fp32 result is a weight-gradient shape (few tiles, long reduction): start from zeros and
            # accumulate, which lets the launcher split the reduction over the idle SMs
            out = torch.zeros(M, N, dtype=F32, device=a.device)
            accumulate = True
        else:
            out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    K.gemm_bf16(a, b, a_mn, b_mn, out, accumulate, bias, row_scale, ssq_in, norm_dim, norm_eps, aux, aux_mode,
                rowcoef, pre_out, act, ssq_out)
    return out


def gemm_fp8(a8, sa, b8, sb, *, out=None, out_dtype=BF16, accumulate=False, bias=None, row_scale=None, aux=None,
             aux_mode=0, pre_out=None, act=ACT_NONE):
    """Block-scaled e4m3 GEMM: ``a8 (M,K)`` with ``sa (K/128, M)``, ``b8 (N,K)`` with ``sb (N/128, K/128)``."""
    M, N = a8.shape[0], b8.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a8.device)
    K.gemm_fp8(a8, sa, b8, sb, out, accumulate, bias, row_scale, aux, aux_mode, pre_out, act)
    return out


def gemm_fp8_mx(a8, pa, b8, pb, *, out=None, out_dtype=BF16, accumulate=False, bias=None, row_scale=None, aux=None,
                aux_mode=0, pre_out=None, act=ACT_NONE, q8=None, q8_p=None, q8_silu=False, store_out=True):
    """Hardware block-scaled e4m3 GEMM: power-of-two scales as packed UE8M0 chunks, ``pa (M/128, K/128, 512)``
    and ``pb (N/128, K/128, 512)`` bytes, applied by the tensor core (no promotion pass).

    ``q8``/``q8_p``: the epilogue also writes the result (through silu with ``q8_silu``) as the e4m3 A operand of
    the next GEMM, with one power-of-two scale per 64 columns of a row; ``store_out=False`` then skips ``out``."""
    M, N = a8.shape[0], b8.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a8.device)
    _attach_gather()
    K.gemm_fp8_mx(a8, pa, b8, pb, out, accumulate, bias, row_scale, aux, aux_mode, pre_out, act, q8, q8_p, q8_silu,
                  store_out)
    return out


def gemm_ok_bf16(M: int, N: int, Kd: int) -> bool:
    return Kd % 8 == 0 and N % 32 == 0 and M % 8 == 0


def gemm_ok_fp8(M: int, N: int, Kd: int) -> bool:
    return Kd % 128 == 0 and N % 128 == 0 and M % 16 == 0


# --------------------------------------------------------------------------------------
# quantisers
# --------------------------------------------------------------------------------------
def quantize_rows(x, pre_silu=False, q=None, s=None, pow2=False, packed=None):
    """1x128 blocks along the last dim: ``(q (M,K) e4m3, s (K/128, M) fp32)``. With ``pow2`` the scales
    are powers of two and ``packed`` (uint8 ``(M/128, K/128, 512)``) receives the UE8M0 chunks."""
    M, Kd = x.shape
    if q is None:
        q = torch.empty(M, Kd, dtype=FP8, device=x.device)
    if s is None:
        s = torch.empty((Kd + 127) // 128, M, dtype=F32, device=x.device)
    K.quant_tile(x, pre_silu, q, s, Q_ROWS, None, None, Q_BLOCK, pow2, packed, None)
    return q, s


def packed_buffer(rows: int, cols: int, device) -> torch.Tensor:
    """Uninitialised buffer for the UE8M0 chunks of a ``(rows, cols)`` operand."""
    return torch.empty(rows // 128, cols // 128, 512, dtype=torch.uint8, device=device)


def quantize_transposed(x, mode, pre_silu=False):
    """``x (M,K)`` -> ``x^T (K,M)`` in e4m3.

    ``mode=Q_COLS``: one scale per output row and 128 input rows, ``s (M/128, K)`` (the A operand
    of a weight-gradient GEMM). ``mode=Q_BLOCK``: 128x128 blocks, ``s (K/128, M/128)`` (the B operand).
    """
    M, Kd = x.shape
    qt = torch.empty(Kd, M, dtype=FP8, device=x.device)
    if mode == Q_COLS:
        st = torch.empty((M + 127) // 128, Kd, dtype=F32, device=x.device)
    else:
        st = torch.empty((Kd + 127) // 128, (M + 127) // 128, dtype=F32, device=x.device)
    K.quant_tile(x, pre_silu, None, None, Q_ROWS, qt, st, mode)
    return qt, st


def quantize_rows_and_transposed(x, col_mode):
    """Both copies from one read of ``x``: row-quantised ``(q, s)`` and transposed ``(qt, st)``."""
    M, Kd = x.shape
    q = torch.empty(M, Kd, dtype=FP8, device=x.device)
    s = torch.empty((Kd + 127) // 128, M, dtype=F32, device=x.device)
    qt = torch.empty(Kd, M, dtype=FP8, device=x.device)
    if col_mode == Q_COLS:
        st = torch.empty((M + 127) // 128, Kd, dtype=F32, device=x.device)
    else:
        st = torch.empty((Kd + 127) // 128, (M + 127) // 128, dtype=F32, device=x.device)
    K.quant_tile(x, False, q, s, Q_ROWS, qt, st, col_mode)
    return q, s, qt, st


def quantize_rows_mx(x, pre_silu=False, q=None, s=None, p=None):
    """1x128 quantisation with power-of-two scales for the hardware-scaled GEMM:
    ``(q (M,K), s (K/128, M) fp32, p (M/128, K/128, 512) packed UE8M0)``. ``q``/``s``/``p`` may be views
    into wider buffers (an operand assembled from several sources along K)."""
    M, Kd = x.shape
    if q is None:
        q = torch.empty(M, Kd, dtype=FP8, device=x.device)
    if s is None:
        s = torch.empty(Kd // 128, M, dtype=F32, device=x.device)
    if p is None:
        p = packed_buffer(M, Kd, x.device)
    K.quant_tile(x, pre_silu, q, s, Q_ROWS, None, None, Q_BLOCK, True, p, None)
    return q, s, p


def quantize_transposed_mx(x, mode, pre_silu=False, qt=None, st=None, pt=None):
    """``x (M,K)`` -> e4m3 ``x^T (K,M)`` with power-of-two scales and packed chunks ``pt (K/128, M/128, 512)``;
    ``mode`` as in :func:`quantize_transposed`."""
    M, Kd = x.shape
    if qt is None:
        qt = torch.empty(Kd, M, dtype=FP8, device=x.device)
    if st is None:
        st = torch.empty((M // 128, Kd) if mode == Q_COLS else (Kd // 128, M // 128), dtype=F32, device=x.device)
    if pt is None:
        pt = packed_buffer(Kd, M, x.device)
    K.quant_tile(x, pre_silu, None, None, Q_ROWS, qt, st, mode, True, None, pt)
    return qt, st, pt


def quantize_both_mx(x, col_mode):
    """Row-quantised and transposed copies from one read, power-of-two scales:
    ``(q, p, qt, pt)`` (the fp32 scale arrays are written too but not returned)."""
    M, Kd = x.shape
    q = torch.empty(M, Kd, dtype=FP8, device=x.device)
    s = torch.empty(Kd // 128, M, dtype=F32, device=x.device)
    p = packed_buffer(M, Kd, x.device)
    qt = torch.empty(Kd, M, dtype=FP8, device=x.device)
    st = torch.empty((M // 128, Kd) if col_mode == Q_COLS else (Kd // 128, M // 128), dtype=F32, device=x.device)
    pt = packed_buffer(Kd, M, x.device)
    K.quant_tile(x, False, q, s, Q_ROWS, qt, st, col_mode, True, p, pt)
    return q, p, qt, pt


def quantize_fp8_tensor(x, scale, need_col=True, out_row=None, out_col=None, amax_buf=None):
    """Per-tensor quantisation with a given scale (reference recipe,
    gdnet/kernel/fp8_linear/quantize.py:59-113): ``(x_row, x_col, amax)``."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1]).contiguous()
    M, Kd = x2.shape
    q = out_row if out_row is not None else torch.empty(M, Kd, dtype=FP8, device=x.device)
    qc = None
    if need_col:
        qc = out_col if out_col is not None else torch.empty(Kd, M, dtype=FP8, device=x.device)
    amax = amax_buf if amax_buf is not None else torch.zeros(1, dtype=F32, device=x.device)
    K.quant_tensor(x2, scale.reshape(-1).to(F32), q, qc, amax)
    return q.reshape(shape), (qc if need_col else q), amax.squeeze()


# --------------------------------------------------------------------------------------
# gradient sinks: fp32 main_grad (training engine) or autograd
# --------------------------------------------------------------------------------------
def set_spread_grads(on: bool) -> None:
    """Kept for callers of earlier versions: whether a gradient buffer is spread over the ranks is now asked per
    tensor (``_is_spread``: it lies inside a buffer registered with ``register_grad_sink``, or it is a ``GradRef``)."""


def _is_spread(mg) -> bool:
    return isinstance(mg, GradRef) or (mg is not None and mg.is_cuda and bool(K.is_spread(mg)))


def _main_grad(p):
    return getattr(p, "main_grad", None)


def accumulate_main_grad(mg, g) -> None:
    """mg += g for a ``main_grad`` view; over NVLink into the owning rank's buffer when gradients are spread."""
    if isinstance(mg, GradRef):
        g = g.reshape(mg.rows, mg.cols)
        if mg.ld == mg.cols:
            K.peer_add_at(mg.sink, mg.off, g.contiguous())
        else:
            for r in range(mg.rows):
                K.peer_add_at(mg.sink, mg.off + r * mg.ld, g[r].contiguous())
        return
    if mg.is_cuda and mg.dtype == F32 and mg.is_contiguous():
        K.peer_add(mg, g.contiguous())       # a plain local add when mg lies in no spread buffer
    else:
        mg.add_(g.view_as(mg))


def _sink_vec(p, g32):
    """Deliver the fp32 gradient of a small parameter: add to ``main_grad`` or return it."""
    mg = _main_grad(p)
    if mg is not None:
        accumulate_main_grad(mg, g32)
        return None
    return g32.to(p.dtype).view_as(p)


_seg_tables: dict = {}


def _sink_vecs(params, packed, views, mgs=None):
    """Deliver the gradients of several small parameters that sit back to back in ``packed`` (``views`` are the
    per-parameter views of it): one ``segment_add`` launch for all of them that have a local fp32 ``main_grad``
    (installed by the training engine); the others (no ``main_grad``, e.g. a derived view such as the conv taps,
    or gradients spread over ranks) go one by one."""
    if mgs is None:
        mgs = [_main_grad(p) for p in params]
    batch = [i for i, m in enumerate(mgs) if m is not None and not isinstance(m, GradRef) and m.dtype == F32
             and m.is_contiguous()]
    if batch and _is_spread(mgs[batch[0]]):      # the small parameters of a step share one flat buffer
        batch = []
    out = [None] * len(params)
    for i, (p, v) in enumerate(zip(params, views)):
        if i not in batch:
            out[i] = _sink_vec(p, v)
    if batch:
        key = tuple(mgs[i].data_ptr() for i in batch) + tuple(batch)
        tab = _seg_tables.get(key)
        if tab is None:
            offs, o = [], 0
            for v in views:
                offs.append(o)
                o += v.numel()
            # segments must be ascending and cover [first offset, total): give the skipped ranges a dummy target
            addrs, segs = [], []
            scratch = torch.zeros(max(v.numel() for v in views), dtype=F32, device=packed.device)
            for i, v in enumerate(views):
                addrs.append(mgs[i].data_ptr() if i in batch else scratch.data_ptr())
                segs.append(offs[i])
            tab = (torch.tensor(addrs, dtype=torch.int64, device=packed.device),
                   torch.tensor(segs, dtype=torch.int32, device=packed.device), scratch)
            _seg_tables[key] = tab
        K.segment_add(packed, tab[0], tab[1])
    return out


def _wgrad_target(p):
    """(buffer to accumulate into, is_main_grad). Without main_grad a fresh zero fp32 buffer."""
    mg = _main_grad(p)
    if mg is not None:
        return mg, True
    return torch.zeros(p.shape, dtype=F32, device=p.device), False


# --------------------------------------------------------------------------------------
# causal depthwise conv
# --------------------------------------------------------------------------------------
class _CausalDWConvFn(torch.autograd.Function):
    """x (B,T,d) bf16, w (d,k), halo (B,k-1,d) or None -> (B,T,d). The halo gets a gradient
    (it is the previous shard's tail), delivered through the halo exchange."""

    @staticmethod
    def forward(ctx, x, w, halo):
        xc = x if x.stride(-1) == 1 else x.contiguous()
        out = torch.empty(x.shape, dtype=BF16, device=x.device)
        K.dwconv_fwd(xc, halo, taps_t(w), out)
        ctx.save_for_backward(xc, w, halo if halo is not None else xc.new_empty(0))
        ctx.has_halo = halo is not None
        return out

    @staticmethod
    def backward(ctx, dc):
        x, w, halo = ctx.saved_tensors
        halo = halo if ctx.has_halo else None
        dc = dc if dc.stride(-1) == 1 else dc.contiguous()
        dx = torch.empty(x.shape, dtype=BF16, device=x.device)
        dw = torch.zeros(w.shape, dtype=F32, device=x.device)
        dhalo = torch.empty_like(halo) if halo is not None else None
        K.dwconv_bwd(dc, x, halo, taps_t(w), None, dx, dhalo, dw)
        return dx, _sink_vec(w, dw), dhalo


def causal_dwconv(x, w, halo=None):
    if x.dtype != BF16:
        return ref.causal_dwconv(x, w, halo)
    return _CausalDWConvFn.apply(x, w, halo)


# --------------------------------------------------------------------------------------
# RMSNorm
# --------------------------------------------------------------------------------------
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], dtype=F32, device=x.device)
        K.rmsnorm_fwd(x2, f32(w), y, rstd, eps)
        ctx.save_for_backward(x2, w, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        dy2 = dy.reshape(x2.shape).contiguous()
        dx = torch.empty_like(x2)
        dw = torch.zeros(w.shape, dtype=F32, device=x2.device)
        K.rmsnorm_bwd(dy2, x2, f32(w), rstd, dx, dw)
        return dx.view(dy.shape), _sink_vec(w, dw), None


def rmsnorm(x, w, eps):
    if x.dtype != BF16 or x.shape[-1] % 8 != 0:
        return ref.rmsnorm(x, w, eps)
    return _RMSNormFn.apply(x, w, float(eps))


# --------------------------------------------------------------------------------------
# fused CAM read
# --------------------------------------------------------------------------------------
class _MemReadFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, gamma, e, tags, vals, alpha):
        args = [t.detach().to(F32).contiguous() for t in (q, gamma, e, tags, vals)]
        al = alpha.detach().to(F32).reshape(1).contiguous()
        B, S, _ = args[3].shape
        w = torch.empty(B, S, dtype=F32, device=q.device)
        out = torch.empty(B, args[4].shape[2], dtype=F32, device=q.device)
        K.mem_read_fwd(*args, al, w, out)
        ctx.save_for_backward(*args, w, al)
        ctx.dtypes = (q.dtype, gamma.dtype, e.dtype, tags.dtype, vals.dtype, alpha.dtype)
        ctx.alpha_shape = alpha.shape
        ctx.mark_non_differentiable(w)
        return out.to(q.dtype), w

    @staticmethod
    def backward(ctx, d_out, _dw):
        q, gamma, e, tags, vals, w, al = ctx.saved_tensors
        d_q, d_gamma, d_e = torch.empty_like(q), torch.empty_like(gamma), torch.zeros_like(e)
        d_tags, d_vals = torch.empty_like(tags), torch.empty_like(vals)
        d_alpha = torch.zeros(1, dtype=F32, device=q.device)
        K.mem_read_bwd(d_out.to(F32).contiguous(), q, gamma, e, tags, vals, w, al, d_q, d_gamma, d_e, d_tags,
                       d_vals, d_alpha)
        dt = ctx.dtypes
        return (d_q.to(dt[0]), d_gamma.to(dt[1]), d_e.to(dt[2]), d_tags.to(dt[3]), d_vals.to(dt[4]),
                d_alpha.to(dt[5]).view(ctx.alpha_shape))


def fused_mem_read(q, gamma, e, tags, vals, alpha):
    """``(retrieved (B,d_c) in q.dtype, w (B,S) fp32, no grad)``; one kernel forward, one backward
    (reference: gdnet/kernel/fused_mem_read/function.py:8-56)."""
    return _MemReadFn.apply(q, gamma, e, tags, vals, alpha)


# --------------------------------------------------------------------------------------
# cross-entropy (mean over non-ignored rows), gradient written in place of the logits
# --------------------------------------------------------------------------------------
class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, vocab, ignore_index):
        n, _ = logits.shape
        tgt = targets.reshape(-1).contiguous()
        # rows whose target is out of range are dropped by the kernel (and reported in the status word)
        count = ((tgt != ignore_index) & (tgt >= 0) & (tgt < vocab)).sum().clamp(min=1).to(F32)
        inv = (1.0 / count).reshape(1)
        row_loss = torch.empty(n, dtype=F32, device=logits.device)
        need_grad = logits.requires_grad
        # the kernel overwrites the logits with d(mean loss)/d(logits): work on the caller's buffer when it
        # is a bf16 temporary that nothing else will read, which is the case for the model's head output
        buf = logits.detach()
        K.cross_entropy(buf, tgt, row_loss, inv, vocab, ignore_index, 1.0, need_grad)
        if need_grad:
            ctx.save_for_backward(buf)
        return row_loss.sum() * inv[0]

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return dlogits * g.to(dlogits.dtype), None, None, None


def cross_entropy(logits, targets, ignore_index=-100, vocab=None):
    """Mean cross-entropy over ``logits (n, V)`` bf16. **Consumes** the logits buffer (it is
    overwritten with the gradient). Columns ``>= vocab`` are excluded from the softmax."""
    if logits.dtype != BF16 or logits.stride(-1) != 1 or logits.stride(0) % 8 != 0 or logits.dim() != 2:
        lg = logits.reshape(-1, logits.shape[-1])
        return ref.cross_entropy(lg if vocab is None else lg[:, :vocab], targets.reshape(-1), ignore_index)
    return _CrossEntropyFn.apply(logits, targets, logits.shape[1] if vocab is None else vocab, ignore_index)


class _LinearCrossEntropyFn(torch.autograd.Function):
    """Vocabulary projection and mean cross-entropy in row chunks: per chunk the head GEMM writes bf16 logits,
    the loss kernel turns them into the gradient in place, and the data- and weight-gradient GEMMs consume them
    at once, so only one chunk of logits exists at a time (0.5 GB instead of 2.1 GB at 32768 x 32000) and the
    gradient of the head is ready when forward returns. Backward only scales by the incoming gradient."""

    @staticmethod
    def forward(ctx, x2, w, targets, vocab, fp8, chunk_rows):
        M, Kd = x2.shape
        Vp = w.shape[0]
        dev = x2.device
        tgt = targets.reshape(-1).contiguous()
        count = ((tgt >= 0) & (tgt < vocab)).sum().clamp(min=1).to(F32)    # -100 (ignored) and bad ids drop out
        inv = (1.0 / count).reshape(1)
        row_loss = torch.empty(M, dtype=F32, device=dev)
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dx = torch.empty_like(x2) if need_dx else None
        dw = torch.zeros(Vp, Kd, dtype=F32, device=dev) if need_dw else None
        qw = quantize_weight(w) if fp8 else None
        for r0 in range(0, M, chunk_rows):
            r1 = min(M, r0 + chunk_rows)
            xc = x2[r0:r1]
            if fp8:
                x8, _, px = quantize_rows_mx(xc)
                logits = gemm_fp8_mx(x8, px, qw.q, qw.p)
            else:
                logits = gemm_bf16(xc, w)
            K.cross_entropy(logits, tgt[r0:r1], row_loss[r0:r1], inv, vocab, -100, 1.0, need_dx or need_dw)
            if need_dx:
                if fp8:
                    d8, _, pd = quantize_rows_mx(logits)
                    gemm_fp8_mx(d8, pd, qw.qt, qw.pt, out=dx[r0:r1])
                else:
                    gemm_bf16(logits, w, b_mn=True, out=dx[r0:r1])
            if need_dw:
                gemm_bf16(logits, xc, a_mn=True, b_mn=True, out=dw, accumulate=True)
        empty = x2.new_empty(0)
        ctx.save_for_backward(dx if dx is not None else empty, dw if dw is not None else empty, w)
        return row_loss.sum() * inv[0]

    @staticmethod
    def backward(ctx, g):
        dx, dw, w = ctx.saved_tensors
        gx = (dx * g.to(dx.dtype)) if dx.numel() else None
        gw = None
        if dw.numel():
            dw = dw * g.to(F32)
            mg = _main_grad(w)
            if mg is not None:
                accumulate_main_grad(mg, dw)
            else:
                gw = dw.to(w.dtype)
        return gx, gw, None, None, None, None


def linear_cross_entropy(x, w, targets, vocab, fp8: bool, chunk_rows: int = 8192):
    """``cross_entropy((x @ w^T)[:, :vocab], targets)`` without keeping the logits; ``x (M, K)`` bf16, ``w (Vp, K)``
    bf16. ``fp8``: block-scaled e4m3 forward and data gradient (M and the chunk multiples of 128)."""
    return _LinearCrossEntropyFn.apply(x, w, targets, int(vocab), bool(fp8), int(chunk_rows))


def linear_cross_entropy_ok(x2, w, fp8: bool) -> bool:
    M, Kd = x2.shape
    ok = x2.dtype == BF16 and w.dtype == BF16 and x2.is_contiguous() and w.is_contiguous()
    ok = ok and Kd % 32 == 0 and w.shape[0] % 32 == 0 and M % 8 == 0
    if fp8:
        ok = ok and M % 128 == 0 and Kd % 128 == 0 and w.shape[0] % 128 == 0
    return ok


# --------------------------------------------------------------------------------------
# linears: bf16 and block-scaled FP8, tensor-core GEMMs for fprop, dgrad and wgrad
# --------------------------------------------------------------------------------------
def _wgrad_bf16(dy, x, w):
    """``dW (N,K) += dy^T x``: reduction over tokens, both operands read MN-major in place."""
    tgt, is_main = _wgrad_target(w)
    gemm_bf16(dy, x, a_mn=True, b_mn=True, out=tgt, accumulate=True)
    return None if is_main else tgt.to(w.dtype)


def _wgrad_bf16_cat(dy, xs, w):
    """``dW (N, sum K_i) += dy^T [x_0 | x_1 | ...]`` without building the concatenation: one GEMM per column
    range of the gradient."""
    tgt, is_main = _wgrad_target(w)
    o = 0
    for x in xs:
        part = tgt.col_range(o, x.shape[1]) if isinstance(tgt, GradRef) else tgt[:, o : o + x.shape[1]]
        gemm_bf16(dy, x, a_mn=True, b_mn=True, out=part, accumulate=True)
        o += x.shape[1]
    return None if is_main else tgt.to(w.dtype)


def _bias_grad(dy, b):
    if b is None:
        return None
    g = torch.zeros(b.shape, dtype=F32, device=dy.device)
    K.colsum(dy, g)
    return _sink_vec(b, g)


class _LinearBf16Fn(torch.autograd.Function):
    """y = x W^T + b with bf16 operands. dgrad reads W MN-major (no transposed copy)."""

    @staticmethod
    def forward(ctx, x2, w, b):
        ctx.save_for_backward(x2, w, b if b is not None else x2.new_empty(0))
        ctx.has_bias = b is not None
        return gemm_bf16(x2, w, bias=b)

    @staticmethod
    def backward(ctx, dy):
        x2, w, b = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm_bf16(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _wgrad_bf16(dy, x2, w)
        db = _bias_grad(dy, b if ctx.has_bias else None)
        return dx, dw, db


def linear_bf16(x, w, b=None):
    """Tensor-core bf16 linear for any leading shape; weights are expected in bf16."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    M, Kd, N = x2.shape[0], shape[-1], w.shape[0]
    if x2.dtype != BF16 or w.dtype != BF16 or not gemm_ok_bf16(M, N, Kd) or N % 8 or Kd % 32 or M % 32:
        return torch.nn.functional.linear(x, w.to(x.dtype), None if b is None else b.to(x.dtype))
    if x2.stride(-1) != 1 or (x2.stride(0) * 2) % 16:
        x2 = x2.contiguous()
    return _LinearBf16Fn.apply(x2, w, b).view(*shape[:-1], N)


class _LinearFp8BlockFn(torch.autograd.Function):
    """Block-scaled e4m3 linear (1x128 activations and gradients, 128x128 weights, power-of-two scales).

    fprop: x8 (rows) x W8.  dgrad: dy8 (rows) x (W^T)8.  The weight gradient dy^T x runs in bf16 with both
    operands read in place (MN-major), accumulated in fp32: it is as fast as the e4m3 form once the transposed
    quantised copies that form needs are counted, and it is the more precise of the two.
    """

    @staticmethod
    def forward(ctx, x2, w, b):
        qw = quantize_weight(w)
        x8, _, px = quantize_rows_mx(x2)
        ctx.save_for_backward(x2 if ctx.needs_input_grad[1] else x2.new_empty(0), w,
                              b if b is not None else x2.new_empty(0))
        ctx.has_bias = b is not None
        return gemm_fp8_mx(x8, px, qw.q, qw.p, bias=b)

    @staticmethod
    def backward(ctx, dy):
        x2, w, b = ctx.saved_tensors
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            qw = quantize_weight(w)
            dy8, _, pdy = quantize_rows_mx(dy)
            dx = gemm_fp8_mx(dy8, pdy, qw.qt, qw.pt)
        dw = _wgrad_bf16(dy, x2, w) if ctx.needs_input_grad[1] else None
        db = _bias_grad(dy, b if ctx.has_bias else None)
        return dx, dw, db


class _LinearFp8TensorFn(torch.autograd.Function):
    """Per-tensor delayed scaling (the reference's recipe) on the same block-scaled kernel: the
    block-scale arrays are filled with the one inverse scale."""

    @staticmethod
    def forward(ctx, x2, w, b, mod):
        M, Kd = x2.shape
        N = w.shape[0]
        x8, xt8, _ = quantize_fp8_tensor(x2, mod.scale_x, True, amax_buf=mod._amax_x)
        quantize_fp8_tensor(w.detach(), mod.scale_w, True, out_row=mod._w_fp8_row, out_col=mod._w_fp8_col,
                            amax_buf=mod._amax_w)
        sx = mod.inv_scale_x.to(F32).expand((Kd + 127) // 128, M).contiguous()
        sw = mod.inv_scale_w.to(F32).expand((N + 127) // 128, (Kd + 127) // 128).contiguous()
        ctx.save_for_backward(xt8, w, b if b is not None else x2.new_empty(0))
        ctx.mod, ctx.has_bias = mod, b is not None
        return gemm_fp8(x8, sx, mod._w_fp8_row, sw, bias=b)

    @staticmethod
    def backward(ctx, dy):
        xt8, w, b = ctx.saved_tensors
        mod = ctx.mod
        dy = dy.contiguous()
        M, N = dy.shape
        Kd = w.shape[1]
        scale_g = (ref.FP8_MAX / dy.abs().amax().float().clamp(min=1e-12)).reshape(1)
        inv_g = scale_g.reciprocal()
        dy8, dyt8, _ = quantize_fp8_tensor(dy, scale_g, True)
        kb, nb, mb = (Kd + 127) // 128, (N + 127) // 128, (M + 127) // 128
        dx = gemm_fp8(dy8, inv_g.expand(nb, M).contiguous(), mod._w_fp8_col,
                      mod.inv_scale_w.to(F32).expand(kb, nb).contiguous())
        tgt, is_main = _wgrad_target(w)
        gemm_fp8(dyt8, inv_g.expand(mb, N).contiguous(), xt8,
                 mod.inv_scale_x.to(F32).expand(kb, mb).contiguous(), out=tgt, accumulate=True)
        dw = None if is_main else tgt.to(w.dtype)
        db = _bias_grad(dy, b if ctx.has_bias else None)
        return dx, dw, db, None


def fp8_linear(x2, mod):
    """Forward of an :class:`FP8Linear` on a ``(M, K)`` bf16 CUDA tensor."""
    M, Kd = x2.shape
    N = mod.out_features
    if not gemm_ok_fp8(M, N, Kd) or M % 128:
        return linear_bf16(x2, mod.weight, mod.bias)
    if x2.stride(-1) != 1 or (x2.stride(0) * 2) % 16:
        x2 = x2.contiguous()
    if mod.recipe == "tensor":
        return _LinearFp8TensorFn.apply(x2, mod.weight, mod.bias, mod)
    return _LinearFp8BlockFn.apply(x2, mod.weight, mod.bias)


# --------------------------------------------------------------------------------------
# one fused GDLayer step
# --------------------------------------------------------------------------------------
_w2w_cache: dict[tuple[int, int], tuple] = {}


def _folded_w2(W2, w_norm):
    """``W2 * w_norm[None, :]`` in bf16, cached per version of both parameters: lets the RMSNorm
    in front of ``W2`` become a per-row scale in the GEMM epilogue."""
    key = (W2.data_ptr(), w_norm.data_ptr(), W2.numel())
    hit = _w2w_cache.get(key)
    stamp = (W2._version, w_norm._version, W2.data_ptr(), _param_epoch)
    if hit is not None and hit[:3] == stamp[:3] and hit[4] == _param_epoch:
        return hit[3]
    out = hit[3] if hit is not None and hit[3].shape == W2.shape else torch.empty_like(W2, dtype=BF16)
    K.scale_cols(W2.detach(), f32(w_norm), out)
    _w2w_cache[key] = (W2._version, w_norm._version, W2.data_ptr(), out, _param_epoch, W2, w_norm)
    return out


# The update kernel of a step also writes the FP8 copy of its side output, straight into the operand buffer
# of the step that will consume it. The hand-over is keyed on the identity (and version) of the side tensor.
_side_offers: dict = {}     # id(side tensor) -> (weak reference, version, (u8, su, pu))


def _alloc_u8(M, d, dev):
    kb = d // 128
    return (torch.empty(M, 2 * d, dtype=FP8, device=dev), torch.empty(2 * kb, M, dtype=F32, device=dev),
            packed_buffer(M, 2 * d, dev))


def _offer_side_q8(side_out, bufs) -> None:
    """After a step: remember the buffers ``bufs = (u8, su, pu)`` its update kernel filled for ``side_out`` (every
    layer keeps its own side stream, so several offers are open at a time; one dies with its tensor)."""
    key = id(side_out)
    _side_offers[key] = (weakref.ref(side_out, lambda _r, k=key: _side_offers.pop(k, None)), side_out._version, bufs)


def _claim_side_q8(side):
    """Before a step: the (u8, su, pu) buffers whose s half already holds ``side`` in FP8, or None."""
    o = _side_offers.pop(id(side), None)
    if o is None or o[0]() is not side or o[1] != side._version:
        return None
    u8 = o[2][0]
    if u8.shape[0] * u8.shape[1] != 2 * side.numel() or u8.shape[1] != 2 * side.shape[-1]:
        return None
    return o[2]


class _LayerStepFn(torch.autograd.Function):
    """conv -> recovery gate R -> forward gate g -> stream update, as one autograd node.

    Inputs: x, s (B,T,d) bf16; halo (B,k-1,d) or None; the 11 parameters of the step.
    Outputs: fwd', side' (B,T,d) bf16 and the sum of g over all elements (fp32 scalar; its mean
    is the information-loss term). ``fp8`` selects block-scaled e4m3 GEMMs for the recovery MLP;
    the gate MLP runs in bf16, as in the reference (gdnet/layer.py:130-139).
    """

    @staticmethod
    def forward(ctx, x, s, halo, conv_w, rW1, rb1, rW2, rb2, rnw, gW1, gb1, gnw, gW2, gb2, fp8, eps_r, eps_g,
                want_gate_sum, side_q8=None, sp=None):
        B, T, d = x.shape
        M = B * T
        dev = x.device
        train = any(ctx.needs_input_grad)
        # outputs nobody differentiates (the FP8 buffers handed to the next step, an unused stream) arrive in backward
        # as None instead of freshly zero-filled tensors
        ctx.set_materialize_grads(False)
        x = x if x.is_contiguous() else x.contiguous()
        s2 = s.reshape(M, d) if s.stride(-1) == 1 else s.contiguous().reshape(M, d)
        c3 = torch.empty(B, T, d, dtype=BF16, device=dev)
        c = c3.view(M, d)
        kb = d // 128
        if fp8:
            # A operand of the first recovery GEMM: [s ; c] in e4m3. The conv kernel writes the c half itself;
            # the s half usually comes from the step that produced s (its update kernel left it in the buffer)
            if side_q8 is not None:
                u8, su, pu = side_q8
            else:
                u8, su, pu = _alloc_u8(M, d, dev)
                quantize_rows_mx(s2, q=u8[:, :d], s=su[:kb], p=pu[:, :kb])
            qargs = (u8[:, d:], su[kb:], pu[:, kb:])
        else:
            qargs = ()
        if sp is not None:
            # sequence parallel: the kernel itself sends this shard's last rows to the next rank and waits for the
            # previous rank's; what it received is kept for the backward pass
            halo = torch.empty(B, conv_w.shape[1] - 1, d, dtype=BF16, device=dev)
            K.dwconv_fwd_sp(x, taps_t(conv_w), c3, halo, *sp.fwd_args(), 0, *qargs)
        else:
            K.dwconv_fwd(x, halo, taps_t(conv_w), c3, *qargs)

        # recovery MLP: z = W2r silu(W1r [s ; c] + b1r) + b2r
        h1_pre = torch.empty(M, d, dtype=BF16, device=dev)
        # fully sharded weights: the operands of this step come from the weight stream (gathered from their owners
        # by the GEMMs themselves); otherwise they are derived from the local parameters and cached
        W = None
        ws = _stream_for(rW1)
        if ws is not None:
            if not fp8:
                raise RuntimeError("fully sharded layer weights need the FP8 block recipe for the recovery MLP")
            W = ws.acquire(rW1, "F")
        if fp8 and W is not None:
            q1q, q1p, q2q, q2p = W.q1, W.p1, W.q2, W.p2
        elif fp8:
            q1, q2 = quantize_weight(rW1), quantize_weight(rW2)
            q1q, q1p, q2q, q2p = q1.q, q1.p, q2.q, q2.p
        if fp8:
            # silu(h1) leaves the first GEMM already quantised for the second; h1 and silu(h1) in bf16 are
            # written only when a backward will need them
            a8 = torch.empty(M, d, dtype=FP8, device=dev)
            pa = packed_buffer(M, d, dev)
            if train:
                a1 = torch.empty(M, d, dtype=BF16, device=dev)
                gemm_fp8_mx(u8, pu, q1q, q1p, out=a1, bias=f32(rb1), pre_out=h1_pre, act=ACT_SILU, q8=a8, q8_p=pa)
            else:
                a1 = None
                gemm_fp8_mx(u8, pu, q1q, q1p, out=h1_pre, bias=f32(rb1), q8=a8, q8_p=pa, q8_silu=True,
                            store_out=False)
            z = gemm_fp8_mx(a8, pa, q2q, q2p, bias=f32(rb2))
        else:
            gemm_bf16(s2, rW1[:, :d], out=h1_pre)
            a1 = torch.empty(M, d, dtype=BF16, device=dev)
            gemm_bf16(c, rW1[:, d:], out=a1, bias=f32(rb1), aux=h1_pre, aux_mode=AUX_ADD, pre_out=h1_pre,
                      act=ACT_SILU)
            z = gemm_bf16(a1, rW2, bias=f32(rb2))

        # gate MLP: g_pre = W2g RMSNorm(silu(W1g c + b1g)) + b2g, the norm folded into W2g and a row scale
        parts = (d + 127) // 128
        ssq = torch.empty(M, parts, dtype=F32, device=dev)
        hg_pre = torch.empty(M, d, dtype=BF16, device=dev) if train else None
        h = gemm_bf16(c, gW1 if W is None else W.gW1, bias=f32(gb1), act=ACT_SILU, pre_out=hg_pre, ssq_out=ssq)
        W2w = _folded_w2(gW2, gnw) if W is None else W.W2w
        g_pre = gemm_bf16(h, W2w, bias=f32(gb2), ssq_in=ssq, norm_dim=d, norm_eps=eps_g)

        fwd_out = torch.empty(B, T, d, dtype=BF16, device=dev)
        side_out = torch.empty(B, T, d, dtype=BF16, device=dev)
        rstd_z = torch.empty(M, dtype=F32, device=dev)
        gate_sum = torch.zeros((), dtype=F32, device=dev) if want_gate_sum else None
        if fp8:
            nu8, nsu, npu = _alloc_u8(M, d, dev)      # the next step's [s ; c] operand: this kernel fills the s half
            K.gate_update_fwd(g_pre, z, c, s2, f32(rnw), fwd_out.view(M, d), side_out.view(M, d), None, rstd_z,
                              gate_sum if want_gate_sum else None, eps_r, nu8[:, :d], nsu[:kb], npu[:, :kb])
        else:
            nu8 = nsu = npu = None
            K.gate_update_fwd(g_pre, z, c, s2, f32(rnw), fwd_out.view(M, d), side_out.view(M, d), None, rstd_z,
                              gate_sum if want_gate_sum else None, eps_r)

        if train:
            empty = x.new_empty(0)
            ctx.save_for_backward(x, s2, halo if halo is not None else empty, c, h1_pre, a1 if a1 is not None else empty,
                                  z, hg_pre, h, ssq, g_pre, rstd_z, conv_w, rW1, rb1, rW2, rb2, rnw, gW1, gb1, gnw,
                                  gW2, gb2)
            ctx.cfg = (B, T, d, fp8, eps_g, halo is not None)
            ctx.sp = sp
            ctx.conv_param = getattr(conv_w, "base_param", None)   # the taps are a view of this parameter
        if nu8 is not None:
            ctx.mark_non_differentiable(nu8, nsu, npu)
        # the last three: the next step's [s ; c] operand with its s half filled (FP8 mode), handed to the caller
        return fwd_out, side_out, gate_sum, nu8, nsu, npu

    @staticmethod
    def backward(ctx, dF, dS, dgsum, _du8=None, _dsu=None, _dpu=None):
        (x, s2, halo, c, h1_pre, a1, z, hg_pre, h, ssq, g_pre, rstd_z, conv_w, rW1, rb1, rW2, rb2, rnw, gW1, gb1,
         gnw, gW2, gb2) = ctx.saved_tensors
        B, T, d, fp8, eps_g, has_halo = ctx.cfg
        M = B * T
        dev = x.device
        halo = halo if has_halo else None

        def rows(t):
            t = t.reshape(M, d) if t.stride(-1) == 1 else t.contiguous().reshape(M, d)
            return t if (t.stride(0) * 2) % 16 == 0 else t.contiguous()

        dF2 = rows(dF) if dF is not None else torch.zeros(M, d, dtype=BF16, device=dev)
        dS2 = rows(dS) if dS is not None else torch.zeros(M, d, dtype=BF16, device=dev)
        # d(loss)/d(mean g) = dgsum * (M*d) because gate_sum = (M*d) * mean
        dgm = None
        if dgsum is not None:
            dgm = (dgsum.to(F32) * float(M * d)).reshape(1)

        dq = torch.empty(M, d, dtype=BF16, device=dev)
        dz = torch.empty(M, d, dtype=BF16, device=dev)
        dsc = torch.empty(M, 2 * d, dtype=BF16, device=dev)
        rowcoef = torch.empty(M, dtype=F32, device=dev)
        # gradients of the seven small parameters of the step live in one zeroed buffer (one fill, and one
        # launch to deliver them): gb2, rnw, rb2, gnw, gb1, rb1, conv taps
        k_taps = conv_w.shape[1]
        vec = torch.zeros(6 * d + d * k_taps, dtype=F32, device=dev)
        db2g, dw_r, db2r, dgnw, db1g, db1r = (vec[i * d : (i + 1) * d] for i in range(6))
        dwc = vec[6 * d :].view(d, k_taps)
        if fp8:      # dz leaves the kernel already row-quantised for the data-gradient GEMM of the recovery MLP
            dz8 = torch.empty(M, d, dtype=FP8, device=dev)
            sdz = torch.empty(d // 128, M, dtype=F32, device=dev)
            pdz = packed_buffer(M, d, dev)
            K.gate_update_bwd(dF2, dS2, g_pre, z, c, s2, f32(rnw), f32(gb2), rstd_z, ssq, eps_g, dgm, dq, dz, dsc,
                              rowcoef, db2g, dw_r, db2r, dz8, sdz, pdz)
        else:
            K.gate_update_bwd(dF2, dS2, g_pre, z, c, s2, f32(rnw), f32(gb2), rstd_z, ssq, eps_g, dgm, dq, dz, dsc,
                              rowcoef, db2g, dw_r, db2r)

        # ---- gate MLP ----
        W = None
        ws = _stream_for(rW1)
        if ws is not None:
            W = ws.acquire(rW1, "B")       # gathered by the first GEMM below (or prefetched by the last step)
        W2w = _folded_w2(gW2, gnw) if W is None else W.W2w
        gW1_op = gW1 if W is None else W.gW1
        gW2_raw = gW2.detach() if W is None else W.gW2
        dW2w = gemm_bf16(dq, h, a_mn=True, b_mn=True, out_dtype=F32)
        tgt2, main2 = _wgrad_target(gW2)
        if main2 and _is_spread(tgt2):
            dW2 = torch.zeros_like(dW2w)
            K.unscale_cols_bwd(dW2w, gW2_raw, f32(gnw), dW2, dgnw)
            accumulate_main_grad(tgt2, dW2)
        else:
            K.unscale_cols_bwd(dW2w, gW2_raw, f32(gnw), tgt2, dgnw)
        dh_pre = gemm_bf16(dq, W2w, b_mn=True, aux=hg_pre, aux_mode=AUX_RMS_SILU_BWD, rowcoef=rowcoef)
        K.colsum(dh_pre, db1g)
        g_gW1 = _wgrad_bf16(dh_pre, c, gW1)
        dc_view = dsc[:, d:]
        gemm_bf16(dh_pre, gW1_op, b_mn=True, out=dc_view, aux=dc_view, aux_mode=AUX_ADD)

        # ---- recovery MLP ----
        if fp8:
            # data gradients in e4m3 (row-quantised dz, dh1); weight gradients in bf16 with both operands read
            # in place, which needs no transposed quantised copies
            if W is not None:
                q1t, p1t, q2t, p2t = W.q1, W.p1, W.q2, W.p2
            else:
                q1, q2 = quantize_weight(rW1), quantize_weight(rW2)
                q1t, p1t, q2t, p2t = q1.qt, q1.pt, q2.qt, q2.pt
            g_rW2 = _wgrad_bf16(dz, a1, rW2)
            dh8 = torch.empty(M, d, dtype=FP8, device=dev)      # dh1 quantised by the GEMM that produces it
            pdh = packed_buffer(M, d, dev)
            dh1 = gemm_fp8_mx(dz8, pdz, q2t, p2t, aux=h1_pre, aux_mode=AUX_MUL_SILU_GRAD, q8=dh8, q8_p=pdh)
            K.colsum(dh1, db1r)
            g_rW1 = _wgrad_bf16_cat(dh1, (s2, c), rW1)
            gemm_fp8_mx(dh8, pdh, q1t, p1t, out=dsc, aux=dsc, aux_mode=AUX_ADD)
        else:
            g_rW2 = _wgrad_bf16(dz, a1, rW2)
            dh1 = gemm_bf16(dz, rW2, b_mn=True, aux=h1_pre, aux_mode=AUX_MUL_SILU_GRAD)
            K.colsum(dh1, db1r)
            g_rW1 = _wgrad_bf16_cat(dh1, (s2, c), rW1)
            gemm_bf16(dh1, rW1, b_mn=True, out=dsc, aux=dsc, aux_mode=AUX_ADD)

        # ---- conv ----
        dx = torch.empty(B, T, d, dtype=BF16, device=dev)
        if ctx.sp is not None:
            # the gradient of the received rows goes to the previous rank and the next rank's is added to the last
            # rows of dx, both inside the kernel
            dhalo = None
            K.dwconv_bwd_sp(dsc.view(B, T, 2 * d)[:, :, d:], x, halo, taps_t(conv_w), dx, dwc, *ctx.sp.bwd_args(), 0)
        else:
            dhalo = torch.empty_like(halo) if halo is not None else None
            K.dwconv_bwd(dsc.view(B, T, 2 * d)[:, :, d:], x, halo, taps_t(conv_w), None, dx, dhalo, dwc)
        ds = dsc.view(B, T, 2 * d)[:, :, :d]

        g_gW2 = None if main2 else tgt2.to(gW2.dtype)
        smalls = (gb2, rnw, rb2, gnw, gb1, rb1, conv_w)
        mgs = [_main_grad(p) for p in smalls]
        if mgs[-1] is None and ctx.conv_param is not None:
            mg = _main_grad(ctx.conv_param)          # the buffer installed for THIS backward pass
            if mg is not None and not _is_spread(mg):
                mgs[-1] = mg.view(conv_w.shape)
        g_gb2, g_rnw, g_rb2, g_gnw, g_gb1, g_rb1, g_conv = _sink_vecs(
            smalls, vec, (db2g, dw_r, db2r, dgnw, db1g, db1r, dwc), mgs)
        return (dx, ds, dhalo, g_conv, g_rW1, g_rb1, g_rW2, g_rb2, g_rnw, g_gW1, g_gb1, g_gnw, g_gW2, g_gb2,
                None, None, None, None, None, None)


class _LayerStepZeroSideFn(torch.autograd.Function):
    """The layer step for a side stream that is identically zero (the first forward step of every layer: the model
    starts its side streams at zero, reference gdnet/model.py:142-146): ``fwd' = c g``, ``side' = c (1 - g)``.

    The recovery gate only ever multiplies the side stream (``fwd' = c g + s R``, gdnet/layer.py:123-145), so with
    ``s = 0`` its value does not reach the outputs and its parameters receive exactly zero gradient from this step;
    the two recovery GEMMs, their data- and weight-gradient GEMMs and the recovery half of the update kernels are
    not run. Outputs and gradients are those of :class:`_LayerStepFn` fed an explicit zero tensor
    (``tests/test_gpu_ops.py::test_zero_side_step_matches_explicit_zeros``).

    Inputs: x (B,T,d) bf16; halo or None; the conv taps and the five gate parameters; ``rW1`` only names the layer
    for the weight stream. Outputs as :class:`_LayerStepFn`."""

    @staticmethod
    def forward(ctx, x, halo, conv_w, rW1, gW1, gb1, gnw, gW2, gb2, fp8, eps_g, want_gate_sum, sp=None):
        B, T, d = x.shape
        M = B * T
        dev = x.device
        train = any(ctx.needs_input_grad)
        ctx.set_materialize_grads(False)
        x = x if x.is_contiguous() else x.contiguous()
        c3 = torch.empty(B, T, d, dtype=BF16, device=dev)
        c = c3.view(M, d)
        if sp is not None:
            halo = torch.empty(B, conv_w.shape[1] - 1, d, dtype=BF16, device=dev)
            K.dwconv_fwd_sp(x, taps_t(conv_w), c3, halo, *sp.fwd_args(), 0)
        else:
            K.dwconv_fwd(x, halo, taps_t(conv_w), c3)
        W = None
        ws = _stream_for(rW1)
        if ws is not None:
            W = ws.acquire(rW1, "F")         # keeps the stream's request order; the gate operands come from it
            ws.settle()                      # the first GEMM here is a bf16 one: it cannot wait on arriving operands
        parts = (d + 127) // 128
        ssq = torch.empty(M, parts, dtype=F32, device=dev)
        hg_pre = torch.empty(M, d, dtype=BF16, device=dev) if train else None
        h = gemm_bf16(c, gW1 if W is None else W.gW1, bias=f32(gb1), act=ACT_SILU, pre_out=hg_pre, ssq_out=ssq)
        W2w = _folded_w2(gW2, gnw) if W is None else W.W2w
        g_pre = gemm_bf16(h, W2w, bias=f32(gb2), ssq_in=ssq, norm_dim=d, norm_eps=eps_g)
        fwd_out = torch.empty(B, T, d, dtype=BF16, device=dev)
        side_out = torch.empty(B, T, d, dtype=BF16, device=dev)
        gate_sum = torch.zeros((), dtype=F32, device=dev) if want_gate_sum else None
        if fp8:
            kb = d // 128
            nu8, nsu, npu = _alloc_u8(M, d, dev)      # the next step's [s ; c] operand: this kernel fills the s half
            K.gate_only_fwd(g_pre, c, fwd_out.view(M, d), side_out.view(M, d), gate_sum, nu8[:, :d], nsu[:kb], npu[:, :kb])
        else:
            nu8 = nsu = npu = None
            K.gate_only_fwd(g_pre, c, fwd_out.view(M, d), side_out.view(M, d), gate_sum)
        if train:
            empty = x.new_empty(0)
            ctx.save_for_backward(x, halo if halo is not None else empty, c, hg_pre, h, ssq, g_pre, conv_w, rW1, gW1, gb1,
                                  gnw, gW2, gb2)
            ctx.cfg = (B, T, d, eps_g, halo is not None)
            ctx.sp = sp
            ctx.conv_param = getattr(conv_w, "base_param", None)
        if nu8 is not None:
            ctx.mark_non_differentiable(nu8, nsu, npu)
        return fwd_out, side_out, gate_sum, nu8, nsu, npu

    @staticmethod
    def backward(ctx, dF, dS, dgsum, _du8=None, _dsu=None, _dpu=None):
        x, halo, c, hg_pre, h, ssq, g_pre, conv_w, rW1, gW1, gb1, gnw, gW2, gb2 = ctx.saved_tensors
        B, T, d, eps_g, has_halo = ctx.cfg
        M = B * T
        dev = x.device
        halo = halo if has_halo else None

        def rows(t):
            t = t.reshape(M, d) if t.stride(-1) == 1 else t.contiguous().reshape(M, d)
            return t if (t.stride(0) * 2) % 16 == 0 else t.contiguous()

        dF2 = rows(dF) if dF is not None else torch.zeros(M, d, dtype=BF16, device=dev)
        dS2 = rows(dS) if dS is not None else torch.zeros(M, d, dtype=BF16, device=dev)
        dgm = None
        if dgsum is not None:
            dgm = (dgsum.to(F32) * float(M * d)).reshape(1)
        dq = torch.empty(M, d, dtype=BF16, device=dev)
        dc = torch.empty(M, d, dtype=BF16, device=dev)
        rowcoef = torch.empty(M, dtype=F32, device=dev)
        k_taps = conv_w.shape[1]
        vec = torch.zeros(3 * d + d * k_taps, dtype=F32, device=dev)        # gb2, gnw, gb1, conv taps
        db2g, dgnw, db1g = (vec[i * d : (i + 1) * d] for i in range(3))
        dwc = vec[3 * d :].view(d, k_taps)
        K.gate_only_bwd(dF2, dS2, g_pre, c, f32(gb2), ssq, eps_g, dgm, dq, dc, rowcoef, db2g)

        W = None
        ws = _stream_for(rW1)
        if ws is not None:
            W = ws.acquire(rW1, "B")
        W2w = _folded_w2(gW2, gnw) if W is None else W.W2w
        gW1_op = gW1 if W is None else W.gW1
        gW2_raw = gW2.detach() if W is None else W.gW2
        dW2w = gemm_bf16(dq, h, a_mn=True, b_mn=True, out_dtype=F32)
        tgt2, main2 = _wgrad_target(gW2)
        if main2 and _is_spread(tgt2):
            dW2 = torch.zeros_like(dW2w)
            K.unscale_cols_bwd(dW2w, gW2_raw, f32(gnw), dW2, dgnw)
            accumulate_main_grad(tgt2, dW2)
        else:
            K.unscale_cols_bwd(dW2w, gW2_raw, f32(gnw), tgt2, dgnw)
        dh_pre = gemm_bf16(dq, W2w, b_mn=True, aux=hg_pre, aux_mode=AUX_RMS_SILU_BWD, rowcoef=rowcoef)
        K.colsum(dh_pre, db1g)
        g_gW1 = _wgrad_bf16(dh_pre, c, gW1)
        gemm_bf16(dh_pre, gW1_op, b_mn=True, out=dc, aux=dc, aux_mode=AUX_ADD)

        dx = torch.empty(B, T, d, dtype=BF16, device=dev)
        if ctx.sp is not None:
            dhalo = None
            K.dwconv_bwd_sp(dc.view(B, T, d), x, halo, taps_t(conv_w), dx, dwc, *ctx.sp.bwd_args(), 0)
        else:
            dhalo = torch.empty_like(halo) if halo is not None else None
            K.dwconv_bwd(dc.view(B, T, d), x, halo, taps_t(conv_w), None, dx, dhalo, dwc)

        g_gW2 = None if main2 else tgt2.to(gW2.dtype)
        smalls = (gb2, gnw, gb1, conv_w)
        mgs = [_main_grad(p) for p in smalls]
        if mgs[-1] is None and ctx.conv_param is not None:
            mg = _main_grad(ctx.conv_param)
            if mg is not None and not _is_spread(mg):
                mgs[-1] = mg.view(conv_w.shape)
        g_gb2, g_gnw, g_gb1, g_conv = _sink_vecs(smalls, vec, (db2g, dgnw, db1g, dwc), mgs)
        return (dx, dhalo, g_conv, None, g_gW1, g_gb1, g_gnw, g_gW2, g_gb2, None, None, None, None)


def zero_side_step_ok(fwd, layer, r) -> bool:
    """The zero-side form of the fused step covers the widths of its update kernels."""
    return fwd.is_cuda and fwd.shape[-1] in (256, 512, 1024, 2048) and _fused_step_ok(fwd, None, layer, r)


# --------------------------------------------------------------------------------------
# public kernel API: gate MLP + stream update with the recovery gate given
# --------------------------------------------------------------------------------------
class _GateMixFn(torch.autograd.Function):
    """``fwd' = c g + s R``, ``side' = c (1 - g) + s (1 - R)`` with ``g = sigmoid(g_pre)``; all four inputs get
    gradients (reference kernels: gdnet/kernel/gated_causal_depthwise_conv/gate_norm.py:34-102)."""

    @staticmethod
    def forward(ctx, g_pre, c, s, R):
        M, d = g_pre.shape
        fo = torch.empty(M, d, dtype=BF16, device=g_pre.device)
        so = torch.empty(M, d, dtype=BF16, device=g_pre.device)
        K.gate_mix_fwd(g_pre, c, s, R, fo, so)
        ctx.save_for_backward(g_pre, c, s, R)
        return fo, so

    @staticmethod
    def backward(ctx, dF, dS):
        g_pre, c, s, R = ctx.saved_tensors
        outs = [torch.empty_like(g_pre) for _ in range(4)]
        K.gate_mix_bwd(dF.contiguous(), dS.contiguous(), g_pre, c, s, R, None, None, 0.0, outs[0], None, outs[1], outs[2],
                       outs[3], None)
        return tuple(outs)


def _rows_bf16(t, M, d):
    t = t.reshape(M, d)
    if t.dtype != BF16:
        t = t.to(BF16)
    return t if t.stride(1) == 1 and (t.stride(0) * 2) % 16 == 0 else t.contiguous()


def gate_stream_update(g_pre, c, s, R):
    """CUDA form of the stand-alone stream update; ``(fwd', side')`` bf16 ``(rows, d)``."""
    M, d = g_pre.shape
    return _GateMixFn.apply(_rows_bf16(g_pre, M, d).contiguous(), _rows_bf16(c, M, d), _rows_bf16(s, M, d), _rows_bf16(R, M, d))


class _GatedOutputFn(torch.autograd.Function):
    """The reference's ``GatedCausalDepthwiseConvFunction`` (gdnet/kernel/gated_causal_depthwise_conv/function.py:11-87)
    on the sm_100a kernels: gate MLP ``g_pre = W2 RMSNorm(silu(W1 c + b1)) + b2`` as two tensor-core GEMMs (silu and
    the row sums of squares in the first epilogue, the norm as a per-row scale in the second, with the norm weight
    folded into ``W2``'s columns), then the stream update with the recovery gate ``R`` given. Backward: one kernel
    for the update and the row terms of the norm, then weight- and data-gradient GEMMs; gradients for all nine inputs."""

    @staticmethod
    def forward(ctx, c, s, R, W1, b1, Wn, W2, b2, eps):
        M, d = c.shape
        dev = c.device
        ssq = torch.empty(M, (d + 127) // 128, dtype=F32, device=dev)
        h_pre = torch.empty(M, d, dtype=BF16, device=dev)
        h = gemm_bf16(c, W1, bias=f32(b1), act=ACT_SILU, pre_out=h_pre, ssq_out=ssq)
        W2w = torch.empty(W2.shape, dtype=BF16, device=dev)
        K.scale_cols(W2.detach().contiguous(), f32(Wn), W2w)
        g_pre = gemm_bf16(h, W2w, bias=f32(b2), ssq_in=ssq, norm_dim=d, norm_eps=eps)
        fo = torch.empty(M, d, dtype=BF16, device=dev)
        so = torch.empty(M, d, dtype=BF16, device=dev)
        K.gate_mix_fwd(g_pre, c, s, R, fo, so)
        ctx.save_for_backward(c, s, R, W1, b1, Wn, W2, b2, h_pre, h, ssq, g_pre, W2w)
        ctx.eps = eps
        return fo, so

    @staticmethod
    def backward(ctx, dF, dS):
        c, s, R, W1, b1, Wn, W2, b2, h_pre, h, ssq, g_pre, W2w = ctx.saved_tensors
        M, d = c.shape
        dev = c.device
        dgp, dq, dc, ds, dR = (torch.empty(M, d, dtype=BF16, device=dev) for _ in range(5))
        rowcoef = torch.empty(M, dtype=F32, device=dev)
        K.gate_mix_bwd(dF.contiguous(), dS.contiguous(), g_pre, c, s, R, ssq, f32(b2), ctx.eps, dgp, dq, dc, ds, dR, rowcoef)
        db2 = torch.zeros(d, dtype=F32, device=dev)
        K.colsum(dgp, db2)
        dW2w = gemm_bf16(dq, h, a_mn=True, b_mn=True, out_dtype=F32)
        dW2 = torch.zeros(W2.shape, dtype=F32, device=dev)
        dWn = torch.zeros(d, dtype=F32, device=dev)
        K.unscale_cols_bwd(dW2w, W2.detach().contiguous(), f32(Wn), dW2, dWn)
        dh_pre = gemm_bf16(dq, W2w, b_mn=True, aux=h_pre, aux_mode=AUX_RMS_SILU_BWD, rowcoef=rowcoef)
        db1 = torch.zeros(d, dtype=F32, device=dev)
        K.colsum(dh_pre, db1)
        dW1 = gemm_bf16(dh_pre, c, a_mn=True, b_mn=True, out_dtype=F32)
        gemm_bf16(dh_pre, W1, b_mn=True, out=dc, aux=dc, aux_mode=AUX_ADD)
        return (dc, ds, dR, dW1.to(W1.dtype), db1.to(b1.dtype), dWn.to(Wn.dtype), dW2.to(W2.dtype), db2.to(b2.dtype), None)


def gated_output_ok(c, W1, W2) -> bool:
    M, d = c.shape
    return c.is_cuda and d % 128 == 0 and M % 128 == 0 and W1.shape == (d, d) and W2.shape == (d, d)


def gated_output(c, s, R, W1, b1, Wn, W2, b2, eps):
    M, d = c.shape
    w1 = W1 if W1.dtype == BF16 and W1.is_contiguous() else W1.to(BF16).contiguous()
    w2 = W2 if W2.dtype == BF16 and W2.is_contiguous() else W2.to(BF16).contiguous()
    return _GatedOutputFn.apply(_rows_bf16(c, M, d), _rows_bf16(s, M, d), _rows_bf16(R, M, d), w1, b1, Wn, w2, b2, float(eps))


def rmsnorm_fwd(x2, w, eps):
    """``(y, rstd)`` of a bf16 ``(rows, d)`` tensor, one kernel (no autograd)."""
    y = torch.empty_like(x2)
    rstd = torch.empty(x2.shape[0], dtype=F32, device=x2.device)
    K.rmsnorm_fwd(x2, f32(w), y, rstd, float(eps))
    return y, rstd


# --------------------------------------------------------------------------------------
# hard spectral norm of one linear (torch.nn.utils.spectral_norm's arithmetic on one kernel)
# --------------------------------------------------------------------------------------
class _SpectralScaleFn(torch.autograd.Function):
    """``W / sigma`` with ``sigma = u^T W v`` for fixed ``u, v``: ``dW = (dWn - <dWn, Wn> u v^T) / sigma``."""

    @staticmethod
    def forward(ctx, W, sigma, u, v):
        Wn = (W.float() / sigma).to(W.dtype)
        ctx.save_for_backward(Wn, sigma, u, v)
        return Wn

    @staticmethod
    def backward(ctx, dWn):
        Wn, sigma, u, v = ctx.saved_tensors
        g = dWn.float()
        inner = (g * Wn.float()).sum()
        return ((g - inner * torch.outer(u, v)) / sigma).to(Wn.dtype), None, None, None


def spectral_weight(mod):
    """The weight of a module wrapped by ``torch.nn.utils.spectral_norm`` (parameters ``weight_orig``, buffers
    ``weight_u`` / ``weight_v``), computed as torch's pre-forward hook computes it: in training mode one power
    iteration that updates ``u`` and ``v`` in place, then ``weight_orig / (u^T W v)`` with the gradient flowing through
    the division and through sigma. The iteration and sigma are one single-block kernel
    (``csrc/loss_optim.cu:sn_power_iter_kernel``); reference: gdnet/memory.py:68."""
    W = mod.weight_orig
    u, v = mod.weight_u, mod.weight_v
    Wm = W.detach().reshape(W.shape[0], -1).contiguous()
    u32, v32 = u.detach().float().contiguous(), v.detach().float().contiguous()
    sigma = torch.empty(1, dtype=F32, device=W.device)
    K.sn_power_iter(Wm, u32, v32, sigma, bool(mod.training), 1e-12)
    if mod.training:
        with torch.no_grad():
            u.copy_(u32)
            v.copy_(v32)
    return _SpectralScaleFn.apply(W, sigma, u32, v32)


# --------------------------------------------------------------------------------------
# read-out of the content-addressed memory
# --------------------------------------------------------------------------------------
class _CamReadoutFn(torch.autograd.Function):
    """``out = fwd (1 - R) + retrieved R`` with ``R = sigmoid(RMSNorm(W2 silu(Ws side + Wf fwd + row_bias) + b2))``
    (reference: gdnet/memory.py:127-139; ``Ws`` / ``Wf`` are the side and forward-stream blocks of the
    spectral-normalised ``W_r1``, the retrieved vector and the entropy enter as ``row_bias (B, d)``, constant along
    T). The token-sized GEMMs run on the tcgen05 kernels, one launch per batch row so that the per-row bias is an
    ordinary column bias; silu is an epilogue; norm, sigmoid and blend are one kernel forward and one backward."""

    @staticmethod
    def forward(ctx, side, fwd, retrieved, row_bias, Ws, Wf, W2, b2, wn, eps):
        B, T, d = fwd.shape
        M = B * T
        dev = fwd.device
        side2, fwd2 = side.reshape(M, d), fwd.reshape(M, d)
        pre = torch.empty(M, d, dtype=BF16, device=dev)
        a = torch.empty(M, d, dtype=BF16, device=dev)
        rb = row_bias.to(F32).contiguous()
        for b in range(B):
            rows = slice(b * T, (b + 1) * T)
            gemm_bf16(side2[rows], Ws, out=pre[rows])
            gemm_bf16(fwd2[rows], Wf, out=a[rows], bias=rb[b], aux=pre[rows], aux_mode=AUX_ADD, pre_out=pre[rows], act=ACT_SILU)
        z = gemm_bf16(a, W2, bias=f32(b2))
        out = torch.empty(M, d, dtype=BF16, device=dev)
        rstd = torch.empty(M, dtype=F32, device=dev)
        retr = retrieved.to(BF16).contiguous()
        K.cam_blend_fwd(z, fwd2, retr, f32(wn), T, eps, out, rstd)
        ctx.save_for_backward(side2, fwd2, retr, Ws, Wf, W2, b2, wn, pre, a, z, rstd)
        ctx.cfg = (B, T, d, eps, retrieved.dtype, row_bias.dtype)
        return out.view(B, T, d)

    @staticmethod
    def backward(ctx, dout):
        side2, fwd2, retr, Ws, Wf, W2, b2, wn, pre, a, z, rstd = ctx.saved_tensors
        B, T, d, eps, retr_dtype, rb_dtype = ctx.cfg
        M = B * T
        dev = fwd2.device
        dout2 = dout.reshape(M, d).contiguous()
        dz = torch.empty(M, d, dtype=BF16, device=dev)
        dfwd = torch.empty(M, d, dtype=BF16, device=dev)
        dretr = torch.zeros(B, d, dtype=F32, device=dev)
        dwn = torch.zeros(d, dtype=F32, device=dev)
        K.cam_blend_bwd(dout2, z, fwd2, retr, f32(wn), rstd, T, eps, dz, dfwd, dretr, dwn)
        g_W2 = _wgrad_bf16(dz, a, W2)
        g_b2 = _bias_grad(dz, b2)
        dpre = gemm_bf16(dz, W2, b_mn=True, aux=pre, aux_mode=AUX_MUL_SILU_GRAD)
        drb = torch.zeros(B, d, dtype=F32, device=dev)
        for b in range(B):
            K.colsum(dpre[b * T : (b + 1) * T], drb[b])
        dside = gemm_bf16(dpre, Ws, b_mn=True)
        gemm_bf16(dpre, Wf, b_mn=True, out=dfwd, aux=dfwd, aux_mode=AUX_ADD)
        dWs = gemm_bf16(dpre, side2, a_mn=True, b_mn=True, out_dtype=F32)
        dWf = gemm_bf16(dpre, fwd2, a_mn=True, b_mn=True, out_dtype=F32)
        return (dside.view(B, T, d), dfwd.view(B, T, d), dretr.to(retr_dtype), drb.to(rb_dtype), dWs.to(Ws.dtype),
                dWf.to(Wf.dtype), g_W2, g_b2, _sink_vec(wn, dwn), None)


def cam_readout_ok(fwd, W2) -> bool:
    B, T, d = fwd.shape
    return fwd.is_cuda and fwd.dtype == BF16 and W2.dtype == BF16 and d % 128 == 0 and T % 128 == 0 and d <= 6144


def cam_readout(side, fwd, retrieved, row_bias, Ws, Wf, W2, b2, wn, eps):
    return _CamReadoutFn.apply(side.to(BF16).contiguous(), fwd.contiguous(), retrieved, row_bias, Ws.to(BF16).contiguous(),
                               Wf.to(BF16).contiguous(), W2, b2, wn, float(eps))


def _fused_step_ok(fwd, side, layer, r) -> bool:
    d = fwd.shape[-1]
    M = fwd.shape[0] * fwd.shape[1]
    return (fwd.dtype == BF16 and d % 128 == 0 and M % 128 == 0 and getattr(layer, f"{r}_W1").weight.dtype == BF16)


def layer_step(fwd, side, layer, conv_name, g, r, sp_group=None, sp_slot=None, return_gate=False):
    """CUDA implementation of :func:`gdnet_b200.ops.functional.layer_step`."""
    from .fp8_linear import FP8Linear

    conv = getattr(layer, conv_name)
    k = conv.size
    w1r, w2r, nr = getattr(layer, f"{r}_W1"), getattr(layer, f"{r}_W2"), getattr(layer, f"{r}_norm")
    w1g, w2g, ng = getattr(layer, f"{g}_W1"), getattr(layer, f"{g}_W2"), getattr(layer, f"{g}_norm")
    halo = None
    sp = None
    zero_side = side is None
    if zero_side and not (return_gate is not True and zero_side_step_ok(fwd, layer, r)):
        side = torch.zeros_like(fwd)          # shapes the zero-side node does not cover: the general step on explicit zeros
        zero_side = False
    fused = return_gate is not True and _fused_step_ok(fwd, side, layer, r)
    if sp_group is not None and k > 1:
        import torch.distributed as dist

        B, T, d = fwd.shape
        in_kernel = (fused and k == 4 and T % 8 == 0 and dist.get_world_size(sp_group) > 1 and sp_slot is not None
                     and os.environ.get("GDNET_SP_TRANSPORT", "symm") == "symm" and os.environ.get("GDNET_SP_INKERNEL", "1") == "1")
        if in_kernel:
            sp = SpExchange(sp_group, int(sp_slot), B * (k - 1) * d * 2, fwd.device)
        else:
            from ..parallel.sp import halo_exchange

            halo = halo_exchange(ref.conv_tail(fwd, k).contiguous(), sp_group, sp_slot)

    if not fused:
        return _composed_step(fwd, side, halo, conv, w1r, w2r, nr, w1g, w2g, ng, return_gate)

    fp8 = isinstance(w1r, FP8Linear) and isinstance(w2r, FP8Linear) and w1r.recipe == "block"
    if zero_side:
        fo, so, gsum, nu8, nsu, npu = _LayerStepZeroSideFn.apply(
            fwd, halo, conv.taps, w1r.weight, w1g.weight, w1g.bias, ng.weight, w2g.weight, w2g.bias, fp8, ref.GATE_EPS,
            return_gate == "mean", sp)
        if fp8 and nu8 is not None:
            _offer_side_q8(so, (nu8, nsu, npu))
        if return_gate == "mean":
            return fo, so, gsum / float(fo.numel())
        return fo, so
    eps_r = nr.eps if nr.eps is not None else ref.default_rms_eps(BF16)
    side_q8 = _claim_side_q8(side) if fp8 and side.dtype == BF16 and side.is_contiguous() else None
    fo, so, gsum, nu8, nsu, npu = _LayerStepFn.apply(
        fwd, side.to(BF16), halo, conv.taps, w1r.weight, w1r.bias, w2r.weight, w2r.bias, nr.weight,
        w1g.weight, w1g.bias, ng.weight, w2g.weight, w2g.bias, fp8, float(eps_r), ref.GATE_EPS,
        return_gate == "mean", side_q8, sp,
    )
    if fp8 and nu8 is not None:
        _offer_side_q8(so, (nu8, nsu, npu))
    if return_gate == "mean":
        return fo, so, gsum / float(fo.numel())
    return fo, so


def _composed_step(fwd, side, halo, conv, w1r, w2r, nr, w1g, w2g, ng, return_gate):
    """The same step from single ops (used for shapes the fused node does not cover and when the
    caller wants the full gate tensor with gradients)."""
    import torch.nn.functional as F

    from .functional import _module_linear

    c = causal_dwconv(fwd, conv.taps, halo)
    s = side.to(c.dtype)
    z = _module_linear(w2r, F.silu(_module_linear(w1r, torch.cat([s, c], dim=-1))))
    eps_r = nr.eps if nr.eps is not None else ref.default_rms_eps(z.dtype)
    R = torch.sigmoid(ref.rmsnorm(z, nr.weight, eps_r).float())
    g_pre = ref.gate_pre(c, w1g.weight, w1g.bias, ng.weight, w2g.weight, w2g.bias)
    fo, so, gate = ref.gate_stream_update(g_pre, c, s, R)
    if return_gate == "mean":
        return fo, so, gate.mean()
    if return_gate:
        return fo, so, gate.to(c.dtype)
    return fo, so


# --------------------------------------------------------------------------------------
# spectral estimates: sigma_i = ||W_i v_i|| for all matrices in one launch
# --------------------------------------------------------------------------------------
def _ptr_table(tensors, device):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=device)


class _SigmaPlan:
    """Everything about a set of matrices that does not change between calls: the pointer tables of the
    batched kernels and persistent buffers for the probe vectors and the products ``y_i = W_i v_i``."""

    def __init__(self, mats):
        dev = mats[0].device
        self.n = len(mats)
        self.rows = [W.shape[0] for W in mats]
        self.cols = [W.shape[1] for W in mats]
        self.v_flat = torch.empty(sum(self.cols), dtype=F32, device=dev)
        self.y_flat = torch.empty(sum(self.rows), dtype=F32, device=dev)
        self.v_views, self.y_views, o = [], [], 0
        for c in self.cols:
            self.v_views.append(self.v_flat[o : o + c])
            o += c
        o = 0
        for r in self.rows:
            self.y_views.append(self.y_flat[o : o + r])
            o += r
        i64, i32 = torch.int64, torch.int32
        self.t_mats = torch.tensor([W.data_ptr() for W in mats], dtype=i64, device=dev)
        self.t_v = torch.tensor([v.data_ptr() for v in self.v_views], dtype=i64, device=dev)
        self.t_y = torch.tensor([y.data_ptr() for y in self.y_views], dtype=i64, device=dev)
        self.t_rows = torch.tensor(self.rows, dtype=i32, device=dev)
        self.t_cols = torch.tensor(self.cols, dtype=i32, device=dev)
        self.t_bf16 = torch.tensor([int(W.dtype == BF16) for W in mats], dtype=i32, device=dev)
        self.max_rows = max(self.rows)
        self.same_rows = len(set(self.rows)) == 1
        self.same_cols = len(set(self.cols)) == 1
        self.sources = list(mats)           # pins the storages the pointer table refers to
        self.mg_tables: dict = {}

    def mg_table(self, mgs):
        key = tuple(m.data_ptr() for m in mgs)
        t = self.mg_tables.get(key)
        if t is None:
            t = torch.tensor(key, dtype=torch.int64, device=self.v_flat.device)
            self.mg_tables[key] = t
        return t


_sigma_plans: dict = {}


def _sigma_plan(mats) -> _SigmaPlan:
    key = tuple((W.data_ptr(), W.shape[0], W.shape[1], W.dtype) for W in mats)
    plan = _sigma_plans.get(key)
    if plan is None:
        plan = _SigmaPlan(mats)
        _sigma_plans[key] = plan
    return plan


class _SigmaFn(torch.autograd.Function):
    """``sigma_i = ||W_i v_i||`` (fp32) for all matrices in one matrix-vector launch. Backward:
    ``dW_i = dsigma_i * (W_i v_i) v_i^T / sigma_i``, all rank-1 updates in one launch when the training engine
    has installed fp32 gradient buffers. The probe vectors were written into the plan's buffer by the caller."""

    @staticmethod
    def forward(ctx, plan, *mats):
        K.batched_gemv(plan.t_mats, plan.t_v, plan.t_y, plan.t_rows, plan.t_cols, plan.t_bf16, plan.max_rows)
        if plan.same_rows:
            sig = plan.y_flat.view(plan.n, plan.rows[0]).norm(dim=1)
        else:
            sig = torch.stack([y.norm() for y in plan.y_views])
        ctx.plan = plan
        ctx.mats = mats
        # the buffers are reused by the next call: keep this call's values for backward
        ctx.save_for_backward(sig, plan.y_flat.clone(), plan.v_flat.clone())
        return sig

    @staticmethod
    def backward(ctx, dsig):
        plan, mats = ctx.plan, ctx.mats
        sig, y_flat, v_flat = ctx.saved_tensors
        coef = (dsig / sig.clamp(min=1e-12)).to(F32).contiguous()
        mgs = [_main_grad(W) for W in mats]
        if all(m is not None and not isinstance(m, GradRef) and m.dtype == F32 and m.is_contiguous() for m in mgs) \
                and not _is_spread(mgs[0]):
            # rebuild the y / v pointer tables for the saved copies (same layout, different base)
            dy = y_flat.data_ptr() - plan.y_flat.data_ptr()
            dv = v_flat.data_ptr() - plan.v_flat.data_ptr()
            K.batched_outer_add(plan.mg_table(mgs), plan.t_y + dy, plan.t_v + dv, coef, plan.t_rows, plan.t_cols,
                                plan.max_rows)
            return (None, *([None] * len(mats)))
        grads, oy, ov = [], 0, 0
        for i, W in enumerate(mats):
            y, v = y_flat[oy : oy + plan.rows[i]], v_flat[ov : ov + plan.cols[i]]
            oy, ov = oy + plan.rows[i], ov + plan.cols[i]
            g = torch.outer(y * coef[i], v)
            if mgs[i] is not None:
                accumulate_main_grad(mgs[i], g)
                grads.append(None)
            else:
                grads.append(g.to(W.dtype))
        return (None, *grads)


def sigma_estimates(mats, vecs=None, generator=None):
    """``||W_i v_i||`` for unit vectors ``v_i`` (given, or drawn here: one normal draw for all matrices,
    normalised per matrix)."""
    ok = all(W.is_contiguous() and W.dtype in (BF16, F32) for W in mats)
    if not ok:
        if vecs is None:
            vecs = [torch.nn.functional.normalize(torch.randn(W.shape[1], device=W.device, generator=generator), dim=0)
                    for W in mats]
        return torch.stack([(W.float() @ v).norm() for W, v in zip(mats, vecs)])
    plan = _sigma_plan(mats)
    with torch.no_grad():
        if vecs is not None:
            torch.cat([v.reshape(-1).to(F32) for v in vecs], out=plan.v_flat)
        else:
            plan.v_flat.normal_(generator=generator)
            if plan.same_cols:
                v2 = plan.v_flat.view(plan.n, plan.cols[0])
                v2.div_(v2.norm(dim=1, keepdim=True))
            else:
                # two or more widths (d and 2d): normalise each width group in one go
                for c in sorted(set(plan.cols)):
                    idx = [i for i, cc in enumerate(plan.cols) if cc == c]
                    grp = torch.stack([plan.v_views[i] for i in idx])
                    grp = grp / grp.norm(dim=1, keepdim=True)
                    for j, i in enumerate(idx):
                        plan.v_views[i].copy_(grp[j])
    return _SigmaFn.apply(plan, *mats)


# --------------------------------------------------------------------------------------
# sequence-parallel halo exchange over symmetric memory (push + flag + bounded wait in-kernel)
# --------------------------------------------------------------------------------------
HALO_RING = 8          # passes that may be in flight before a slot is reused
HALO_SLOTS = 512       # exchanges per pass (2 * n_layers * n_cycles must not exceed this)
_halo_state: dict = {}


def _halo_ctx(group, nbytes, device):
    import torch.distributed as dist

    from ..parallel.symm import get_buffer

    key = id(group)
    st = _halo_state.get(key)
    slot_bytes = -(-nbytes // 256) * 256
    if st is None or st["slot_bytes"] < slot_bytes:
        total = 2 * HALO_RING * HALO_SLOTS
        data = get_buffer(("halo_data", slot_bytes), total * slot_bytes, group, device)
        flags = get_buffer(("halo_flags", slot_bytes), total * 4, group, device)
        st = {"slot_bytes": slot_bytes, "data": data, "flags": flags, "pass_fwd": {}, "rank": dist.get_rank(group),
              "world": dist.get_world_size(group),
              "counters": torch.zeros(total, dtype=torch.int32, device=device)}
        _halo_state[key] = st
    return st


class SpExchange:
    """One halo exchange done inside the conv kernels: the forward use of a slot and, when the step is
    differentiated, the gradient exchanges that answer it (up to two per forward use with a retained graph; each
    has its own sequence number and ring position, so a fast rank cannot overwrite a message that was not read)."""

    def __init__(self, group, slot, nbytes, device):
        if slot >= HALO_SLOTS:
            raise ValueError("halo exchange over symmetric memory needs a slot index below HALO_SLOTS")
        st = _halo_ctx(group, nbytes, device)
        self.st, self.slot = st, slot
        self.n_use = st["pass_fwd"].get(slot, 0) + 1        # counted identically on all ranks
        st["pass_fwd"][slot] = self.n_use
        self.bwd_runs = 0

    def _args(self, idx, seq):
        st = self.st
        return (st["data"].ptr_table, st["flags"].ptr_table, st["counters"][idx : idx + 1], idx * st["slot_bytes"], idx,
                st["rank"], st["world"], seq)

    def fwd_args(self):
        return self._args((self.n_use % HALO_RING) * HALO_SLOTS + self.slot, self.n_use)

    def bwd_args(self):
        self.bwd_runs += 1
        seq = self.n_use * 2 + min(self.bwd_runs, 2) - 1
        return self._args(HALO_RING * HALO_SLOTS + (seq % HALO_RING) * HALO_SLOTS + self.slot, seq)


class _HaloExchangeSymm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tail, group, slot):
        st = _halo_ctx(group, tail.numel() * tail.element_size(), tail.device)
        # sequence number of this slot: how many times it has been used, counted identically on all ranks
        n_use = st["pass_fwd"].get(slot, 0) + 1
        st["pass_fwd"][slot] = n_use
        ring = n_use % HALO_RING
        idx = ring * HALO_SLOTS + slot
        halo = torch.empty_like(tail)
        K.halo_push_wait(tail.contiguous(), halo, st["data"].ptr_table, st["flags"].ptr_table,
                         idx * st["slot_bytes"], idx, st["rank"], st["world"], n_use, False)
        ctx.group, ctx.slot, ctx.n_use = group, slot, n_use
        return halo

    @staticmethod
    def backward(ctx, d_halo):
        st = _halo_state[id(ctx.group)]
        # the backward of use n of a slot gets its own sequence number in the second half of the area
        key = ("b", ctx.slot, ctx.n_use)
        cnt = st["pass_fwd"].get(key, 0) + 1
        if cnt >= 2:
            st["pass_fwd"].pop(key, None)      # a forward use is differentiated at most twice: drop its counter
        else:
            st["pass_fwd"][key] = cnt
            for old in [k for k in st["pass_fwd"] if isinstance(k, tuple) and k[1] == ctx.slot and k[2] < ctx.n_use - HALO_RING]:
                del st["pass_fwd"][old]        # counters of uses that were differentiated only once
        # a retained graph runs this backward up to twice per forward use; every run has its own
        # sequence number and ring position, so a fast rank cannot overwrite an unread message
        seq = ctx.n_use * 2 + min(cnt, 2) - 1
        idx = HALO_RING * HALO_SLOTS + (seq % HALO_RING) * HALO_SLOTS + ctx.slot
        d_tail = torch.empty_like(d_halo)
        K.halo_push_wait(d_halo.contiguous(), d_tail, st["data"].ptr_table, st["flags"].ptr_table,
                         idx * st["slot_bytes"], idx, st["rank"], st["world"], seq, True)
        return d_tail, None, None


def halo_exchange(tail, group, slot):
    if slot is None or slot >= HALO_SLOTS:
        raise ValueError("halo exchange over symmetric memory needs a slot index below HALO_SLOTS")
    return _HaloExchangeSymm.apply(tail, group, int(slot))
