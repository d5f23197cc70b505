"""B200 training engine: flat buffers, fused projection + AdamW, fused gradient collective.

The engine owns, per parameter dtype (bf16 matrices, fp32 vectors):

* one flat parameter buffer (every ``nn.Parameter`` becomes a view into it),
* two flat fp32 gradient buffers, ``g_task`` and ``g_info``; during a backward pass each
  parameter carries ``main_grad`` = its view of the active buffer, and the weight-gradient
  GEMM epilogues accumulate straight into it (gradients that autograd delivers through
  ``.grad`` are folded in after the pass),
* fp32 AdamW moments for the slice of the flat buffer this rank updates.

One step = one forward, two backward passes (task; info + transition), then

* 1 GPU: ``grad_dots`` + ``projected_adamw`` (two kernels per dtype group);
* N GPUs, ``comm="fused"``: every rank reduces its shard of both gradient buffers by reading
  the peers' buffers over NVLink, applies projection + AdamW to that shard and writes the new
  parameters into every rank's parameter buffer, all in one kernel (``csrc/comm.cu``); the
  buffers live in symmetric memory;
* N GPUs, ``comm="scatter"``: the reduce-scatter happens *during* backward, tile by tile: the flat
  gradient buffers are spread over the ranks, and every weight-gradient GEMM epilogue (and every
  small-parameter gradient) adds its values with vector atomics over NVLink straight into the shard
  of the owning rank (``csrc/gemm_sm100.cu:epilogue_chunk``, ``csrc/comm.cu:peer_add_kernel``). After
  backward each rank holds the sum over ranks of its shard; the update kernel then only does the
  barrier, projection + AdamW on the shard and the parameter all-gather. The projection coefficient
  in this mode is computed from the reduced gradients (no rank ever holds its full local gradient);
* N GPUs, ``comm="nccl"``: NCCL all-reduce of the flat gradients, then the 1-GPU update.

The projection coefficient uses the sum over ranks of the *local* dot products, exactly as
the reference does (gdnet/loss.py:228-235), and the reduced gradient is the mean over ranks
(gdnet/loss.py:241-251).
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as ops
from ..utils.fp8 import autocast as make_autocast
from .step import build_cam_buffer, info_losses, unwrap

ALIGN = 128  # elements; keeps every parameter view 256-byte aligned in bf16


class _Group:
    """All parameters of one dtype, flattened; every rank holds all of them."""

    sharded = False

    def __init__(self, params, dtype, device, world, rank, symmetric, pg):
        self.params, self.dtype = params, dtype
        offs, n = [], 0
        for p in params:
            offs.append(n)
            n += -(-p.numel() // ALIGN) * ALIGN
        per = -(-n // world)
        per = -(-per // ALIGN) * ALIGN
        self.n = per * world            # padded so every rank's shard has the same length
        self.offsets = offs
        self.per = per
        self.shard = (rank * per, (rank + 1) * per)
        item = 2 if dtype == torch.bfloat16 else 4
        if symmetric:
            from ..parallel.symm import SymmBuffer

            self._sp = SymmBuffer(self.n * item, pg, device)
            self._sgt = SymmBuffer(self.n * 4, pg, device)
            self._sgi = SymmBuffer(self.n * 4, pg, device)
            self.flat = self._sp.view(dtype, self.n)
            self.g_task = self._sgt.view(torch.float32, self.n)
            self.g_info = self._sgi.view(torch.float32, self.n)
        else:
            self.flat = torch.zeros(self.n, dtype=dtype, device=device)
            self.g_task = torch.zeros(self.n, dtype=torch.float32, device=device)
            self.g_info = torch.zeros(self.n, dtype=torch.float32, device=device)
        with torch.no_grad():
            for p, o in zip(params, offs):
                view = self.flat[o : o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
        m_len = per if symmetric else self.n   # fused mode updates only this rank's shard
        self.m = torch.zeros(m_len, dtype=torch.float32, device=device)
        self.v = torch.zeros(m_len, dtype=torch.float32, device=device)
        self.sums = torch.zeros(8, dtype=torch.float32, device=device)
        # NVLink multicast addresses of the three buffers: the update kernel then reduces inside the switch and
        # broadcasts with one store. Used from four ranks on (on two ranks the peer loads measured faster: 2.9 against
        # 4.9 ms for 350 M parameters); GDNET_MULTIMEM=1 / 0 forces it on / off; 0 where the switch gives no address.
        self.mc = (0, 0, 0)
        if symmetric:
            self.tab_p, self.tab_gt, self.tab_gi = self._sp.ptr_table, self._sgt.ptr_table, self._sgi.ptr_table
            mc = (self._sgt.multicast_ptr, self._sgi.multicast_ptr, self._sp.multicast_ptr)
            want = os.environ.get("GDNET_MULTIMEM", "1" if world >= 4 else "0")
            if all(mc) and want != "0":
                self.mc = mc
        self.p_range = (0, self.n)                                   # flat range of the parameters held locally
        self.mv_range = self.shard if symmetric else (0, self.n)     # flat range the moments cover

    def views(self, flat):
        return [flat[o : o + p.numel()].view(p.shape) for p, o in zip(self.params, self.offsets)]


class _ShardedGroup:
    """Large bf16 matrices spread over the ranks, whole matrices, balanced by size: a rank holds the bf16 masters,
    the two fp32 gradient buffers and the AdamW moments of the matrices it owns and nothing of the others.

    The flat index space is ``world`` segments of ``per`` elements, segment ``r`` holding rank ``r``'s matrices back
    to back, so everything that works on "this rank's shard of the flat range" (the update kernel, the gradient
    sinks of the weight-gradient epilogues) applies unchanged. The pointer tables handed to the kernels hold every
    rank's shard base *minus* that rank's segment offset: ``table[idx / per] + idx`` is element ``idx``.
    A parameter this rank does not own becomes a one-element placeholder of the right shape (stride 0); its
    gradient handle is a :class:`gdnet_b200.ops.cuda.GradRef`."""

    sharded = True

    def __init__(self, params, device, world, rank, pg, broadcast_src=None):
        from ..ops import cuda as cu
        from ..parallel.symm import SymmBuffer

        self.params, self.dtype = params, torch.bfloat16
        sizes = [-(-p.numel() // ALIGN) * ALIGN for p in params]
        load = [0] * world
        owner = [0] * len(params)
        for i in sorted(range(len(params)), key=lambda i: (-sizes[i], i)):      # largest first, to the lightest rank
            r = min(range(world), key=lambda r: (load[r], r))
            owner[i] = r
            load[r] += sizes[i]
        per = -(-max(max(load), ALIGN) // ALIGN) * ALIGN
        fill = [0] * world
        offs = []
        for i in range(len(params)):
            offs.append(owner[i] * per + fill[owner[i]])
            fill[owner[i]] += sizes[i]
        self.owner, self.offsets, self.per, self.n = owner, offs, per, per * world
        self.shard = (rank * per, (rank + 1) * per)
        self.index = {id(p): (o, f) for p, o, f in zip(params, owner, offs)}
        self._sp = SymmBuffer(per * 2, pg, device)
        self._sgt = SymmBuffer(per * 4, pg, device)
        self._sgi = SymmBuffer(per * 4, pg, device)
        self.flat = self._sp.view(torch.bfloat16, per)            # this rank's shard only
        self.g_task = self._sgt.view(torch.float32, per)
        self.g_info = self._sgi.view(torch.float32, per)

        def biased(buf, item):
            return torch.tensor([p - r * per * item for r, p in enumerate(buf.ptrs)], dtype=torch.int64, device=device)

        self.tab_p, self.tab_gt, self.tab_gi = biased(self._sp, 2), biased(self._sgt, 4), biased(self._sgi, 4)
        self.sink_task = int(cu.K.register_virtual_grad_sink(self.tab_gt, self.n, per))
        self.sink_info = int(cu.K.register_virtual_grad_sink(self.tab_gi, self.n, per))
        with torch.no_grad():
            for p, o, f in zip(params, owner, offs):
                if broadcast_src is not None:
                    dist.broadcast(p.data, src=broadcast_src, group=pg)
                if o == rank:
                    view = self.flat[f - rank * per : f - rank * per + p.numel()].view(p.shape)
                    view.copy_(p.data)
                    p.data = view
                else:
                    p.data = torch.zeros(1, dtype=p.dtype, device=device).expand(p.shape)
                p._gd_owner, p._gd_world, p._gd_rank = o, world, rank
        self.m = torch.zeros(per, dtype=torch.float32, device=device)
        self.v = torch.zeros(per, dtype=torch.float32, device=device)
        self.sums = torch.zeros(8, dtype=torch.float32, device=device)
        self.mc = (0, 0, 0)              # nothing to reduce or broadcast: the producers add into the owner's shard
        self.p_range = self.shard
        self.mv_range = self.shard

    def grad_refs(self, which: str):
        from ..ops.cuda import GradRef

        sink = self.sink_task if which == "task" else self.sink_info
        return [GradRef(sink, f, p.shape[0], p.shape[1]) for p, f in zip(self.params, self.offsets)]


class TrainEngine(nn.Module):
    """Wraps a GDNet for training on CUDA. ``engine(tokens, ...)`` forwards to the model;
    ``engine.projected_step(...)`` (or ``gdnet_b200.loss.projected_step(engine, ...)``) runs a step."""

    is_gdnet_engine = True

    def __init__(self, model: nn.Module, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2, precision: str = "fp8", process_group=None, sp_group=None,
                 comm: str = "fused", broadcast: bool = True, projection: str = "local",
                 share_fp8_weights: bool = False, fused_ce: bool = True, shard: str = "none",
                 overlap_task_reduce: bool = True):
        super().__init__()
        self.module = model
        self.precision = precision
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.sp_group = sp_group
        # "local": coefficient from the sum over ranks of per-rank dot products (gdnet/loss.py:228-235);
        # "global": from the dot products of the reduced gradients (the only choice for comm="scatter")
        if projection not in ("local", "global"):
            raise ValueError(f"unknown projection {projection!r}")
        self.projection = projection
        self.step_count = 0
        self.comm_seq = 0
        # project to the vocabulary and take the loss chunk by chunk, never holding all logits
        self.fused_ce = bool(fused_ce)
        self.time_updates = False
        self._update_events: list = []
        dev = next(model.parameters()).device
        self.device = dev
        self.distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(process_group) > 1
        self.pg = process_group if process_group is not None else (dist.group.WORLD if self.distributed else None)
        self.world = dist.get_world_size(self.pg) if self.distributed else 1
        self.rank = dist.get_rank(self.pg) if self.distributed else 0
        self.comm = comm if self.distributed else "local"
        if self.comm not in ("fused", "scatter", "nccl", "local"):
            raise ValueError(f"unknown comm backend {comm!r}")
        if shard not in ("none", "full"):
            raise ValueError(f"unknown shard mode {shard!r}")
        # "full": the large layer matrices live on one owner rank each (masters, gradients, moments); the GEMMs
        # gather the operands they need from the owners (parallel/weight_stream.py). A single GPU has nothing to shard.
        self.shard = shard if self.distributed else "none"
        if self.shard == "full":
            if dev.type != "cuda" or precision != "fp8":
                raise ValueError('shard="full" needs CUDA and precision="fp8"')
            self.comm = "scatter"           # gradients go to their owner from the weight-gradient epilogues
        symmetric = self.comm in ("fused", "scatter")
        self._sink_ids: list[int] = []
        self._shared = None

        params = [p for p in model.parameters() if p.requires_grad]
        sharded_params = self._layer_matrices(model) if self.shard == "full" else []
        taken = {id(p) for p in sharded_params}
        by_dtype: dict[torch.dtype, list] = {}
        for p in params:
            if id(p) not in taken:
                by_dtype.setdefault(p.dtype, []).append(p)
        for dt in by_dtype:
            if dt not in (torch.bfloat16, torch.float32):
                raise TypeError(f"unsupported parameter dtype {dt}")
        src0 = dist.get_global_rank(self.pg, 0) if self.distributed else None
        self.groups = [
            _Group(ps, dt, dev, self.world, self.rank, symmetric, self.pg) for dt, ps in by_dtype.items()
        ]
        if sharded_params:
            self.groups.append(_ShardedGroup(sharded_params, dev, self.world, self.rank, self.pg,
                                             broadcast_src=src0 if broadcast else None))
        self.params = params
        if self.distributed and broadcast:
            for g in self.groups:
                if not g.sharded:
                    dist.broadcast(g.flat, src=src0, group=self.pg)
            for b in model.buffers():
                dist.broadcast(b, src=src0, group=self.pg)
        if symmetric:
            from ..parallel.symm import SymmBuffer

            self._flags = SymmBuffer(4096, self.pg, dev)
            for g in self.groups:
                g._sp.barrier()
        if self.comm == "scatter":
            from ..ops import cuda as cu

            for g in self.groups:
                if g.sharded:
                    self._sink_ids += [g.sink_task, g.sink_info]
                else:
                    self._sink_ids.append(int(cu.K.register_grad_sink(g.g_task, g._sgt.ptr_table, g.per)))
                    self._sink_ids.append(int(cu.K.register_grad_sink(g.g_info, g._sgi.ptr_table, g.per)))
        self.scalars = torch.zeros(2, dtype=torch.float32, device=dev)
        # comm="fused": the task gradient is complete after the first backward pass, so its reduce-scatter runs on a
        # side stream while the second pass computes the information gradient; the update kernel then pulls only the
        # information gradient from the peers
        self.overlap_task_reduce = bool(overlap_task_reduce) and self.comm == "fused"
        self.task_seq = 0
        self._task_event = None
        if self.overlap_task_reduce:
            self._side_stream = torch.cuda.Stream(device=dev)
            for g in self.groups:
                g.t_red = torch.zeros(g.per, dtype=torch.float32, device=dev)
        self._timing = torch.zeros(4, dtype=torch.int64, device=dev) if dev.type == "cuda" else None
        if dev.type == "cuda":
            from ..ops import cuda as cu

            cu.clear_caches()     # cached copies made from the pre-flattening parameter storages
            if share_fp8_weights and symmetric and precision == "fp8":
                # each FP8 weight is quantised by one rank per update and stored into every rank's cache by
                # that rank's quantisation kernel (the all-gather of the e4m3 weights, inside the producer)
                from ..ops.fp8_linear import FP8Linear

                ws = [m.weight for m in model.modules() if isinstance(m, FP8Linear) and m.recipe == "block"
                      and m.weight.dtype == torch.bfloat16 and m.weight.shape[0] % 128 == 0 and m.weight.shape[1] % 128 == 0]
                seen, uniq = set(), []
                for w in ws:
                    if w.data_ptr() not in seen:
                        seen.add(w.data_ptr())
                        uniq.append(w)
                if uniq:
                    self._shared = cu.share_fp8_weights(uniq, self.pg, dev)
            self.weight_stream = None
            if self.shard == "full":
                from ..parallel.weight_stream import LayerSet, WeightStream

                sets = []
                for layer in model.layers:
                    for g_, r_ in (("gf", "rf"), ("gb", "rb")):
                        sets.append(LayerSet(getattr(layer, f"{r_}_W1").weight, getattr(layer, f"{r_}_W2").weight,
                                             getattr(layer, f"{g_}_W1").weight, getattr(layer, f"{g_}_W2").weight,
                                             getattr(layer, f"{g_}_norm").weight))
                self.weight_stream = WeightStream(self.pg, dev, self.groups[-1], sets)
                cu.add_weight_stream(self.weight_stream)

    def close(self) -> None:
        """Take this engine's registrations out of the op layer (gradient sinks spread over the ranks, the shared FP8
        cache, the weight stream). Collective in the sense that every rank should close at the same point; the
        engine must not step afterwards."""
        if self.device.type != "cuda":
            return
        from ..ops import cuda as cu

        for sid in self._sink_ids:
            cu.K.unregister_grad_sink(sid)
        self._sink_ids = []
        for obj in (self._shared, getattr(self, "weight_stream", None)):
            if obj is not None:
                cu.remove_provider(obj)
        self._shared = None
        self.weight_stream = None

    @staticmethod
    def _layer_matrices(model):
        """The parameters that ``shard="full"`` spreads over the ranks: the eight large matrices of every GDLayer."""
        out = []
        for layer in getattr(model, "layers", []):
            for prefix in ("gf", "gb", "rf", "rb"):
                for which in ("W1", "W2"):
                    w = getattr(layer, f"{prefix}_{which}").weight
                    if w.dtype != torch.bfloat16 or w.dim() != 2 or w.shape[0] % 128 or w.shape[1] % 128:
                        raise ValueError('shard="full" needs bf16 layer matrices with dimensions that are multiples of 128')
                    out.append(w)
        return out

    def full_state_dict(self) -> dict:
        """The model's ``state_dict`` with every parameter complete on every rank. Collective when matrices are
        sharded (each is broadcast by its owner); otherwise the plain ``state_dict``."""
        base = unwrap(self.module)
        sd = base.state_dict()
        names = {id(p): n for n, p in base.named_parameters()}
        for g in self.groups:
            if not g.sharded:
                continue
            for p, o in zip(g.params, g.owner):
                t = p.data.clone() if o == self.rank else torch.empty(p.shape, dtype=p.dtype, device=self.device)
                dist.broadcast(t, src=dist.get_global_rank(self.pg, o), group=self.pg)
                sd[names[id(p)]] = t
        return sd

    def resident_bytes(self) -> dict:
        """Bytes of parameters, gradients and optimizer state this rank holds (for reports and tests)."""
        out = {"params": 0, "grads": 0, "optimizer": 0}
        for g in self.groups:
            out["params"] += g.flat.numel() * g.flat.element_size()
            out["grads"] += (g.g_task.numel() + g.g_info.numel()) * 4
            out["optimizer"] += (g.m.numel() + g.v.numel()) * 4
        return out

    # -- nn.Module plumbing -----------------------------------------------------------------
    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    def parameters_flat(self):
        return [g.flat for g in self.groups]

    # -- gradient buffers -------------------------------------------------------------------
    def _point_main_grad(self, which: str) -> None:
        for g in self.groups:
            handles = g.grad_refs(which) if g.sharded else g.views(g.g_task if which == "task" else g.g_info)
            for p, v in zip(g.params, handles):
                p.main_grad = v

    def _fold_autograd_grads(self) -> None:
        for p in self.params:
            if p.grad is not None:
                if self.comm == "scatter":
                    from ..ops import cuda as cu

                    cu.accumulate_main_grad(p.main_grad, p.grad)
                else:
                    p.main_grad.add_(p.grad)
                p.grad = None

    # -- the step ---------------------------------------------------------------------------
    def projected_step(self, tokens, targets, beta: float = 0.1, write_chunks=None, grad_clip: float = 0.0,
                       accum_steps: int = 1, loss_mask=None):
        """One optimizer step. Returns the task loss as a 0-dim device tensor (no host sync)."""
        model = self.module
        base = unwrap(model)
        B = tokens.shape[0]
        if B % accum_steps:
            raise ValueError(f"batch size {B} not divisible by accum_steps {accum_steps}")
        mb = B // accum_steps
        for g in self.groups:
            if self.comm != "scatter":   # spread buffers are cleared by the update kernel that consumed them
                g.g_task.zero_()
                g.g_info.zero_()
            g.sums.zero_()
        total = torch.zeros((), dtype=torch.float32, device=tokens.device)
        dev_type = tokens.device.type

        for i in range(accum_steps):
            sl = slice(i * mb, (i + 1) * mb)
            tok_i, tgt_i = tokens[sl], targets[sl]
            with make_autocast(self.precision, dev_type):
                tags = vals = None
                if write_chunks is not None and base.cam_enabled:
                    tags, vals = build_cam_buffer(model, write_chunks[sl], sp_group=self.sp_group)
                logits, side, _, _, gate_vals, _, _ = model(tok_i, tags, vals, return_gates="mean",
                                                            sp_group=self.sp_group,
                                                            need_logits="features" if self.fused_ce else True)
                tgt = tgt_i.reshape(-1)
                if loss_mask is not None:
                    tgt = torch.where(loss_mask[sl].reshape(-1), tgt, torch.full_like(tgt, -100))
                if self.fused_ce:
                    loss_task = ops.linear_cross_entropy(logits, base.head, tgt, base.vocab_size) / accum_steps
                else:
                    loss_task = ops.cross_entropy(logits.reshape(-1, logits.shape[-1]), tgt) / accum_steps
            self._point_main_grad("task")
            loss_task.backward(retain_graph=True)
            self._fold_autograd_grads()
            if self.overlap_task_reduce and i == accum_steps - 1:
                self._start_task_reduce()
            with make_autocast(self.precision, dev_type):
                loss_info = info_losses(base, side, gate_vals, accum_steps)
            self._point_main_grad("info")
            loss_info.backward()
            self._fold_autograd_grads()
            total += loss_task.detach().float()

        timed = self.time_updates and self.device.type == "cuda"
        if timed:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        self._update(beta, grad_clip)
        if timed:
            ev1.record()
            self._update_events.append((ev0, ev1))
        from ..ops import cuda as cu

        cu.invalidate_param_caches()
        if self._shared is not None:
            cu.refresh_shared_weights(self._shared)     # collective, here where every rank is at the same point of the step
        if getattr(self, "weight_stream", None) is not None:
            self.weight_stream.refresh()    # owners re-derive the GEMM operands of their matrices (collective)
            self.weight_stream.end_step()
        return total

    def _start_task_reduce(self) -> None:
        """Reduce-scatter of the (final) task gradient on the side stream, beside the second backward pass."""
        from ..ops import cuda as cu

        done = torch.cuda.Event()
        done.record()
        self.task_seq += 1
        with torch.cuda.stream(self._side_stream):
            self._side_stream.wait_event(done)
            for gi, g in enumerate(self.groups):
                cu.K.allreduce_adamw(g.tab_gt, g.tab_gi, g.tab_p, self._flags.ptr_table, g.m, g.v, self.scalars, g.n,
                                     self.rank, self.world, self.task_seq * 8 + gi, 6, g.dtype == torch.bfloat16,
                                     0.0, 0.0, 0.9, 0.9, 1e-8, 0.0, 1, g.sums, True, g.t_red, None, g.mc[0], 0, 0)
            self._task_event = torch.cuda.Event()
            self._task_event.record()

    def update_breakdown_ms(self) -> dict | None:
        """Of the last update kernel of the largest group (``time_updates`` on, several GPUs): time spent waiting for
        the other ranks at the opening barrier, moving and updating the shard, and in the closing barrier."""
        if self._timing is None or self.comm not in ("fused", "scatter"):
            return None
        t = self._timing.tolist()
        if not all(t):
            return None
        return {"wait_ms": (t[1] - t[0]) / 1e6, "transfer_update_ms": (t[2] - t[1]) / 1e6, "close_ms": (t[3] - t[2]) / 1e6}

    def update_times_ms(self) -> list[float]:
        """Device time of the update phase (gradient collective + projection + AdamW + parameter all-gather,
        including any wait for slower ranks) of every step since the last call; needs ``time_updates=True``."""
        torch.cuda.synchronize(self.device)
        out = [a.elapsed_time(b) for a, b in self._update_events]
        self._update_events.clear()
        return out

    def _update(self, beta: float, grad_clip: float) -> None:
        from ..ops import cuda as cu

        self.step_count += 1
        K = cu.K
        if self.comm == "scatter":
            return self._update_scattered(beta, grad_clip)
        glob = self.projection == "global" and self.distributed
        b1, b2 = self.betas
        common = (beta, self.lr, b1, b2, self.eps, self.weight_decay, self.step_count)
        self.scalars[1] = 1.0

        def dots():
            sums = torch.zeros(4, dtype=torch.float32, device=self.device)
            for g in self.groups:
                K.grad_dots(g.g_task, g.g_info, sums)
            return sums

        coef = None
        if not glob:
            # sum over ranks of the local dot products <gt,gt>, <gi,gt>
            sums = dots()
            if self.distributed:
                dist.all_reduce(sums, group=self.pg)
            coef = sums[1] / sums[0].clamp(min=1e-8)
        if self.comm == "nccl":
            for g in self.groups:
                dist.all_reduce(g.g_task, group=self.pg)
                dist.all_reduce(g.g_info, group=self.pg)
            self.scalars[1] = 1.0 / self.world
            if glob:
                sums = dots()       # of the reduced gradients; the ratio does not depend on their scale
                coef = sums[1] / sums[0].clamp(min=1e-8)
        if coef is not None:
            self.scalars[0] = coef

        if self.comm in ("local", "nccl"):
            if grad_clip > 0.0:
                red = torch.zeros(4, dtype=torch.float32, device=self.device)
                for g in self.groups:
                    K.grad_dots(g.g_task, g.g_info, red)
                self.scalars[1] = self.scalars[1] * self._clip_factor(red * self.scalars[1] ** 2, coef, beta, grad_clip)
            for g in self.groups:
                K.projected_adamw(g.flat, g.g_task, g.g_info, g.m, g.v, self.scalars, *common)
            return

        # fused: reduce-scatter + projection + AdamW + all-gather over peer memory
        self.comm_seq += 1
        t_reds = [None] * len(self.groups)
        if self._task_event is not None:        # the task gradient's shard was reduced beside the second backward pass
            torch.cuda.current_stream().wait_event(self._task_event)
            self._task_event = None
            t_reds = [g.t_red for g in self.groups]
        big = max(range(len(self.groups)), key=lambda i: self.groups[i].n)
        if self.time_updates:
            self._timing.zero_()
        phases = (0,) if grad_clip <= 0.0 and not glob else (1, 2)
        for phase in phases:
            if phase == 2:
                red = torch.zeros(4, dtype=torch.float32, device=self.device)
                for g in self.groups:
                    red[:3] += g.sums[:3]
                dist.all_reduce(red, group=self.pg)
                if glob:
                    coef = red[1] / red[0].clamp(min=1e-8)
                    self.scalars[0] = coef
                if grad_clip > 0.0:
                    self.scalars[1] = self._clip_factor(red, coef, beta, grad_clip)
            for gi, g in enumerate(self.groups):
                K.allreduce_adamw(g.tab_gt, g.tab_gi, g.tab_p, self._flags.ptr_table,
                                  g.m, g.v, self.scalars, g.n, self.rank, self.world,
                                  self.comm_seq * 8 + gi, phase, g.dtype == torch.bfloat16, *common, g.sums, True,
                                  t_reds[gi] if phase != 2 else None,
                                  self._timing if self.time_updates and gi == big and phase in (0, 2) else None, *g.mc)

    def _update_scattered(self, beta: float, grad_clip: float) -> None:
        """Gradients were reduce-scattered by the producers. Barrier + shard dot products, one tiny
        all-reduce for the projection coefficient (and the clip factor), then AdamW + all-gather."""
        from ..ops import cuda as cu

        K = cu.K
        b1, b2 = self.betas
        common = (beta, self.lr, b1, b2, self.eps, self.weight_decay, self.step_count)
        self.comm_seq += 1
        for phase in (3, 4):
            if phase == 4:
                red = torch.zeros(4, dtype=torch.float32, device=self.device)
                for g in self.groups:
                    red[:3] += g.sums[:3]
                dist.all_reduce(red, group=self.pg)
                coef = red[1] / red[0].clamp(min=1e-8)
                self.scalars[0] = coef
                self.scalars[1] = self._clip_factor(red, coef, beta, grad_clip) if grad_clip > 0.0 else 1.0
            for gi, g in enumerate(self.groups):
                K.allreduce_adamw(g.tab_gt, g.tab_gi, g.tab_p, self._flags.ptr_table,
                                  g.m, g.v, self.scalars, g.n, self.rank, self.world,
                                  self.comm_seq * 8 + gi, phase, g.dtype == torch.bfloat16, *common, g.sums,
                                  not g.sharded)

    @staticmethod
    def _clip_factor(red, coef, beta, grad_clip):
        """min(1, clip/||g||) for g = (1-beta*coef) gt + beta gi, from the three dot products."""
        kt = 1.0 - beta * coef
        norm2 = kt * kt * red[0] + 2.0 * kt * beta * red[1] + beta * beta * red[2]
        return (grad_clip / (norm2.clamp(min=0).sqrt() + 1e-6)).clamp(max=1.0)

    # -- optimizer-like helpers -------------------------------------------------------------
    def set_lr(self, lr: float) -> None:
        self.lr = float(lr)

    def state_dict_optim(self) -> dict:
        return {"step": self.step_count, "lr": self.lr, "world": self.world, "rank": self.rank,
                "m": [g.m.clone() for g in self.groups], "v": [g.v.clone() for g in self.groups]}

    def load_state_dict_optim(self, sd: dict) -> None:
        """Inverse of :meth:`state_dict_optim` for the same world size and sharding (the moments are this rank's
        own); anything else goes through ``runtime.ckpt.save_sharded`` / ``load_sharded``, which re-slice."""
        if len(sd["m"]) != len(self.groups):
            raise ValueError(f"optimizer state has {len(sd['m'])} groups, the engine {len(self.groups)}")
        if int(sd.get("world", self.world)) != self.world or int(sd.get("rank", self.rank)) != self.rank:
            raise ValueError(f"optimizer state of rank {sd.get('rank')} / world {sd.get('world')} cannot be loaded into "
                             f"rank {self.rank} / world {self.world}: use a sharded checkpoint")
        for g, m, v in zip(self.groups, sd["m"], sd["v"]):
            if m.numel() != g.m.numel() or v.numel() != g.v.numel():
                raise ValueError(f"optimizer moments have {m.numel()} elements, this rank holds {g.m.numel()}")
        self.step_count, self.lr = int(sd["step"]), float(sd["lr"])
        for g, m, v in zip(self.groups, sd["m"], sd["v"]):
            g.m.copy_(m)
            g.v.copy_(v)
