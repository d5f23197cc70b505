"""Device-timed microbenchmarks of the peer-memory collectives against their NCCL counterparts.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/bench_fused_collectives.py [--params 350e6] [--json out.json]

* gradient reduce-scatter + projection + AdamW + parameter all-gather in one kernel
  (``fused_reduce_adamw_kernel``) against NCCL all-reduce of both gradient buffers + the local AdamW kernel;
* the task gradient's reduce-scatter alone (the part that runs beside the second backward pass) and the update kernel
  that is left after backward (pulls the information gradient only);
* the parameter gather of the fully sharded engine: 32 MB pulled from a peer by gather jobs, stand-alone and carried by
  a tensor-core GEMM;
* halo push/flag/wait kernel against ``dist.batch_isend_irecv`` of the same message;
* one-shot MAX all-reduce of a small vector against ``dist.all_reduce(MAX)``.

Times are CUDA events on the launching stream, max over ranks. The roofline of the update kernel is the
slower direction of its NVLink traffic at 770 GB/s per direction: every rank pulls its shard of two fp32
buffers from N-1 peers and pushes its updated bf16 shard to N-1 peers.
"""

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn, iters, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=float, default=350e6)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from gdnet_b200.ops import cuda as cu
    from gdnet_b200.parallel.symm import SymmBuffer, max_allreduce_

    K = cu.K
    per = -(-int(args.params) // world)
    per = -(-per // 128) * 128
    n = per * world
    grp = dist.group.WORLD
    sp, sgt, sgi = SymmBuffer(n * 2, grp, dev), SymmBuffer(n * 4, grp, dev), SymmBuffer(n * 4, grp, dev)
    flags = SymmBuffer(4096, grp, dev)
    gt, gi = sgt.view(torch.float32, n), sgi.view(torch.float32, n)
    gt.normal_()
    gi.normal_()
    m, v = torch.zeros(per, device=dev), torch.zeros(per, device=dev)
    scalars = torch.tensor([0.1, 1.0], device=dev)
    sums = torch.zeros(8, device=dev)
    sp.barrier()
    seq = [0]

    def fused():
        seq[0] += 1
        K.allreduce_adamw(sgt.ptr_table, sgi.ptr_table, sp.ptr_table, flags.ptr_table, m, v, scalars, n, rank, world,
                          seq[0] * 8, 0, True, 0.1, 1e-3, 0.9, 0.999, 1e-8, 0.01, seq[0], sums)

    p_l = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    g1, g2 = torch.randn(n, device=dev), torch.randn(n, device=dev)
    m2, v2 = torch.zeros(n, device=dev), torch.zeros(n, device=dev)

    def nccl():
        dist.all_reduce(g1)
        dist.all_reduce(g2)
        K.projected_adamw(p_l, g1, g2, m2, v2, scalars, 0.1, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1)

    t_red = torch.zeros(per, device=dev)
    tseq = [0]

    def task_reduce():            # what runs beside the second backward pass
        tseq[0] += 1
        K.allreduce_adamw(sgt.ptr_table, sgi.ptr_table, sp.ptr_table, flags.ptr_table, m, v, scalars, n, rank, world,
                          tseq[0] * 8, 6, True, 0.0, 0.0, 0.9, 0.9, 1e-8, 0.0, 1, sums, True, t_red)

    def fused_info_only():        # what is left after backward: pulls the information gradient only
        seq[0] += 1
        K.allreduce_adamw(sgt.ptr_table, sgi.ptr_table, sp.ptr_table, flags.ptr_table, m, v, scalars, n, rank, world,
                          seq[0] * 8, 0, True, 0.1, 1e-3, 0.9, 0.999, 1e-8, 0.01, seq[0], sums, True, t_red)

    mc = (sgt.multicast_ptr, sgi.multicast_ptr, sp.multicast_ptr)

    def fused_multicast():        # the same kernel reading through the NVLink multicast address (in-switch sum, one-store broadcast)
        seq[0] += 1
        K.allreduce_adamw(sgt.ptr_table, sgi.ptr_table, sp.ptr_table, flags.ptr_table, m, v, scalars, n, rank, world,
                          seq[0] * 8, 0, True, 0.1, 1e-3, 0.9, 0.999, 1e-8, 0.01, seq[0], sums, True, None, None, *mc)

    res = {"world": world, "params": n}
    res["fused_update_ms"] = timed(fused, args.iters)
    if all(mc) and os.environ.get("GDNET_MULTIMEM", "1") != "0":
        res["fused_update_multicast_ms"] = timed(fused_multicast, args.iters)
        # the sum is formed in the switch, so a rank receives its reduced shard only once; but every rank still has to
        # send the other ranks' shards of its two fp32 buffers: the outbound side sets the same bound as the peer loads
        res["multicast_roofline_ms"] = (world - 1) * per * 8 / 770e9 * 1e3
    res["task_reduce_side_stream_ms"] = timed(task_reduce, args.iters)
    res["fused_update_info_only_ms"] = timed(fused_info_only, args.iters)
    res["info_only_roofline_ms"] = max((world - 1) * per * 4, (world - 1) * per * 2) / 770e9 * 1e3
    res["nccl_allreduce_plus_adamw_ms"] = timed(nccl, args.iters)
    link = 770e9
    pulled, pushed = (world - 1) * per * 8, (world - 1) * per * 2      # bytes in / out per rank
    nvlink_bytes = pulled + pushed
    res["fused_nvlink_bytes_per_rank"] = nvlink_bytes
    res["fused_roofline_ms"] = max(pulled, pushed) / link * 1e3
    res["fused_fraction_of_nvlink_roofline"] = res["fused_roofline_ms"] / res["fused_update_ms"] if world > 1 else None

    # halo exchange: (B, k-1, d) bf16 messages, as in the 1.3B sequence-parallel config
    tail = torch.randn(1, 3, 2048, device=dev, dtype=torch.bfloat16)
    slot = [0]

    def halo_kernel():
        slot[0] = (slot[0] + 1) % cu.HALO_SLOTS
        cu.halo_exchange(tail, dist.group.WORLD, slot[0])

    def halo_nccl():
        ops, recv = [], torch.empty_like(tail)
        if rank + 1 < world:
            ops.append(dist.P2POp(dist.isend, tail, rank + 1))
        if rank > 0:
            ops.append(dist.P2POp(dist.irecv, recv, rank - 1))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    with torch.no_grad():
        res["halo_kernel_us"] = timed(halo_kernel, 50) * 1e3
        res["halo_nccl_sendrecv_us"] = timed(halo_nccl, 50) * 1e3

    # parameter gather of the fully sharded engine: 64 KB jobs pulling from the next rank's memory into local
    # staging, stand-alone and carried by a tensor-core GEMM (8192 x 2048 x 2048 bf16, about 45 us of math)
    nbytes = 32 * 1024 * 1024
    src_buf = SymmBuffer(nbytes, grp, dev)
    src_buf.local.random_(0, 255)
    src_buf.barrier()
    dst = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    peer = (rank + 1) % world
    rows = [[src_buf.ptrs[peer] + o, dst.data_ptr() + o, 0, 65536 // 16] for o in range(0, nbytes, 65536)]
    table = torch.tensor(rows, dtype=torch.int64, device=dev)
    a_, b_ = torch.randn(8192, 2048, device=dev).bfloat16(), torch.randn(2048, 2048, device=dev).bfloat16()
    out_ = torch.empty(8192, 2048, device=dev, dtype=torch.bfloat16)

    def gemm_plain():
        cu.gemm_bf16(a_, b_, out=out_)

    def gemm_carrying():
        K.attach_gather_jobs(table)
        cu.gemm_bf16(a_, b_, out=out_)

    t_alone = timed(lambda: K.gather_jobs(table), 20)
    t_plain = timed(gemm_plain, 20)
    t_carry = timed(gemm_carrying, 20)
    res["gather_32MB_stand_alone_us"] = t_alone * 1e3
    res["gather_stand_alone_GBs"] = nbytes / t_alone / 1e6
    res["gemm_plain_us"] = t_plain * 1e3
    res["gemm_carrying_32MB_gather_us"] = t_carry * 1e3
    res["gather_inside_gemm_GBs"] = nbytes / t_carry / 1e6

    vec = torch.rand(512, device=dev)
    res["max_allreduce_kernel_us"] = timed(lambda: max_allreduce_(vec), 50) * 1e3
    res["max_allreduce_nccl_us"] = timed(lambda: dist.all_reduce(vec, op=dist.ReduceOp.MAX), 50) * 1e3
    torch.cuda.synchronize()
    from gdnet_b200 import _ext

    _ext.check_status(vec)
    if rank == 0:
        print(json.dumps(res, indent=1))
        if args.json:
            with open(args.json, "w") as f:
                json.dump(res, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
