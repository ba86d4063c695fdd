"""Expert-parallel execution of the routed block over the GPUs of one node.

The reference has no distributed layer at all; expert parallelism is what BASELINE.json asks for
because experts shard naturally.  Layout: rank r owns the contiguous experts
[r*E/G, (r+1)*E/G) (their quantized gate/up/down stacks), the router weight is replicated, every
rank routes its own tokens.  Because experts are contiguous per rank, the expert-sorted rows of
a rank are already grouped by destination, so one forward is

    route -> sort -> (counts all-to-all) -> dispatch all-to-all-v of bf16 rows
          -> local SwitchGLU on the received rows -> combine all-to-all-v back
          -> weighted un-sort + k-way sum on the source rank.

torch.distributed (NCCL over NVLink on GPUs, gloo on CPU in the tests) is the transport; the
compute steps go through a small backend object so that the exchange protocol can be tested on
CPU ranks.  Returned rows travel as bf16 (one rounding per expert output more than the
single-GPU path, which keeps the weighted rows in float32).
"""
import statistics

import torch
import torch.distributed as dist


class B200Backend:
    """Compute steps on this rank's GPU through the C ABI."""

    def __init__(self, pkg, gate_weight, local_switch_mlp, top_k, norm_topk_prob=True, router_mode=0,
                 router_logit_bias=None, ctx=None):
        self.pkg, self.ctx = pkg, ctx
        self.gate_weight, self.mlp = gate_weight, local_switch_mlp
        self.top_k, self.norm, self.mode, self.bias = top_k, norm_topk_prob, router_mode, router_logit_bias

    def router(self, x):
        return self.pkg.nn.router_topk(x, self.gate_weight, self.top_k, self.mode, self.norm, self.bias, ctx=self.ctx)

    def permute(self, flat_idx, n_experts):
        return self.pkg.ops.moe_permute(flat_idx, n_experts, ctx=self.ctx)

    def take_rows(self, x, perm, div):
        return self.pkg.ops.take_rows(x, perm, div, ctx=self.ctx)

    def experts(self, rows, local_ids):
        if rows.shape[0] == 0:
            return rows
        return self.mlp.forward(rows, local_ids.view(-1, 1)).view(rows.shape[0], -1)

    def combine(self, y_sorted, inv, scores):
        return self.pkg.ops.moe_combine(y_sorted, inv, scores, ctx=self.ctx)


def split_sizes(counts_2d):
    """Rows per peer from a [G, E/G] count matrix (host list)."""
    return [int(v) for v in counts_2d.sum(dim=1).tolist()]


def local_expert_ids(recv_counts):
    """Expert (local numbering) of every received row: rows arrive grouped by source rank and,
    within a source, sorted by expert.  recv_counts [G, E/G] (on the rows' device)."""
    G, Eg = recv_counts.shape
    ids = torch.arange(Eg, dtype=torch.int32, device=recv_counts.device).repeat(G)
    return torch.repeat_interleave(ids, recv_counts.reshape(-1).long())


class ExpertParallelMoe:
    def __init__(self, backend, n_experts, top_k, group=None):
        self.be, self.E, self.k = backend, n_experts, top_k
        self.group = group
        self.G = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if n_experts % self.G:
            raise ValueError("the number of experts must be divisible by the number of ranks")
        self.last = {}

    def forward(self, x):
        """x: this rank's tokens [T, H] bf16 -> [T, H] bf16."""
        G, E, k = self.G, self.E, self.k
        Eg = E // G
        T, H = x.shape
        idx, scores = self.be.router(x)
        perm, inv, counts, offsets = self.be.permute(idx.reshape(-1), E)
        rows = self.be.take_rows(x, perm, k)                      # sorted by expert == grouped by destination rank
        send_counts = counts.view(G, Eg).contiguous()
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        both = torch.stack([send_counts, recv_counts]).cpu()      # the one host synchronisation of the step
        sc, rc = split_sizes(both[0]), split_sizes(both[1])
        n_recv = sum(rc)
        recv_rows = torch.empty((n_recv, H), dtype=rows.dtype, device=rows.device)
        dist.all_to_all_single(recv_rows.view(torch.uint8), rows.view(torch.uint8), rc, sc, group=self.group)
        ids = local_expert_ids(recv_counts)
        y = self.be.experts(recv_rows, ids)
        back = torch.empty_like(rows)
        dist.all_to_all_single(back.view(torch.uint8), y.contiguous().view(torch.uint8), sc, rc, group=self.group)
        out = self.be.combine(back, inv, scores)
        self.last = dict(idx=idx, scores=scores, perm=perm, counts=counts, sent_rows=sum(sc) - sc[self.rank],
                         recv_rows=n_recv)
        return out


def shard_switch_mlp(pkg, switch_mlp, rank, world):
    """The contiguous expert shard of a SwitchGlu for `rank` (views, no copy)."""
    E = switch_mlp.n_experts
    lo, hi = rank * E // world, (rank + 1) * E // world

    def cut(q):
        return pkg.nn.QuantizedSwitchLinear(q.weight[lo:hi].contiguous(), q.scales[lo:hi].contiguous(),
                                            q.biases[lo:hi].contiguous(), q.group_size, q.bits)
    return pkg.nn.SwitchGlu(cut(switch_mlp.gate_proj), cut(switch_mlp.up_proj), cut(switch_mlp.down_proj))


def bench_main(args, pkg, shape, peaks, metric, unit, workload_name):
    """bench.py for N > 1: weak scaling, `--tokens` tokens per GPU, experts sharded E/N per GPU.
    Timing: barrier + synchronize, per-step CUDA events, max over ranks."""
    import json
    import os
    rank, world = dist.get_rank(), dist.get_world_size()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    H, I, E, k = shape["hidden"], shape["inter"], shape["n_experts"], shape["top_k"]
    Eg = E // world
    T = args.tokens
    ctx = pkg.default_context()
    # identical router on every rank; each rank draws only its own experts (seeded by expert range)
    g = torch.Generator(device=dev).manual_seed(args.seed)
    wr = (torch.randn(E, H, generator=g, device=dev, dtype=torch.float32) * 0.02).bfloat16()
    gl = torch.Generator(device=dev).manual_seed(args.seed + 1000 + rank)
    lin = []
    for r_, c_ in ((I, H), (I, H), (H, I)):
        w = (torch.randn(Eg, r_, c_, generator=gl, device=dev, dtype=torch.float32) * 0.02).bfloat16()
        lin.append(pkg.nn.QuantizedSwitchLinear.from_weight(w, shape["group_size"], shape["bits"]))
        del w
    mlp = pkg.nn.SwitchGlu(*lin)
    be = B200Backend(pkg, wr, mlp, k)
    ep = ExpertParallelMoe(be, E, k)
    gx = torch.Generator(device=dev).manual_seed(args.seed + 2000 + rank)
    x = torch.randn(T, H, generator=gx, device=dev, dtype=torch.float32).bfloat16()
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            flush_buf.fill_(1)
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for a, b in evs:
            flush_buf.fill_(1)
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([sum(a.elapsed_time(b) for a, b in evs)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps

    l0 = ctx.launch_count()
    ms = timed(lambda: ep.forward(x), args.steps, args.warmup)
    launches = (ctx.launch_count() - l0) // (args.steps + args.warmup) * args.steps
    xh = x.cpu().pin_memory()
    oh = torch.empty_like(xh).pin_memory()
    xd = torch.empty_like(x)

    def e2e_step():
        xd.copy_(xh, non_blocking=True)
        oh.copy_(ep.forward(xd), non_blocking=True)
    e2e_ms = timed(e2e_step, args.steps, args.warmup)
    sent = torch.tensor([float(ep.last["sent_rows"])], device=dev)
    dist.all_reduce(sent, op=dist.ReduceOp.SUM)
    if rank == 0:
        total = T * world
        flops = total * (k * 3 * 2 * H * I + 2 * H * E)
        line = dict(metric=metric, value=total / (ms * 1e-3), unit=unit, n_gpus=world, steps=args.steps,
                    warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype="bf16", data="synthetic",
                    config=dict(workload=workload_name(T) + f" per GPU, {Eg} experts per GPU", tokens_per_gpu=T,
                                l2="flushed between iterations (512 MB overwrite)",
                                parallelism=f"ep{world} (NCCL all-to-all-v dispatch + combine)", **shape),
                    roofline=dict(bound="tensor", achieved=flops / (ms * 1e-3) / 1e12 / world, peak=peaks["tensor"],
                                  unit="TFLOP/s", frac=flops / (ms * 1e-3) / 1e12 / world / peaks["tensor"],
                                  traffic=None, peak_source=peaks["source"],
                                  kernel="whole expert-parallel step per GPU (all kernels and both exchanges)"),
                    cpu_baseline=None,
                    e2e=dict(value=total / (e2e_ms * 1e-3), unit=unit, h2d_bytes_per_step=xh.numel() * 2 * world,
                             d2h_bytes_per_step=oh.numel() * 2 * world),
                    gpu_launches=launches,
                    exchange=dict(rows_sent_off_rank_per_step=sent.item(), bytes_each_way=sent.item() * H * 2))
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()
