"""Expert-parallel execution of the routed block over the GPUs of one node.

The reference has no distributed layer at all; expert parallelism is what BASELINE.json asks for
because experts shard naturally.  Layout: rank r owns the contiguous experts
[r*E/G, (r+1)*E/G) (their quantized gate/up/down stacks), the router weight is replicated, every
rank routes its own tokens.  Because experts are contiguous per rank, the expert-sorted rows of
a rank are already grouped by destination, so one forward is

    route -> sort -> (counts all-to-all) -> dispatch all-to-all-v of bf16 rows
          -> local SwitchGLU on the received rows -> combine all-to-all-v back
          -> weighted un-sort + k-way sum on the source rank.

Two transports:

* `PeerExpertParallelMoe` (the product path on GPUs): each rank maps its peers' exchange buffers
  (CUDA IPC) and the library's own kernels move the rows - the gather into expert order stores
  straight into the owner's buffer, the weighted combine reads the expert outputs straight out of
  the owners' buffers.  NCCL carries only the [G, E] count table and two one-word barriers.
* `ExpertParallelMoe`: torch.distributed all-to-all-v (NCCL on GPUs, gloo on CPU in the tests); the
  compute steps go through a small backend object so that the exchange protocol can be tested on
  CPU ranks.  It is the baseline the peer-memory path is measured against.

Returned rows travel as bf16 in both (one rounding per expert output more than the single-GPU
path, which keeps the weighted rows in float32).
"""
import ctypes as C

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

    def forward(self, x, out=None):
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
        res = self.be.combine(back, inv, scores)
        if out is not None:
            out.copy_(res)
            res = out
        self.last = dict(idx=idx, scores=scores, perm=perm, counts=counts, sent_rows=sum(sc) - sc[self.rank],
                         recv_rows=n_recv)
        return res


def layout_tables(all_counts, rank):
    """Host mirror of b200_ep_layout (numpy/torch CPU ints): (dst_row0 [E], local_counts [E/G])."""
    G, E = all_counts.shape
    Eg = E // G
    c = all_counts.to(torch.int64).cpu()
    per_expert = c.sum(dim=0)                                   # rows arriving for every expert
    dst_row0 = torch.zeros(E, dtype=torch.int64)
    for e in range(E):
        first = (e // Eg) * Eg
        dst_row0[e] = per_expert[first:e].sum() + c[:rank, e].sum()
    return dst_row0.to(torch.int32), per_expert[rank * Eg:(rank + 1) * Eg].to(torch.int32)


class PeerBuffers:
    """This rank's two exchange buffers (arriving rows, expert outputs; capacity_rows x hidden bf16
    each) and the mapped addresses of every peer's.  Collective: every rank of `group` constructs it."""

    def __init__(self, pkg, hidden, capacity_rows, group=None, ctx=None):
        from . import _lib as L
        self.L, self.ctx = L, (ctx or L.default_context())
        self.group, self.hidden, self.capacity = group, hidden, int(capacity_rows)
        self.rank, self.G = dist.get_rank(group), dist.get_world_size(group)
        nbytes = self.capacity * hidden * 2
        self.own, handles = [], []
        for _ in range(2):
            p = C.c_void_p()
            h = C.create_string_buffer(64)
            L.check(L.lib().b200_ep_buffer_alloc(self.ctx.handle, nbytes, C.byref(p), h))
            self.own.append(p.value)
            handles.append(bytes(h.raw))
        gathered = [None] * self.G
        dist.all_gather_object(gathered, handles, group=group)
        self.rows_ptrs, self.y_ptrs, self._opened = [], [], []
        for r in range(self.G):
            for which, lst in ((0, self.rows_ptrs), (1, self.y_ptrs)):
                if r == self.rank:
                    lst.append(self.own[which])
                else:
                    p = C.c_void_p()
                    L.check(L.lib().b200_ep_buffer_open(self.ctx.handle, gathered[r][which], C.byref(p)))
                    lst.append(p.value)
                    self._opened.append(p.value)
        dist.barrier(group=group)

    def close(self):
        """Collective: unmap the peers' buffers, then (after every rank has) free this rank's."""
        torch.cuda.synchronize()
        for p in self._opened:
            self.L.check(self.L.lib().b200_ep_buffer_close(self.ctx.handle, C.c_void_p(p)))
        self._opened = []
        dist.barrier(group=self.group)
        for p in self.own:
            self.L.check(self.L.lib().b200_ep_buffer_free(self.ctx.handle, C.c_void_p(p)))
        self.own = []


class PeerExpertParallelMoe:
    """One forward = route -> sort -> all-gather of the counts -> dispatch kernel (peer stores) ->
    barrier -> SwitchGLU on the arrived rows in place -> barrier -> combine kernel (peer loads).
    The barriers are one-word all-reduces: stream-ordered, so no kernel of this library ever waits
    on another GPU.  The next forward's all-gather is what keeps a fast rank from overwriting
    buffers that a slow rank still reads.

    With `chunks` = 2 the rank's tokens are cut in two halves that use separate exchange buffers:
    the second half's dispatch and the first half's combine run on a side stream, under the expert
    products of the other half.  Measured on 2, 4 and 8 GPUs this is not faster than one chunk
    (the halves fill the 256-row tiles worse and the transfers compete with the products for the
    memory system), so one chunk is the default.  `buffers` is then a list of two PeerBuffers."""

    def __init__(self, pkg, gate_weight, local_switch_mlp, n_experts, top_k, buffers, norm_topk_prob=True,
                 router_mode=0, router_logit_bias=None, fused_return=False, ctx=None):
        self.pkg, self.ctx = pkg, ctx
        # fused_return: the down projection's epilogue stores every finished row straight into the
        # source rank's return buffer (peer stores, overlapped with the products) and the combine is
        # local; otherwise outputs stay on the owner and the combine kernel reads them over NVLink.
        # Measured at 2 GPUs the pull form is the faster one (1.76 against 1.82 ms per step: the
        # epilogue's 32-byte row pieces make poor NVLink packets), hence the default.
        self.fused_return = fused_return
        self.bufs = list(buffers) if isinstance(buffers, (list, tuple)) else [buffers]
        self.chunks = len(self.bufs)
        self.gate_weight, self.mlp = gate_weight, local_switch_mlp
        self.E, self.k = n_experts, top_k
        self.norm, self.mode, self.bias = norm_topk_prob, router_mode, router_logit_bias
        b0 = self.bufs[0]
        self.group, self.G, self.rank = b0.group, b0.G, b0.rank
        if n_experts % self.G:
            raise ValueError("the number of experts must be divisible by the number of ranks")
        dev = gate_weight.device
        self._flag = torch.zeros(1, dtype=torch.int32, device=dev)
        self._all_counts = torch.empty((self.G, self.chunks, n_experts), dtype=torch.int32, device=dev)
        self._views = [(_device_view(b.own[0], b.capacity, b.hidden, dev), _device_view(b.own[1], b.capacity, b.hidden, dev))
                       for b in self.bufs]
        self._side = torch.cuda.Stream(device=dev) if self.chunks > 1 else None
        # the count table goes to the host on its own stream, so that waiting for it overlaps the dispatch
        self._copy = torch.cuda.Stream(device=dev)
        self._table_host = torch.empty((self.G, self.chunks, n_experts), dtype=torch.int32).pin_memory()
        self.last = {}
        self.profile = False      # one-chunk forwards record an event after every phase into self.phase_ms

    def _barrier(self):
        dist.all_reduce(self._flag, group=self.group)

    def forward(self, x, out=None):
        ops, E, k, G, C = self.pkg.ops, self.E, self.k, self.G, self.chunks
        Eg = E // G
        T, H = x.shape
        marks = []

        def mark(name):
            if self.profile and C == 1:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))
        mark("start")
        idx, scores = self.pkg.nn.router_topk(x, self.gate_weight, k, self.mode, self.norm, self.bias, ctx=self.ctx)
        mark("router")
        bounds = [(c * T // C, (c + 1) * T // C) for c in range(C)]
        sort = [ops.moe_permute(idx[lo:hi].reshape(-1), E, ctx=self.ctx) for lo, hi in bounds]   # perm, inv, counts, offsets
        mine = torch.stack([s_[2] for s_ in sort])                                                # [C, E]
        dist.all_gather_into_tensor(self._all_counts.view(-1), mine.view(-1), group=self.group)
        tables, chunk_counts = [], []
        for c in range(C):
            per_chunk = self._all_counts[:, c, :].contiguous()
            chunk_counts.append(per_chunk)
            tables.append(ops.ep_layout(per_chunk, self.rank, self.bufs[c].capacity, ctx=self.ctx))
        mark("sort+allgather+layout")
        gathered = torch.cuda.Event()
        gathered.record()
        with torch.cuda.stream(self._copy):
            self._copy.wait_event(gathered)
            self._table_host.copy_(self._all_counts, non_blocking=True)
            on_host = torch.cuda.Event()
            on_host.record(self._copy)
        if out is None:
            out = torch.empty_like(x)
        main = torch.cuda.current_stream()
        side = self._side or main

        def dispatch(c):
            lo, hi = bounds[c]
            perm, inv, counts, offsets = sort[c]
            ops.ep_dispatch(x[lo:hi], idx[lo:hi], perm, offsets, tables[c][0], self.bufs[c].rows_ptrs, self.bufs[c].capacity,
                            E, rank=self.rank, ctx=self.ctx)

        def combine(c):
            lo, hi = bounds[c]
            perm, inv, counts, offsets = sort[c]
            if self.fused_return:   # my tokens' expert outputs were stored here by their owners, in my sorted order
                ops.moe_combine(self._views[c][1][:(hi - lo) * k], inv, scores[lo:hi], out=out[lo:hi], ctx=self.ctx)
            else:
                ops.ep_combine(self.bufs[c].y_ptrs, idx[lo:hi], inv, offsets, tables[c][0], scores[lo:hi], H,
                               self.bufs[c].capacity, E, out=out[lo:hi], ctx=self.ctx)

        sent = [torch.cuda.Event() for _ in range(C)]
        if C > 1:
            side.wait_stream(main)
        with torch.cuda.stream(side):
            for c in range(C):
                dispatch(c)
                sent[c].record(side)
        # The dispatch needs nothing from the host (the kernels check the capacity themselves and skip rows
        # that would not fit), so the one host synchronisation of the step happens while it runs.
        on_host.synchronize()
        table = self._table_host.to(torch.int64)
        arriving = table.view(G, C, G, Eg).sum(dim=(0, 3))             # [C, destination rank]
        n_recv = []
        for c in range(C):
            if int(arriving[c].max()) > self.bufs[c].capacity:
                raise self.pkg.B200Error(f"a rank would receive {int(arriving[c].max())} rows; the exchange buffers hold "
                                         f"{self.bufs[c].capacity}")
            n_recv.append(int(arriving[c, self.rank]))
            if self.fused_return and (bounds[c][1] - bounds[c][0]) * k > self.bufs[c].capacity:
                raise self.pkg.B200Error("the return buffer is smaller than this rank's own assignments")
        for c in range(C):
            main.wait_event(sent[c])
            mark("dispatch")
            self._barrier()                       # every rank's rows of chunk c have landed
            mark("barrier1")
            if n_recv[c]:
                rows_view, y_view = self._views[c]
                if self.fused_return:
                    addr = ops.ep_return_table(chunk_counts[c], self.rank, self.bufs[c].y_ptrs, H, n_recv[c], self.bufs[c].capacity,
                                               ctx=self.ctx)
                    self.mlp.forward_sorted_scatter(rows_view, tables[c][1], n_recv[c], addr)
                else:
                    self.mlp.forward_sorted(rows_view, tables[c][1], n_recv[c], out=y_view)
            mark("experts")
            self._barrier()                       # every rank's outputs of chunk c are complete
            mark("barrier2")
            if C > 1 and c + 1 < C:
                done = torch.cuda.Event()
                done.record(main)
                with torch.cuda.stream(side):
                    side.wait_event(done)
                    combine(c)                    # under the next chunk's expert products
            else:
                combine(c)
        if C > 1:
            main.wait_stream(side)
        mark("combine")
        if marks:
            torch.cuda.synchronize()
            self.phase_ms = {b[0]: a[1].elapsed_time(b[1]) for a, b in zip(marks, marks[1:])}
        own = table[self.rank].view(C, G, Eg)
        self.last = dict(idx=idx, scores=scores, counts=mine.sum(dim=0).to(torch.int32), recv_rows=sum(n_recv),
                         sent_rows=int(own.sum() - own[:, self.rank].sum()))
        return out


class EpComm:
    """This rank's exchange buffers and control block of the one-call expert-parallel block, connected to every
    peer's (`b200_ep_comm_create` / `_connect`).  Constructing and closing are collective: the handles travel over
    torch.distributed once.  One communicator serves any number of layers of the same shape (their steps follow
    one another on the stream)."""
    N_HANDLES = 6

    def __init__(self, n_experts, top_k, hidden, capacity_rows, capacity_tokens=None, group=None, ctx=None):
        from . import _lib as L
        self.L, self.ctx, self.group = L, (ctx or L.default_context()), group
        self.G, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if n_experts % self.G:
            raise ValueError("the number of experts must be divisible by the number of ranks")
        self.E, self.k, self.hidden = n_experts, top_k, hidden
        self.capacity = int(capacity_rows)
        # token rows a rank can receive: at worst every assignment belongs to a different token
        self.capacity_tokens = int(capacity_tokens if capacity_tokens is not None else capacity_rows)
        h = C.c_void_p()
        mine = C.create_string_buffer(self.N_HANDLES * 64)
        L.check(L.lib().b200_ep_comm_create(self.ctx.handle, self.G, self.rank, n_experts, top_k, hidden, self.capacity,
                                            self.capacity_tokens, C.byref(h), mine))
        self.handle = h
        self.chunks = 1
        gathered = [None] * self.G
        dist.all_gather_object(gathered, bytes(mine.raw), group=group)
        L.check(L.lib().b200_ep_comm_connect(self.ctx.handle, self.handle, b"".join(gathered)))
        dist.barrier(group=group)

    def set_chunks(self, chunks):
        """Half-steps per step (1 or 2); every rank must set the same value.  Two: the exchange of one half of the
        tokens runs under the expert products of the other half."""
        self.L.check(self.L.lib().b200_ep_comm_set_chunks(self.ctx.handle, self.handle, int(chunks)))
        self.chunks = int(chunks)

    def close(self):
        """Collective: every rank stops using the buffers before any rank unmaps or frees them."""
        if self.handle:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            self.L.check(self.L.lib().b200_ep_comm_destroy(self.ctx.handle, self.handle))
            self.handle = None
            dist.barrier(group=self.group)


class DeviceSyncExpertParallelMoe:
    """The expert-parallel block as ONE library call per step (`b200_moe_block_forward_ep`): route, sort, exchange
    of the counts, de-duplicated dispatch, this rank's experts, partial sums and the combine are enqueued on the
    current stream with no host synchronisation and no collective; the ranks order their phases through control
    blocks in each other's memory.  `comm` is an EpComm (shared by the layers of a stack) or the capacity in rows
    of a communicator this object creates and owns."""

    def __init__(self, pkg, gate_weight, local_switch_mlp, n_experts, top_k, comm, capacity_tokens=None,
                 norm_topk_prob=True, router_mode=0, router_logit_bias=None, group=None, ctx=None, keep_routing=True):
        from . import _lib as L
        self.pkg, self.L, self.ctx = pkg, L, (ctx or L.default_context())
        self.gate_weight, self.mlp, self.bias = gate_weight, local_switch_mlp, router_logit_bias
        self.E, self.k, self.hidden = n_experts, top_k, local_switch_mlp.hidden
        self._own_comm = not isinstance(comm, EpComm)
        self.comm = comm if isinstance(comm, EpComm) else EpComm(n_experts, top_k, self.hidden, comm, capacity_tokens,
                                                                   group=group, ctx=self.ctx)
        self.G, self.rank = self.comm.G, self.comm.rank
        self.cfg = L.MoeConfig(self.hidden, local_switch_mlp.inter, n_experts, top_k, local_switch_mlp.gate_proj.bits,
                               local_switch_mlp.gate_proj.group_size, router_mode, int(norm_topk_prob))
        self.params = local_switch_mlp._params(gate_weight, router_logit_bias)
        self.keep_routing, self._aux, self.last = keep_routing, None, {}

    def forward(self, x, out=None):
        L = self.L
        T = x.shape[0]
        if out is None:
            out = torch.empty_like(x)
        aux_c = None
        if self.keep_routing:
            if self._aux is None or self._aux["indices"].shape[0] != T:
                dev = x.device
                self._aux = dict(indices=torch.empty((T, self.k), dtype=torch.int32, device=dev),
                                 scores=torch.empty((T, self.k), dtype=torch.bfloat16, device=dev),
                                 counts=torch.empty(self.E, dtype=torch.int32, device=dev))
            a = self._aux
            aux_c = L.MoeAux(a["indices"].data_ptr(), a["scores"].data_ptr(), None, None, a["counts"].data_ptr(), None, None, None)
            self.last = dict(idx=a["indices"], scores=a["scores"], counts=a["counts"])
        L.check(L.lib().b200_moe_block_forward_ep(self.ctx.handle, self.comm.handle, C.byref(self.cfg), C.byref(self.params),
                                                  L.ptr(x), T, L.ptr(out), C.byref(aux_c) if aux_c is not None else None,
                                                  L.stream_ptr()))
        return out

    def sent_rows(self):
        """Token rows of the last step that left this GPU: one per (token, other rank that owns one of its experts)."""
        idx = self.last["idx"].long()
        dest = idx // (self.E // self.G)
        hit = torch.zeros((idx.shape[0], self.G), dtype=torch.int32, device=idx.device)
        hit.scatter_(1, dest, 1)
        per_rank = hit.sum(dim=0)
        return int(per_rank.sum() - per_rank[self.rank])

    def close(self):
        if self._own_comm:
            self.comm.close()


def _device_view(address, rows, cols, device):
    """A torch bf16 [rows, cols] view of device memory the library allocated (no ownership)."""
    class _Holder:
        pass
    h = _Holder()
    h.__cuda_array_interface__ = dict(shape=(rows, cols), typestr="<i2", data=(int(address), False), version=3)
    return torch.as_tensor(h, device=device).view(torch.bfloat16)


def shard_switch_mlp(pkg, switch_mlp, rank, world):
    """The contiguous expert shard of a SwitchGlu for `rank` (views, no copy)."""
    E = switch_mlp.n_experts
    lo, hi = rank * E // world, (rank + 1) * E // world

    def cut(q):
        return pkg.nn.QuantizedSwitchLinear(q.weight[lo:hi].contiguous(), q.scales[lo:hi].contiguous(),
                                            q.biases[lo:hi].contiguous(), q.group_size, q.bits)
    return pkg.nn.SwitchGlu(cut(switch_mlp.gate_proj), cut(switch_mlp.up_proj), cut(switch_mlp.down_proj))


def _draw_shard(pkg, shape, seed, rank, n_local, dev):
    """The quantized experts rank `rank` owns (seeded by rank, so any process can rebuild any shard)."""
    H, I = shape["hidden"], shape["inter"]
    gl = torch.Generator(device=dev).manual_seed(seed + 1000 + rank)
    lin = []
    for r_, c_ in ((I, H), (I, H), (H, I)):
        parts = []
        for e0 in range(0, n_local, 16):
            w = (torch.randn(min(16, n_local - e0), r_, c_, generator=gl, device=dev, dtype=torch.float32) * 0.02).bfloat16()
            parts.append(pkg.ops.quantize(w, shape["group_size"], shape["bits"]))
            del w
        lin.append(tuple(torch.cat([p_[i] for p_ in parts]) for i in range(3)))
    return lin


def ep_parity(pkg, shape, cfg, seed, world, wr, bias, x, y_ep, idx_ep, n_sample=32):
    """Checks this rank's expert-parallel output against a single-process computation of the same
    tokens: every rank rebuilds ALL experts (the shards are seeded by rank), runs the one-GPU block on
    `n_sample` of its tokens and compares routing (exactly) and outputs (|d| <= 2e-2 rms + two bf16
    roundings: expert outputs cross NVLink as bf16).  -> (max|d| / rms, ok)."""
    dev = x.device
    E, k = shape["n_experts"], shape["top_k"]
    shards = [_draw_shard(pkg, shape, seed, r, E // world, dev) for r in range(world)]
    lin = [pkg.nn.QuantizedSwitchLinear(*(torch.cat([sh[m][i] for sh in shards]) for i in range(3)), shape["group_size"],
                                        shape["bits"]) for m in range(3)]
    del shards
    block = pkg.nn.MoeBlock(wr, pkg.nn.SwitchGlu(*lin), k, cfg["norm_topk_prob"], cfg["router_mode"], bias)
    T = x.shape[0]
    g = torch.Generator().manual_seed(seed + 77)
    rows = torch.randperm(T, generator=g)[:min(n_sample, T)].sort().values.to(dev)
    ref, aux = block.forward(x[rows].contiguous(), return_aux=True)
    torch.cuda.synchronize()
    same_routing = bool(torch.equal(aux["indices"], idx_ep[rows]))
    ref32, got = aux["out_f32"], y_ep[rows].float()
    rms = float(ref32.double().pow(2).mean().sqrt())
    d = (got - ref32).abs()
    ok = same_routing and bool((d <= 2e-2 * rms + 2.0 ** -7 * ref32.abs()).all())
    del block, lin
    torch.cuda.empty_cache()
    return float(d.max()) / max(rms, 1e-30), ok


def bench_main(args, pkg, shape, cfg, peaks, metric, unit, workload_name, clock_sampler, zipf_bias):
    """bench.py for N > 1: weak scaling, `--tokens` tokens per GPU, experts sharded E/N per GPU.
    Timing: barrier + synchronize, per-step CUDA events, max over ranks.  Before anything is timed one
    step's output is checked against the single-GPU block on sampled tokens of every rank (`ep_parity`);
    the run fails when that check does."""
    import json
    import os
    rank, world = dist.get_rank(), dist.get_world_size()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    H, I, E, k = shape["hidden"], shape["inter"], shape["n_experts"], shape["top_k"]
    if E % world:
        raise SystemExit(f"{E} experts do not divide over {world} GPUs")
    Eg = E // world
    T = args.tokens
    ctx = pkg.default_context()
    # identical router on every rank; each rank draws only its own experts (seeded by expert range)
    g = torch.Generator(device=dev).manual_seed(args.seed)
    wr = (torch.randn(E, H, generator=g, device=dev, dtype=torch.float32) * 0.02).bfloat16()
    bias = torch.tensor(zipf_bias(E), dtype=torch.float32, device=dev) if cfg["zipf"] else None
    lin = [pkg.nn.QuantizedSwitchLinear(*t_, shape["group_size"], shape["bits"])
           for t_ in _draw_shard(pkg, shape, args.seed, rank, Eg, dev)]
    mlp = pkg.nn.SwitchGlu(*lin)
    bufs = None
    if args.ep_transport == "device":
        cap = T * k * world if cfg["zipf"] else min(T * k * world, 2 * T * k + 4096)
        ep = DeviceSyncExpertParallelMoe(pkg, wr, mlp, E, k, cap + 64, T * world, norm_topk_prob=cfg["norm_topk_prob"],
                                         router_mode=cfg["router_mode"], router_logit_bias=bias)
        # two half-steps (the exchange of one half under the products of the other) only on request: measured slower
        # than one at 2 and 4 GPUs (1.43 against 1.29 ms and 1.53 against 1.46 ms per step at 8192 tokens per GPU) -
        # the second set of small launches costs more than the overlap returns
        ep.comm.set_chunks(args.ep_chunks or 1)
    elif args.ep_transport in ("peer", "peer_push"):
        # every rank can at worst receive every assignment of every rank; 2x the balanced load is what uniform
        # random routing needs; skewed routing (one expert per GPU owning 43 % of all rows) needs the worst case
        C_ = args.ep_chunks or 1
        cap = T * k * world if cfg["zipf"] else min(T * k * world, 2 * T * k + 4096)
        bufs = [PeerBuffers(pkg, H, cap // C_ + 64) for _ in range(C_)]
        ep = PeerExpertParallelMoe(pkg, wr, mlp, E, k, bufs, norm_topk_prob=cfg["norm_topk_prob"],
                                   router_mode=cfg["router_mode"], router_logit_bias=bias,
                                   fused_return=(args.ep_transport == "peer_push"))
    else:
        ep = ExpertParallelMoe(B200Backend(pkg, wr, mlp, k, cfg["norm_topk_prob"], cfg["router_mode"], bias), E, k)
    gx = torch.Generator(device=dev).manual_seed(args.seed + 2000 + rank)
    x = torch.randn(T, H, generator=gx, device=dev, dtype=torch.float32).bfloat16()
    y0 = ep.forward(x).clone()
    ctx.check()
    par_rel, par_ok = ep_parity(pkg, shape, cfg, args.seed, world, wr, bias, x, y0, ep.last["idx"])
    par = torch.tensor([par_rel, 0.0 if par_ok else 1.0], device=dev)
    dist.all_reduce(par, op=dist.ReduceOp.MAX)
    parity = dict(max_rel=par[0].item(), ok=par[1].item() == 0.0, sampled_tokens_per_rank=min(32, T),
                  against="the single-GPU block on the same tokens with all experts rebuilt on every rank")
    del y0
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
    with clock_sampler(local) as clk:
        ms = timed(lambda: ep.forward(x), args.steps, args.warmup)
    launches = (ctx.launch_count() - l0) // (args.steps + args.warmup) * args.steps
    # end to end from pinned host buffers through HostPipeline (upload of step i+1 and download of
    # step i-1 under step i's kernels and exchanges); every step's copies are inside the timed region
    xhs = [x.cpu().pin_memory(), x.cpu().pin_memory()]
    ohs = [torch.empty_like(xhs[0]).pin_memory(), torch.empty_like(xhs[0]).pin_memory()]
    xh, oh = xhs[0], ohs[0]
    pipe = pkg.nn.HostPipeline(ep, T, H, dev, depth=2)
    for i in range(max(3, args.warmup)):
        pipe.submit(xhs[i % 2], ohs[i % 2])
    pipe.drain()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        pipe.submit(xhs[i % 2], ohs[i % 2])
    pipe.drain()
    ev1.record()
    torch.cuda.synchronize()
    dist.barrier()
    e2e_t = torch.tensor([ev0.elapsed_time(ev1) / args.steps], device=dev)
    dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_ms = e2e_t.item()
    sent = torch.tensor([float(ep.sent_rows() if hasattr(ep, "sent_rows") else ep.last["sent_rows"])], device=dev)
    dist.all_reduce(sent, op=dist.ReduceOp.SUM)
    phases = None
    if bufs and len(bufs) == 1 and os.environ.get("B200_EP_PHASES"):
        ep.profile = True
        acc = {}
        for _ in range(5):
            flush_buf.fill_(1)
            ep.forward(x)
            for kk, vv in ep.phase_ms.items():
                acc[kk] = acc.get(kk, 0.0) + vv / 5
        ep.profile = False
        phases = acc
    if rank == 0:
        total = T * world
        flops = total * (k * 3 * 2 * H * I + 2 * H * E)
        line = dict(metric=metric, value=total / (ms * 1e-3), unit=unit, n_gpus=world, steps=args.steps,
                    warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype="bf16", data="synthetic",
                    config=dict(workload=workload_name(T) + f" per GPU, {Eg} experts per GPU", tokens_per_gpu=T,
                                router_mode=cfg["router_mode"], norm_topk_prob=cfg["norm_topk_prob"], zipf_skew=cfg["zipf"],
                                l2="flushed between iterations (512 MB overwrite)",
                                parallelism=f"ep{world} (" + (
                                    "one library call per step: dispatch/combine kernels over mapped peer memory, phases "
                                    "ordered on the device, no host synchronisation" if args.ep_transport == "device" else
                                    ("dispatch kernel + return fused into the down projection" if args.ep_transport == "peer_push"
                                     else "dispatch/combine kernels") + " over mapped peer memory, NCCL-ordered"
                                    if bufs else "NCCL all-to-all-v dispatch + combine") + ")",
                                ep_chunks=(len(bufs) if bufs else getattr(getattr(ep, "comm", None), "chunks", 1)),
                                **shape),
                    roofline=dict(bound="tensor", achieved=flops / (ms * 1e-3) / 1e12 / world, peak=peaks["tensor"],
                                  unit="TFLOP/s", frac=flops / (ms * 1e-3) / 1e12 / world / peaks["tensor"],
                                  traffic=None, peak_source=peaks["source"],
                                  kernel="whole expert-parallel step per GPU (all kernels and both exchanges)"),
                    cpu_baseline=None,
                    e2e=dict(value=total / (e2e_ms * 1e-3), unit=unit, h2d_bytes_per_step=xh.numel() * 2 * world,
                             d2h_bytes_per_step=oh.numel() * 2 * world),
                    gpu_launches=launches, clocks=clk.summary(), phase_ms=phases, ep_parity=parity,
                    exchange=dict(rows_sent_off_rank_per_step=sent.item(), bytes_each_way=sent.item() * H * 2))
        print(json.dumps(line))
    ctx.check()
    for b in bufs or []:
        b.close()
    if hasattr(ep, "close"):
        ep.close()
    dist.barrier()
    dist.destroy_process_group()
    if not parity["ok"]:
        raise SystemExit("expert-parallel output differs from the single-GPU block: " + json.dumps(parity))


def bench_stack(args, pkg, shape, cfg, peaks, metric, unit, clock_sampler):
    """bench.py --config 2 for N > 1: the 48-layer stack of pre-RMSNorm MoE blocks with residuals, experts sharded
    E/N per GPU, every layer the one-call expert-parallel block over one shared communicator.  The work is the
    single-GPU run's (strong scaling): the 2048 prefill tokens are split evenly over the ranks, the 256 decode
    steps carry ONE token, which lives on rank 0 - the other ranks take part in every step with no tokens of
    their own (their experts still receive the token's rows).  The decode step is replayed from a CUDA graph on
    every rank.  Timing: per-rank CUDA events, max over ranks."""
    import json
    import os
    import statistics as st
    rank, world = dist.get_rank(), dist.get_world_size()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    H, I, E, k = shape["hidden"], shape["inter"], shape["n_experts"], shape["top_k"]
    Eg = E // world
    n_layers, t_prefill, n_decode = args.layers, 2048, 256
    Tp = t_prefill // world
    ctx = pkg.default_context()
    comm = EpComm(E, k, H, t_prefill * k, t_prefill, ctx=ctx)
    blocks = []
    for l in range(n_layers):
        g = torch.Generator(device=dev).manual_seed(args.seed + l)
        wr = (torch.randn(E, H, generator=g, device=dev, dtype=torch.float32) * 0.02).bfloat16()
        lin = [pkg.nn.QuantizedSwitchLinear(*t_, shape["group_size"], shape["bits"])
               for t_ in _draw_shard(pkg, shape, args.seed + 7919 * (l + 1), rank, Eg, dev)]
        blocks.append(DeviceSyncExpertParallelMoe(pkg, wr, pkg.nn.SwitchGlu(*lin), E, k, comm, keep_routing=False, ctx=ctx))
    stack = pkg.nn.MoeStack(blocks, eps=1e-6)
    gx = torch.Generator(device=dev).manual_seed(args.seed + 99 + rank)
    xp = torch.randn(Tp, H, generator=gx, device=dev, dtype=torch.float32).bfloat16()
    xd = torch.zeros(1 if rank == 0 else 0, H, dtype=torch.bfloat16, device=dev)
    holder = {}

    def decode_step():
        holder["o"] = stack.forward(xd)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        decode_step()
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        decode_step()

    def sequence():
        out = stack.forward(xp)
        if rank == 0:
            xd.copy_(out[-1:])
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(n_decode):
            graph.replay()
            if rank == 0:
                xd.copy_(holder["o"])
        ev1.record()
        return ev0, ev1
    for _ in range(max(1, args.warmup // 3)):
        sequence()
    torch.cuda.synchronize()
    dist.barrier()
    tot, dec = [], []
    with clock_sampler(local) as clk:
        for _ in range(args.steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            e0, e1 = sequence()
            b.record()
            torch.cuda.synchronize()
            dist.barrier()
            tot.append(a.elapsed_time(b))
            dec.append(e0.elapsed_time(e1))
    ctx.check()
    t = torch.tensor([st.mean(tot), st.mean(dec)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, dms = t[0].item(), t[1].item()
    if rank == 0:
        line = dict(metric=metric, value=(t_prefill + n_decode) / (ms * 1e-3), unit=unit, n_gpus=world, steps=args.steps,
                    warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16",
                    data="synthetic",
                    config=dict(workload=f"configs[2]: {n_layers} x (RMSNorm eps 1e-6 + MoE block + residual), 2048-token "
                                         f"prefill ({Tp} per GPU) then 256 single-token decode steps (the token lives on rank 0)",
                                l2="working set 2 GB per GPU per pass, far larger than L2",
                                parallelism=f"ep{world}, {Eg} experts per GPU, one library call per layer, phases ordered on the "
                                            "device", cuda_graph="decode steps", **shape),
                    prefill=dict(tokens=t_prefill, ms=ms - dms, tokens_per_s=t_prefill / ((ms - dms) * 1e-3)),
                    decode=dict(steps=n_decode, ms_per_token=dms / n_decode, tokens_per_s=n_decode / (dms * 1e-3)),
                    roofline=None, cpu_baseline=None, e2e=None, clocks=clk.summary())
        print(json.dumps(line))
    comm.close()
    dist.barrier()
    dist.destroy_process_group()
