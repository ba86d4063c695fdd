"""GPU (one device): the peer-memory expert-parallel kernels with G ranks emulated one after another on
a single GPU - every "peer" buffer is a local allocation, and since none of these kernels waits on
another, running the ranks' phases in sequence is the same computation as G processes."""
import numpy as np
import pytest
import torch

from tests.helpers import make_block, to_device

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cfg,G", [(dict(T=96, H=256, E=8, I=128, k=2, seed=3), 2),
                                   (dict(T=700, H=512, E=16, I=256, k=4, seed=5), 4),
                                   (dict(T=2400, H=512, E=8, I=256, k=2, seed=9), 2)])   # tensor-core regime
def test_peer_exchange_emulated_ranks(pkg, O, cfg, G):
    from importlib import import_module
    ep = import_module("mlx_rs_b200.ep")
    ops, dev = pkg.ops, torch.device("cuda", 0)
    blk = make_block(**cfg)
    full = to_device(pkg, blk)
    T, E, k, H = blk["T"], blk["E"], blk["k"], blk["H"]
    Eg = E // G
    cap = T * k
    rows_buf = [torch.zeros((cap, H), dtype=torch.bfloat16, device=dev) for _ in range(G)]
    y_buf = [torch.zeros((cap, H), dtype=torch.bfloat16, device=dev) for _ in range(G)]
    rows_ptrs, y_ptrs = [b.data_ptr() for b in rows_buf], [b.data_ptr() for b in y_buf]
    mlps = [ep.shard_switch_mlp(pkg, full.switch_mlp, r, G) for r in range(G)]
    xs, routed = [], []
    for r in range(G):
        lo, hi = r * T // G, (r + 1) * T // G
        x = torch.from_numpy(blk["x"][lo:hi]).bfloat16().to(dev)
        idx, scores = pkg.nn.router_topk(x, full.gate_weight, k, 0, True, None)
        perm, inv, counts, offsets = ops.moe_permute(idx.reshape(-1), E)
        xs.append(x)
        routed.append((idx, scores, perm, inv, counts, offsets))
    all_counts = torch.stack([rt[4] for rt in routed]).contiguous()
    tables = []
    for r in range(G):
        dst_row0, local_counts = ops.ep_layout(all_counts, r, cap)
        want_row0, want_counts = ep.layout_tables(all_counts, r)
        assert torch.equal(dst_row0.cpu(), want_row0) and torch.equal(local_counts.cpu(), want_counts)
        tables.append((dst_row0, local_counts))
    for r in range(G):      # phase 1 on every rank, then the barrier
        idx, scores, perm, inv, counts, offsets = routed[r]
        ops.ep_dispatch(xs[r], idx, perm, offsets, tables[r][0], rows_ptrs, cap, E, rank=r)
    for r in range(G):      # phase 2
        n_recv = int(tables[r][1].sum())
        if n_recv:
            mlps[r].forward_sorted(rows_buf[r], tables[r][1], n_recv, out=y_buf[r])
    ref = O.moe_block(blk["x"], blk["wr"], blk["gate"], blk["up"], blk["down"], k)
    rms = np.sqrt((ref["out_f32"] ** 2).mean())
    # the same again with the return fused into the down projection: every owner's epilogue stores the
    # rows into the SOURCE rank's return buffer (sorted order of the source), the combine is local
    ret_buf = [torch.zeros((cap, H), dtype=torch.bfloat16, device=dev) for _ in range(G)]
    ret_ptrs = [b.data_ptr() for b in ret_buf]
    for r in range(G):
        n_recv = int(tables[r][1].sum())
        if n_recv:
            addr = ops.ep_return_table(all_counts, r, ret_ptrs, H, n_recv, cap)
            mlps[r].forward_sorted_scatter(rows_buf[r], tables[r][1], n_recv, addr)
    for r in range(G):
        idx, scores, perm, inv, counts, offsets = routed[r]
        n_own = idx.numel()
        out = ops.moe_combine(ret_buf[r][:n_own], inv, scores)
        pkg.default_context().check()
        lo, hi = r * T // G, (r + 1) * T // G
        d = np.abs(out.float().cpu().numpy() - ref["out_f32"][lo:hi])
        assert np.all(d <= 2e-2 * rms + 2.0 ** -8 * np.abs(ref["out_f32"][lo:hi]))
    for r in range(G):      # phase 3
        idx, scores, perm, inv, counts, offsets = routed[r]
        out = ops.ep_combine(y_ptrs, idx, inv, offsets, tables[r][0], scores, H, cap, E)
        pkg.default_context().check()
        lo, hi = r * T // G, (r + 1) * T // G
        assert np.array_equal(idx.cpu().numpy().view(np.uint32), ref["idx"][lo:hi])
        d = np.abs(out.float().cpu().numpy() - ref["out_f32"][lo:hi])
        assert np.all(d <= 2e-2 * rms + 2.0 ** -8 * np.abs(ref["out_f32"][lo:hi]))   # bf16 output: one rounding allowed


def test_peer_exchange_reports_overflow(pkg):
    dev = torch.device("cuda", 0)
    all_counts = torch.tensor([[5, 0], [4, 1]], dtype=torch.int32, device=dev)
    pkg.ops.ep_layout(all_counts, 1, 8)          # rank 0 would receive 9 rows, its buffers hold 8
    with pytest.raises(pkg.B200Error, match="more rows"):
        pkg.default_context().check()
    pkg.default_context().check()                # the status word is cleared by the failed check


def test_sorted_entry_points_keep_to_their_bounds(pkg):
    """Counts that promise more rows than the call holds, and a return table whose buffers are too small: the
    rows beyond the bound are neither read nor written, and the status check reports it."""
    dev = torch.device("cuda", 0)
    blk = make_block(T=64, H=256, E=4, I=128, k=1, seed=12)
    mlp = to_device(pkg, blk).switch_mlp
    ctx = pkg.default_context()
    rows = torch.randn(40, 256, device=dev).bfloat16()
    out = torch.full((48, 256), 7.0, dtype=torch.bfloat16, device=dev)
    counts = torch.tensor([10, 10, 10, 30], dtype=torch.int32, device=dev)        # 60 > 40
    mlp.forward_sorted(rows, counts, 40, out=out[:40])
    with pytest.raises(pkg.B200Error, match="counts"):
        ctx.check()
    assert bool((out[40:] == 7.0).all()), "rows past the call's bound were written"
    ok = torch.tensor([10, 10, 10, 10], dtype=torch.int32, device=dev)
    want = mlp.forward_sorted(rows, ok, 40)
    assert torch.equal(out[:30].view(torch.int16), want[:30].view(torch.int16))   # the first three experts are unaffected
    # return table: one rank, its own return buffer holds 32 of the 40 rows
    ret = torch.full((40, 256), 7.0, dtype=torch.bfloat16, device=dev)
    all_counts = ok.reshape(1, 4)
    addr = pkg.ops.ep_return_table(all_counts, 0, [ret.data_ptr()], 256, 40, 32)
    with pytest.raises(pkg.B200Error, match="more rows"):
        ctx.check()
    assert int((addr == 0).sum()) == 8
    mlp.forward_sorted_scatter(rows, ok, 40, addr)
    ctx.check()
    assert torch.equal(ret[:32].view(torch.int16), want[:32].view(torch.int16)) and bool((ret[32:] == 7.0).all())


@pytest.mark.parametrize("chunks", [1, 2])
@pytest.mark.parametrize("cfg", [dict(T=96, H=256, E=8, I=128, k=2, seed=3),          # register kernel
                                 dict(T=2401, H=512, E=8, I=256, k=2, seed=9)])      # tensor-core regime
def test_one_call_block_single_rank(pkg, O, cfg, chunks, tmp_path):
    """`b200_moe_block_forward_ep` with a group of ONE rank on one GPU: the device-side phase ordering runs
    against its own flags (a rank is its own peer), twice in a row (step counter, buffer reuse), and a step
    whose arrivals exceed the capacity drops them and reports it.  (Two and more ranks need one GPU each:
    tests/test_gpu_ep.py.)"""
    import torch.distributed as dist
    from importlib import import_module
    ep = import_module("mlx_rs_b200.ep")
    dist.init_process_group("gloo", init_method=f"file://{tmp_path}/rdv", rank=0, world_size=1)
    try:
        blk = make_block(**cfg)
        full = to_device(pkg, blk)
        T, E, k = blk["T"], blk["E"], blk["k"]
        x = torch.from_numpy(blk["x"]).bfloat16().cuda()
        ref = O.moe_block(blk["x"], blk["wr"], blk["gate"], blk["up"], blk["down"], k)
        rms = np.sqrt((ref["out_f32"] ** 2).mean())
        moe = ep.DeviceSyncExpertParallelMoe(pkg, full.gate_weight, full.switch_mlp, E, k, T * k)
        moe.comm.set_chunks(chunks)      # two: the step as two half-steps, exchanges on the communicator's side stream
        for _ in range(2):
            out = moe.forward(x)
        pkg.default_context().check()
        assert np.array_equal(moe.last["idx"].cpu().numpy().view(np.uint32), ref["idx"])
        assert np.array_equal(moe.last["counts"].cpu().numpy().view(np.uint32), ref["counts"])
        d = np.abs(out.float().cpu().numpy() - ref["out_f32"])
        assert np.all(d <= 2e-2 * rms + 2.0 ** -7 * np.abs(ref["out_f32"]))   # expert outputs and the result are bf16
        assert moe.sent_rows() == 0
        moe.close()
        small = ep.DeviceSyncExpertParallelMoe(pkg, full.gate_weight, full.switch_mlp, E, k, T * k - 1)
        small.forward(x)
        with pytest.raises(pkg.B200Error, match="more rows"):
            pkg.default_context().check()
        pkg.default_context().check()
        small.close()
    finally:
        dist.destroy_process_group()


def test_stack_of_expert_parallel_blocks_single_rank(pkg, tmp_path):
    """MoeStack over blocks that only have forward(x) (the one-call expert-parallel block, here a group of one rank)
    against the same stack over plain blocks, within the output tolerance (the exchange keeps fp16 partial sums)."""
    import torch.distributed as dist
    from importlib import import_module
    ep = import_module("mlx_rs_b200.ep")
    dist.init_process_group("gloo", init_method=f"file://{tmp_path}/rdv", rank=0, world_size=1)
    try:
        T, H, E, I, k = 24, 256, 8, 128, 2
        blks = [make_block(T, H, E, I, k, seed=500 + l) for l in range(3)]
        plain = [to_device(pkg, b) for b in blks]
        comm = ep.EpComm(E, k, H, T * k, T)
        eps_ = [ep.DeviceSyncExpertParallelMoe(pkg, p.gate_weight, p.switch_mlp, E, k, comm, keep_routing=False) for p in plain]
        x = torch.from_numpy(blks[0]["x"]).bfloat16().cuda()
        want = pkg.nn.MoeStack(plain, eps=1e-6).forward(x)
        got = pkg.nn.MoeStack(eps_, eps=1e-6).forward(x)
        pkg.default_context().check()
        d = (got.float() - want.float()).abs()
        rms = float(want.float().pow(2).mean().sqrt())
        ok = (d <= 2e-2 * rms + 2.0 ** -7 * want.float().abs()).all(dim=1)
        assert float(ok.float().mean()) >= 0.9      # (a last-bit difference can flip a near-tie in a later layer's routing)
        comm.close()
    finally:
        dist.destroy_process_group()
