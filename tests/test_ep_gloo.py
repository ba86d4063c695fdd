"""CPU, world_size 2 over gloo: the expert-parallel exchange protocol of `mlx_rs_b200.ep`.

The compute steps are served by the CPU oracle here (a test double for the GPU backend), so what
is under test is the host logic: destination grouping, counts exchange, split sizes of the two
all-to-all-v calls, local expert numbering of received rows, and the return path."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.helpers import make_block


class OracleBackend:
    def __init__(self, O, blk, rank, world, mode=0, renorm=True):
        self.O, self.blk, self.mode, self.renorm = O, blk, mode, renorm
        E = blk["E"]
        lo, hi = rank * E // world, (rank + 1) * E // world
        self.local = [tuple(a[lo:hi] for a in blk[n]) for n in ("gate", "up", "down")]

    @staticmethod
    def _np(t):
        return t.float().numpy() if t.dtype == torch.bfloat16 else t.numpy()

    def router(self, x):
        idx, sc = self.O.router(self._np(x), self.blk["wr"], self.blk["k"], self.mode, self.renorm, self.blk["bias"])
        return torch.from_numpy(idx.view(np.int32)), torch.from_numpy(sc).bfloat16()

    def permute(self, flat_idx, n_experts):
        return tuple(torch.from_numpy(a.view(np.int32)) for a in self.O.permute(flat_idx.numpy().view(np.uint32), n_experts))

    def take_rows(self, x, perm, div):
        return x[(perm.long() // div)]

    def experts(self, rows, local_ids):
        if rows.shape[0] == 0:
            return rows
        y = self.O.switch_glu(self._np(rows), local_ids.numpy().view(np.uint32)[:, None], *self.local, scores=None,
                              bits=self.blk["bits"])
        return torch.from_numpy(y[:, 0, :]).bfloat16()

    def combine(self, y_sorted, inv, scores):
        T, k = scores.shape
        y = y_sorted.float()[inv.long()].view(T, k, -1)
        return (y * scores.float()[..., None]).sum(1).bfloat16()


def _worker(rank, world, port, cfg, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import __graft_entry__ as ge
        from importlib import import_module
        ge.load_package()
        ep = import_module("mlx_rs_b200.ep")
        from oracle import oracle as O
        blk = make_block(**cfg)
        T = blk["T"]
        lo, hi = rank * T // world, (rank + 1) * T // world
        if cfg.get("uneven") and rank == 1:
            hi = lo          # a rank with no tokens at all
        x = torch.from_numpy(blk["x"][lo:hi]).bfloat16()
        moe = ep.ExpertParallelMoe(OracleBackend(O, blk, rank, world), blk["E"], blk["k"])
        out = moe.forward(x)
        ret[rank] = dict(out=out.float().numpy(), idx=moe.last["idx"].numpy().view(np.uint32),
                         perm=moe.last["perm"].numpy().view(np.uint32), counts=moe.last["counts"].numpy().view(np.uint32),
                         lo=lo, hi=hi)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("cfg", [dict(T=24, H=128, E=8, I=64, k=2, seed=3),
                                 dict(T=10, H=128, E=4, I=64, k=2, seed=4, zipf_bias=True)])
def test_two_rank_exchange_matches_single_process(O, cfg):
    world = 2
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, _free_port(), cfg, ret), nprocs=world, join=True)
        ret = dict(ret)
    blk = make_block(**cfg)
    ref = O.moe_block(blk["x"], blk["wr"], blk["gate"], blk["up"], blk["down"], blk["k"], 0, True, blk["bias"])
    rms = np.sqrt((ref["out_f32"] ** 2).mean())
    for r in range(world):
        lo, hi = ret[r]["lo"], ret[r]["hi"]
        assert np.array_equal(ret[r]["idx"], ref["idx"][lo:hi])                       # routing of its own tokens
        p, _, c, _ = O.permute(ref["idx"][lo:hi], blk["E"])
        assert np.array_equal(ret[r]["perm"], p) and np.array_equal(ret[r]["counts"], c)
        assert np.abs(ret[r]["out"] - ref["out_f32"][lo:hi]).max() <= 2e-2 * rms + 2.0 ** -8 * np.abs(ref["out_f32"][lo:hi]).max()


def test_helpers_for_split_sizes_and_local_ids():
    import __graft_entry__ as ge
    from importlib import import_module
    ge.load_package()
    ep = import_module("mlx_rs_b200.ep")
    counts = torch.tensor([[2, 0, 1], [0, 3, 0]], dtype=torch.int32)   # 2 source ranks, 3 local experts
    assert ep.split_sizes(counts) == [3, 3]
    assert ep.local_expert_ids(counts).tolist() == [0, 0, 2, 1, 1, 1]
    assert ep.local_expert_ids(torch.zeros((2, 3), dtype=torch.int32)).numel() == 0


def test_peer_layout_tables_tile_every_receive_buffer():
    """Host mirror of the peer-memory layout: the segments that all ranks write into one owner's
    buffer are disjoint, gap-free, grouped by local expert and, within an expert, ordered by source."""
    import __graft_entry__ as ge
    from importlib import import_module
    ge.load_package()
    ep = import_module("mlx_rs_b200.ep")
    rng = np.random.default_rng(0)
    G, E = 4, 16
    Eg = E // G
    counts = rng.integers(0, 7, size=(G, E))
    counts[:, 5] = 0                                    # an expert nobody picked
    t = torch.from_numpy(counts.astype(np.int32))
    tables = [ep.layout_tables(t, r) for r in range(G)]
    for d in range(G):
        segs = []
        for el in range(Eg):
            e = d * Eg + el
            for s in range(G):
                segs.append((int(tables[s][0][e]), int(counts[s, e]), el, s))
        pos = 0
        for start, length, el, s in segs:                # already in (expert, source) order
            assert start == pos
            pos += length
        assert pos == counts[:, d * Eg:(d + 1) * Eg].sum()
        assert np.array_equal(tables[d][1].numpy(), counts[:, d * Eg:(d + 1) * Eg].sum(axis=0))
