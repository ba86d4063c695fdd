"""GPU (needs 2 devices, skipped otherwise): expert-parallel block over NCCL against the CPU oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.helpers import make_block

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, cfg, transport, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import __graft_entry__ as ge
        from importlib import import_module
        pkg = ge.load_package()
        ep = import_module("mlx_rs_b200.ep")
        from tests.helpers import to_device
        blk = make_block(**cfg)
        full = to_device(pkg, blk)
        mlp = ep.shard_switch_mlp(pkg, full.switch_mlp, rank, world)
        T = blk["T"]
        bufs = None
        if transport.startswith("device"):
            moe = ep.DeviceSyncExpertParallelMoe(pkg, full.gate_weight, mlp, blk["E"], blk["k"], T * blk["k"])
            if transport == "device2":          # two half-steps: exchanges on the side stream under the other half's products
                moe.comm.set_chunks(2)
        elif transport.startswith("peer"):
            bufs = [ep.PeerBuffers(pkg, blk["H"], T * blk["k"]) for _ in range(2 if transport == "peer2" else 1)]
            moe = ep.PeerExpertParallelMoe(pkg, full.gate_weight, mlp, blk["E"], blk["k"], bufs,
                                           fused_return=(transport == "peer_push"))
        else:
            moe = ep.ExpertParallelMoe(ep.B200Backend(pkg, full.gate_weight, mlp, blk["k"]), blk["E"], blk["k"])
        lo, hi = rank * T // world, (rank + 1) * T // world
        x = torch.from_numpy(blk["x"][lo:hi]).bfloat16().cuda()
        for _ in range(2):                      # twice: scratch reuse across calls
            out = moe.forward(x)
        pkg.default_context().check()
        ret[rank] = dict(out=out.float().cpu().numpy(), idx=moe.last["idx"].cpu().numpy().view(np.uint32),
                         counts=moe.last["counts"].cpu().numpy().view(np.uint32), lo=lo, hi=hi)
        for b in bufs or []:
            b.close()
        if hasattr(moe, "close"):
            moe.close()
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("cfg", [dict(T=96, H=256, E=8, I=128, k=2, seed=3),
                                 dict(T=700, H=512, E=16, I=256, k=4, seed=5),
                                 dict(T=4801, H=512, E=8, I=256, k=2, seed=9)])     # tensor-core regime, odd halves
@pytest.mark.parametrize("transport", ["nccl", "peer", "peer2", "peer_push", "device", "device2"])
def test_expert_parallel_two_gpus(O, cfg, transport):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, _free_port(), cfg, transport, ret), nprocs=world, join=True)
        ret = dict(ret)
    blk = make_block(**cfg)
    ref = O.moe_block(blk["x"], blk["wr"], blk["gate"], blk["up"], blk["down"], blk["k"])
    rms = np.sqrt((ref["out_f32"] ** 2).mean())
    for r in range(world):
        lo, hi = ret[r]["lo"], ret[r]["hi"]
        assert np.array_equal(ret[r]["idx"], ref["idx"][lo:hi])
        assert np.array_equal(ret[r]["counts"], O.permute(ref["idx"][lo:hi], blk["E"])[2])
        d = np.abs(ret[r]["out"] - ref["out_f32"][lo:hi])
        assert np.all(d <= 2e-2 * rms + 2.0 ** -8 * np.abs(ref["out_f32"][lo:hi]))   # bf16 output: one rounding allowed
