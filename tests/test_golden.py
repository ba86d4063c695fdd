"""Committed fixtures (tests/golden/, written by tests/golden/make_golden.py from the CPU oracle).

CPU: the oracle still reproduces them bit for bit.  GPU: the CUDA path agrees with the files
themselves (bit-exact packed codes, routing, permutation, counts; outputs within tolerance), so a
parity claim does not rest on the oracle and the kernels drifting together."""
import glob
import os

import numpy as np
import pytest
import torch

from tests.helpers import close_up_to_bf16_rounding, rel_err

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
BLOCKS = sorted(glob.glob(os.path.join(GOLDEN, "block_*.npz")))
TOL = 2e-2


def _block(path):
    d = np.load(path)
    trip = {n: (d[n + "_wq"], d[n + "_s"], d[n + "_b"]) for n in ("gate", "up", "down")}
    return d, trip


def test_fixtures_exist():
    assert len(BLOCKS) >= 2 and os.path.exists(os.path.join(GOLDEN, "quantize_arange.npz"))


def test_oracle_reproduces_quantize_fixture(O):
    d = np.load(os.path.join(GOLDEN, "quantize_arange.npz"))
    for bits in (2, 4, 8):
        wq, s, b = O.quantize(d["x"], 128, bits, bf16_params=False)
        assert np.array_equal(wq, d[f"wq{bits}"]) and np.array_equal(s, d[f"s{bits}"]) and np.array_equal(b, d[f"b{bits}"])
        deq = O.dequantize(wq, s, b, 128, bits)
        assert np.array_equal(deq, d[f"deq{bits}"])
        # the relation the reference's own test asserts (mlx-rs/src/ops/quantization.rs:297-315)
        assert np.abs(deq - d["x"]).max() <= 127.0 / 2 ** bits


@pytest.mark.parametrize("path", BLOCKS, ids=[os.path.basename(p) for p in BLOCKS])
def test_oracle_reproduces_block_fixture(O, path):
    d, trip = _block(path)
    ref = O.moe_block(d["x"], d["wr"], trip["gate"], trip["up"], trip["down"], int(d["k"]))
    for key in ("idx", "scores", "perm", "inv", "counts", "offsets", "out"):
        assert np.array_equal(ref[key], d[key]), key
    assert rel_err(ref["out_f32"], d["out_f32"]) < 1e-6      # float32 sums: thread count may reorder nothing, but allow a ulp


@pytest.mark.gpu
def test_cuda_quantizer_matches_fixture(pkg):
    d = np.load(os.path.join(GOLDEN, "quantize_arange.npz"))
    x = torch.from_numpy(d["x"]).cuda()
    for bits in (2, 4, 8):
        wq, s, b = pkg.ops.quantize(x, 128, bits)
        assert np.array_equal(wq.cpu().numpy().view(np.uint32), d[f"wq{bits}"])
        assert np.array_equal(s.cpu().numpy(), d[f"s{bits}"]) and np.array_equal(b.cpu().numpy(), d[f"b{bits}"])
        assert np.array_equal(pkg.ops.dequantize(wq, s, b, 128, bits).cpu().numpy(), d[f"deq{bits}"])


@pytest.mark.gpu
@pytest.mark.parametrize("path", BLOCKS, ids=[os.path.basename(p) for p in BLOCKS])
def test_cuda_block_matches_fixture(pkg, path):
    d, trip = _block(path)
    blk = dict(x=d["x"], wr=d["wr"], gate=trip["gate"], up=trip["up"], down=trip["down"], bias=None, k=int(d["k"]),
               bits=int(d["bits"]))
    from tests.helpers import to_device
    block = to_device(pkg, blk)
    x = torch.from_numpy(d["x"]).bfloat16().cuda()
    out, aux = block.forward(x, return_aux=True)
    pkg.default_context().check()
    u = lambda t: t.cpu().numpy().view(np.uint32)
    assert np.array_equal(u(aux["indices"]), d["idx"])
    assert np.array_equal(aux["scores"].float().cpu().numpy(), d["scores"])
    assert np.array_equal(u(aux["perm"]), d["perm"]) and np.array_equal(u(aux["inv_perm"]), d["inv"])
    assert np.array_equal(u(aux["counts"]), d["counts"]) and np.array_equal(u(aux["offsets"]), d["offsets"])
    assert rel_err(aux["out_f32"].cpu().numpy(), d["out_f32"]) <= TOL
    assert close_up_to_bf16_rounding(out.float().cpu().numpy(), d["out_f32"], TOL)
