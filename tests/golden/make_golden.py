"""Writes the committed fixtures of tests/golden/ from the CPU oracle.

The reference's own tests hold no golden vectors for this path (their numeric constants depend on
MLX's random generator), so these fixtures pin the ORACLE, not the reference: they freeze what the
oracle computed when they were written, so that a later change of the oracle (or of a kernel) that
moves a routing decision, a packed code or an output shows up as a diff against a committed file.

    python tests/golden/make_golden.py          # rewrites tests/golden/*.npz

Inputs come from seeded torch generators and are stored in the files together with the outputs, so
the fixtures do not depend on a generator staying stable across torch versions."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle as O  # noqa: E402
from tests.helpers import make_block  # noqa: E402


def quantize_fixture():
    """The deterministic input of the reference's test_quantize_dequantize
    (mlx-rs/src/ops/quantization.rs:297-315): x[r, c] = c, group 128, bits 2 / 4 / 8."""
    out = {}
    x = np.tile(np.arange(512, dtype=np.float32), (4, 1))
    for bits in (2, 4, 8):
        wq, s, b = O.quantize(x, 128, bits, bf16_params=False)   # float32 input -> float32 scales and biases
        out[f"wq{bits}"], out[f"s{bits}"], out[f"b{bits}"] = wq, s, b
        out[f"deq{bits}"] = O.dequantize(wq, s, b, 128, bits)
    out["x"] = x
    return out


def block_fixture(**cfg):
    blk = make_block(**cfg)
    ref = O.moe_block(blk["x"], blk["wr"], blk["gate"], blk["up"], blk["down"], blk["k"])
    out = dict(x=blk["x"], wr=blk["wr"], k=np.int32(blk["k"]), bits=np.int32(blk["bits"]))
    for name in ("gate", "up", "down"):
        wq, s, b = blk[name]
        out[name + "_wq"], out[name + "_s"], out[name + "_b"] = wq, s, b
    for key in ("idx", "scores", "perm", "inv", "counts", "offsets", "out_f32", "out"):
        out[key] = ref[key]
    return out


def main():
    np.savez_compressed(os.path.join(HERE, "quantize_arange.npz"), **quantize_fixture())
    np.savez_compressed(os.path.join(HERE, "block_T6_H128_E4_I64_k2.npz"), **block_fixture(T=6, H=128, E=4, I=64, k=2, seed=101))
    np.savez_compressed(os.path.join(HERE, "block_T24_H256_E8_I128_k2.npz"),
                        **block_fixture(T=24, H=256, E=8, I=128, k=2, seed=102))


if __name__ == "__main__":
    main()
