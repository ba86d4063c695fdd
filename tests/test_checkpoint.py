"""Checkpoint ingestion (mlx-rs_b200/checkpoint.py): the safetensors container and the MLX naming of a
quantized MoE block.  CPU: container round trip and error paths.  GPU: a block loaded from a file
computes exactly what the block built from the same arrays computes."""
import json
import struct

import numpy as np
import pytest
import torch

from tests.helpers import make_block, to_device


def _ckpt():
    import __graft_entry__ as ge
    from importlib import import_module
    ge.load_package()
    return import_module("mlx_rs_b200.checkpoint")


def _tensors(blk, prefix):
    out = {f"{prefix}.gate.weight": torch.from_numpy(blk["wr"]).bfloat16()}
    for name in ("gate", "up", "down"):
        wq, s, b = blk[name]
        base = f"{prefix}.switch_mlp.{name}_proj"
        out[base + ".weight"] = torch.from_numpy(wq.view(np.int32))
        out[base + ".scales"] = torch.from_numpy(s).bfloat16()
        out[base + ".biases"] = torch.from_numpy(b).bfloat16()
    return out


def test_safetensors_round_trip(tmp_path):
    ck = _ckpt()
    blk = make_block(T=4, H=128, E=4, I=64, k=2, seed=7)
    tensors = _tensors(blk, "model.layers.0.mlp")
    tensors["extra.f32"] = torch.arange(6, dtype=torch.float32).reshape(2, 3)
    path = str(tmp_path / "m.safetensors")
    ck.save_file(tensors, path, metadata={"format": "mlx"})
    with open(path, "rb") as f:                     # the container itself: length, JSON, offsets that tile the data
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    assert header["__metadata__"] == {"format": "mlx"}
    spans = sorted(v["data_offsets"] for k, v in header.items() if k != "__metadata__")
    assert spans[0][0] == 0 and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert header["model.layers.0.mlp.switch_mlp.gate_proj.weight"]["dtype"] == "U32"
    for name, t in tensors.items():
        got = ck.load_tensor(path, name)
        assert got.dtype == t.dtype and got.shape == t.shape
        assert torch.equal(got.view(torch.uint8) if got.dtype == torch.bfloat16 else got,
                           t.view(torch.uint8) if t.dtype == torch.bfloat16 else t)


def test_safetensors_errors(tmp_path):
    ck = _ckpt()
    path = str(tmp_path / "m.safetensors")
    ck.save_file({"a": torch.zeros(3, dtype=torch.float32)}, path)
    with pytest.raises(KeyError):
        ck.load_tensor(path, "b")
    bad = str(tmp_path / "bad.safetensors")
    with open(bad, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40))
    with pytest.raises(ValueError):
        ck.read_header(bad)
    with pytest.raises(ValueError):
        ck.save_file({"a": torch.zeros(3, dtype=torch.float64)}, path)


@pytest.mark.gpu
def test_block_loaded_from_checkpoint_matches(pkg, tmp_path):
    ck = _ckpt()
    blk = make_block(T=40, H=256, E=8, I=128, k=2, seed=17)
    path = str(tmp_path / "layer.safetensors")
    ck.save_file(_tensors(blk, "model.layers.5.mlp"), path)
    loaded = ck.load_moe_block(pkg, path, "model.layers.5.mlp", top_k=2)
    direct = to_device(pkg, blk)
    x = torch.from_numpy(blk["x"]).bfloat16().cuda()
    a, b = loaded.forward(x), direct.forward(x)
    pkg.default_context().check()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    with pytest.raises(ValueError):                 # wrong quantization parameters are caught before any launch
        ck.load_moe_block(pkg, path, "model.layers.5.mlp", top_k=2, bits=8)
