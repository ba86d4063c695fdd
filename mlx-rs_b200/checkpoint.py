"""Checkpoint ingestion: MLX-format safetensors -> the quantized block's device tensors.

The reference loads safetensors through MLX (`Array::load_safetensors`, used by
mlx-lm/src/models/qwen3.rs:521-538) and names a quantized layer's parameters `weight` (uint32
packed codes), `scales`, `biases` (mlx-rs/src/nn/quantized.rs:307-335); an MoE block stores its
experts stacked on a leading axis under `switch_mlp.{gate_proj,up_proj,down_proj}` and its router
under `gate` (the layout BASELINE.json's checkpoints use).  This module reads that layout straight
from the file format - an 8-byte little-endian header length, a JSON header
{name: {dtype, shape, data_offsets}}, then the raw little-endian tensor bytes - with numpy only,
and hands the arrays to the library untouched (the packed layout IS the kernel layout).

A writer is included so that tests and tools can produce such files without MLX.
"""
import json
import struct

import numpy as np
import torch

_NP = {"U32": np.uint32, "I32": np.int32, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "U8": np.uint8,
       "I64": np.int64, "U16": np.uint16}
_TORCH = {"U32": torch.int32, "I32": torch.int32, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
          "U8": torch.uint8, "I64": torch.int64}


def read_header(path):
    """-> (header dict without '__metadata__', offset of the data section)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        if n <= 0 or n > (1 << 27):
            raise ValueError(f"{path}: implausible safetensors header length {n}")
        header = json.loads(f.read(n).decode("utf-8"))
    header.pop("__metadata__", None)
    return header, 8 + n


def load_tensor(path, name, header=None, data_start=None, device="cpu"):
    """One tensor as a torch tensor (uint32 comes back as int32 with the same bits, the dtype the
    library's Python layer uses for packed words)."""
    if header is None:
        header, data_start = read_header(path)
    if name not in header:
        raise KeyError(f"{path}: no tensor named {name!r}")
    meta = header[name]
    dt = meta["dtype"]
    if dt not in _NP:
        raise ValueError(f"{name}: unsupported safetensors dtype {dt}")
    lo, hi = meta["data_offsets"]
    count = int(np.prod(meta["shape"], dtype=np.int64)) if meta["shape"] else 1
    if (hi - lo) != count * np.dtype(_NP[dt]).itemsize:
        raise ValueError(f"{name}: data_offsets do not match shape and dtype")
    arr = np.fromfile(path, dtype=_NP[dt], count=count, offset=data_start + lo).reshape(meta["shape"])
    if dt == "U32":
        t = torch.from_numpy(arr.view(np.int32))
    elif dt == "BF16":
        t = torch.from_numpy(arr.view(np.int16)).view(torch.bfloat16)
    elif dt == "U16":
        t = torch.from_numpy(arr.view(np.int16))
    else:
        t = torch.from_numpy(arr)
    return t.to(device)


def save_file(tensors, path, metadata=None):
    """Writes {name: torch tensor} as safetensors (int32 tensors whose name ends in '.weight' and that hold
    packed codes are stored as U32, the dtype MLX writes)."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype == torch.bfloat16:
            dt, raw = "BF16", t.view(torch.int16).numpy().tobytes()
        elif t.dtype == torch.int32:
            dt, raw = "U32", t.numpy().view(np.uint32).tobytes()
        elif t.dtype == torch.float32:
            dt, raw = "F32", t.numpy().tobytes()
        elif t.dtype == torch.float16:
            dt, raw = "F16", t.numpy().tobytes()
        else:
            raise ValueError(f"{name}: dtype {t.dtype} is not written by this helper")
        header[name] = {"dtype": dt, "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def load_moe_block(pkg, path, prefix, top_k, group_size=64, bits=4, norm_topk_prob=True, router_mode=0, device="cuda",
                   ctx=None):
    """The block stored under `prefix` (e.g. "model.layers.3.mlp"): router `<prefix>.gate.weight` [E, H] and
    the stacked experts `<prefix>.switch_mlp.{gate_proj,up_proj,down_proj}.{weight,scales,biases}` ->
    nn.MoeBlock on `device`.  Shapes are checked against the quantization parameters before anything is
    handed to the library."""
    header, start = read_header(path)

    def get(name):
        return load_tensor(path, f"{prefix}.{name}", header, start, device)

    def linear(which):
        w, s, b = get(f"switch_mlp.{which}.weight"), get(f"switch_mlp.{which}.scales"), get(f"switch_mlp.{which}.biases")
        if w.dim() != 3 or s.shape != b.shape or s.shape[:2] != w.shape[:2]:
            raise ValueError(f"{prefix}.switch_mlp.{which}: expected stacked [E, out, .] weight / scales / biases")
        k = w.shape[2] * 32 // bits
        if s.shape[2] * group_size != k:
            raise ValueError(f"{prefix}.switch_mlp.{which}: scales {tuple(s.shape)} do not match {k} inputs at group size "
                             f"{group_size} and {bits} bits")
        return pkg.nn.QuantizedSwitchLinear(w.contiguous(), s.to(torch.bfloat16).contiguous(),
                                            b.to(torch.bfloat16).contiguous(), group_size, bits)

    gate_w = get("gate.weight").to(torch.bfloat16).contiguous()
    mlp = pkg.nn.SwitchGlu(linear("gate_proj"), linear("up_proj"), linear("down_proj"), ctx=ctx)
    if gate_w.shape != (mlp.n_experts, mlp.hidden):
        raise ValueError(f"{prefix}.gate.weight {tuple(gate_w.shape)} does not match {mlp.n_experts} experts x hidden {mlp.hidden}")
    return pkg.nn.MoeBlock(gate_w, mlp, top_k, norm_topk_prob, router_mode, ctx=ctx)
