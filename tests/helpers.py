"""Seeded synthetic inputs shared by the CPU and GPU tests (shapes follow BASELINE.json's configs)."""
import numpy as np
import torch

from oracle import oracle as O


def make_block(T, H, E, I, k, bits=4, seed=0, zipf_bias=False):
    """One seed -> activations, router and quantized experts, as numpy (oracle side)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).bfloat16().float().numpy()
    wr = (torch.randn(E, H, generator=g) * 0.02).bfloat16().float().numpy()
    q = []
    for r, c in ((I, H), (I, H), (H, I)):
        w = (torch.randn(E, r, c, generator=g) * 0.02).bfloat16().float().numpy()
        q.append(O.quantize(w, 64, bits))
    bias = None
    if zipf_bias:  # skewed routing: 2*ln(p_e), p_e ~ rank^-1.2
        bias = (-2.4 * np.log(np.arange(1, E + 1))).astype(np.float32)
    return dict(x=x, wr=wr, gate=q[0], up=q[1], down=q[2], bias=bias, T=T, H=H, E=E, I=I, k=k, bits=bits)


def to_device(pkg, blk, mode=0, renorm=True):
    def dev(t):
        wq, s, b = t
        return pkg.nn.QuantizedSwitchLinear(torch.from_numpy(wq.view(np.int32)).cuda(),
                                            torch.from_numpy(s).bfloat16().cuda(),
                                            torch.from_numpy(b).bfloat16().cuda(), 64, blk["bits"])
    sw = pkg.nn.SwitchGlu(dev(blk["gate"]), dev(blk["up"]), dev(blk["down"]))
    bias = torch.from_numpy(blk["bias"]).cuda() if blk["bias"] is not None else None
    return pkg.nn.MoeBlock(torch.from_numpy(blk["wr"]).bfloat16().cuda(), sw, blk["k"], renorm, mode, bias)


def bf16_cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).bfloat16().cuda()


def u32(t):
    return t.cpu().numpy().view(np.uint32)


def rel_err(got, ref):
    """max|delta| / rms(reference): the tolerance of the north star is 2e-2 on this quantity."""
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - ref).max() / max(np.sqrt((ref ** 2).mean()), 1e-30))


def close_up_to_bf16_rounding(got, ref, tol):
    """|got - ref| <= tol * rms(ref) + one bf16 rounding of ref (half an ulp is at most 2^-9 |ref|):
    for results that only exist as bf16 (an output of magnitude 8 rms carries a rounding error of
    up to 3 % of rms by itself, more than the tolerance)."""
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    rms = max(np.sqrt((ref ** 2).mean()), 1e-30)
    return bool(np.all(np.abs(got - ref) <= tol * rms + 2.0 ** -8 * np.abs(ref)))
