"""numpy front-end of the CPU oracle (`moe_oracle.cpp`).  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline legs of the benchmark may import
this module, and only as the checker.  The shipped package never does.

bf16 tensors travel as float32 numpy arrays whose values are bf16-representable
(`round_bf16` makes them so); packed weights are uint32; indices are uint32.
Function names follow the reference's op surface (mlx-rs/src/ops/quantization.rs,
sort.rs, indexing/mod.rs, arithmetic.rs); each C function cites its call site.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(_build.build())
    return _lib


def _p(a, ty):
    return a.ctypes.data_as(C.POINTER(ty)) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def num_threads():
    return int(lib().orc_num_threads())


def set_num_threads(n=0):
    """n <= 0: one OpenMP thread per available processor (undoes an inherited OMP_NUM_THREADS=1)."""
    return int(lib().orc_set_num_threads(int(n)))


def to_bf16_bits(a):
    a = _f32(a)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16(_p(a, C.c_float), C.c_int64(a.size), _p(out, C.c_uint16))
    return out


def from_bf16_bits(b):
    b = np.ascontiguousarray(b, dtype=np.uint16)
    out = np.empty(b.shape, dtype=np.float32)
    lib().orc_bf16_to_f32(_p(b, C.c_uint16), C.c_int64(b.size), _p(out, C.c_float))
    return out


def round_bf16(a):
    return from_bf16_bits(to_bf16_bits(a))


def f64_to_bf16(a):
    a = np.ascontiguousarray(a, dtype=np.float64)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().orc_f64_to_bf16(_p(a, C.c_double), C.c_int64(a.size), _p(out, C.c_uint16))
    return from_bf16_bits(out)


def quantize(w, group_size=64, bits=4, bf16_params=True):
    w = _f32(w)
    K = w.shape[-1]
    rows = w.size // K
    epw = 32 // bits
    wq = np.empty(w.shape[:-1] + (K // epw,), dtype=np.uint32)
    s = np.empty(w.shape[:-1] + (K // group_size,), dtype=np.float32)
    b = np.empty_like(s)
    rc = lib().orc_quantize(_p(w, C.c_float), C.c_int64(rows), C.c_int64(K), group_size, bits,
                            int(bf16_params), _p(wq, C.c_uint32), _p(s, C.c_float), _p(b, C.c_float))
    if rc:
        raise ValueError("quantize: unsupported group_size/bits/shape")
    return wq, s, b


def dequantize(wq, scales, biases, group_size=64, bits=4):
    wq, scales, biases = _u32(wq), _f32(scales), _f32(biases)
    epw = 32 // bits
    K = wq.shape[-1] * epw
    rows = wq.size // wq.shape[-1]
    out = np.empty(wq.shape[:-1] + (K,), dtype=np.float32)
    rc = lib().orc_dequantize(_p(wq, C.c_uint32), _p(scales, C.c_float), _p(biases, C.c_float),
                              C.c_int64(rows), C.c_int64(K), group_size, bits, _p(out, C.c_float))
    if rc:
        raise ValueError("dequantize: unsupported group_size/bits/shape")
    return out


def quantized_matmul(x, wq, scales, biases, transpose=False, group_size=64, bits=4):
    x, wq, scales, biases = _f32(x), _u32(wq), _f32(scales), _f32(biases)
    epw = 32 // bits
    K = x.shape[-1]
    M = x.size // K
    N = wq.shape[0] if transpose else wq.shape[1] * epw
    out = np.empty(x.shape[:-1] + (N,), dtype=np.float32)
    rc = lib().orc_quantized_matmul(_p(x, C.c_float), C.c_int64(M), C.c_int64(K), _p(wq, C.c_uint32),
                                    _p(scales, C.c_float), _p(biases, C.c_float), C.c_int64(N),
                                    int(transpose), group_size, bits, _p(out, C.c_float))
    if rc:
        raise ValueError("quantized_matmul failed")
    return out


def gather_mm(a, b, lhs_indices=None, rhs_indices=None):
    a, b = _f32(a), _f32(b)
    M, K = a.shape[-2:]
    N = b.shape[-1]
    Ba, Bb = a.size // (M * K), b.size // (K * N)
    lhs = _u32(lhs_indices).ravel() if lhs_indices is not None else None
    rhs = _u32(rhs_indices).ravel() if rhs_indices is not None else None
    n = (lhs if lhs is not None else rhs).size
    shape = (np.shape(lhs_indices) if lhs_indices is not None else np.shape(rhs_indices))
    out = np.empty(tuple(shape) + (M, N), dtype=np.float32)
    rc = lib().orc_gather_mm(_p(a, C.c_float), C.c_int64(Ba), C.c_int64(M), C.c_int64(K), _p(b, C.c_float),
                             C.c_int64(Bb), C.c_int64(N), _p(lhs, C.c_uint32), _p(rhs, C.c_uint32),
                             C.c_int64(n), _p(out, C.c_float))
    if rc:
        raise IndexError("gather_mm: index out of range")
    return out


def gather_qmm(x, wq, scales, biases, lhs_indices=None, rhs_indices=None, transpose=True, group_size=64, bits=4):
    assert transpose, "the oracle restates the transpose=true form used by every layer"
    x, wq, scales, biases = _f32(x), _u32(wq), _f32(scales), _f32(biases)
    M, K = x.shape[-2:]
    Bx = x.size // (M * K)
    N = wq.shape[-2]
    E = wq.size // (N * wq.shape[-1])
    lhs = _u32(lhs_indices).ravel() if lhs_indices is not None else None
    rhs = _u32(rhs_indices).ravel()
    shape = np.shape(rhs_indices)
    out = np.empty(tuple(shape) + (M, N), dtype=np.float32)
    rc = lib().orc_gather_qmm(_p(x, C.c_float), C.c_int64(Bx), C.c_int64(M), C.c_int64(K), _p(wq, C.c_uint32),
                              _p(scales, C.c_float), _p(biases, C.c_float), C.c_int64(E), C.c_int64(N),
                              _p(lhs, C.c_uint32), _p(rhs, C.c_uint32), C.c_int64(rhs.size), group_size, bits,
                              _p(out, C.c_float))
    if rc:
        raise IndexError("gather_qmm: index out of range")
    return out


def softmax(a):
    a = _f32(a)
    cols = a.shape[-1]
    out = np.empty(a.shape, dtype=np.float64)
    lib().orc_softmax_f64(_p(a, C.c_float), C.c_int64(a.size // cols), C.c_int64(cols), _p(out, C.c_double))
    return out


def argsort(keys):
    keys = _u32(keys)
    cols = keys.shape[-1]
    out = np.empty(keys.shape, dtype=np.uint32)
    lib().orc_argsort_u32(_p(keys, C.c_uint32), C.c_int64(keys.size // cols), C.c_int64(cols), _p(out, C.c_uint32))
    return out


def argpartition(a, kth):
    a = _f32(a)
    cols = a.shape[-1]
    out = np.empty(a.shape, dtype=np.uint32)
    lib().orc_argpartition_f32(_p(a, C.c_float), C.c_int64(a.size // cols), C.c_int64(cols), int(kth),
                               _p(out, C.c_uint32))
    return out


def take_along_axis(a, idx):
    a, idx = _f32(a), _u32(idx)
    cols, icol = a.shape[-1], idx.shape[-1]
    out = np.empty(idx.shape, dtype=np.float32)
    rc = lib().orc_take_along_last(_p(a, C.c_float), C.c_int64(a.size // cols), C.c_int64(cols),
                                   _p(idx, C.c_uint32), C.c_int64(icol), _p(out, C.c_float))
    if rc:
        raise IndexError("take_along_axis: index out of range")
    return out


def rms_norm(x, weight=None, eps=1e-5):
    x = _f32(x)
    cols = x.shape[-1]
    w = _f32(weight) if weight is not None else None
    out = np.empty_like(x)
    lib().orc_rms_norm(_p(x, C.c_float), _p(w, C.c_float), C.c_int64(x.size // cols), C.c_int64(cols),
                       C.c_float(eps), _p(out, C.c_float))
    return out


def router(x, wr, top_k, mode=0, renorm=True, logit_bias=None, return_logits=False):
    """-> (idx [T,k] uint32, scores [T,k] bf16-valued float32[, logits [T,E]])."""
    x, wr = _f32(x), _f32(wr)
    T, H = x.shape
    E = wr.shape[0]
    idx = np.empty((T, top_k), dtype=np.uint32)
    sc = np.empty((T, top_k), dtype=np.float32)
    lg = np.empty((T, E), dtype=np.float32) if return_logits else None
    lb = _f32(logit_bias) if logit_bias is not None else None
    rc = lib().orc_router(_p(x, C.c_float), _p(wr, C.c_float), C.c_int64(T), C.c_int64(H), C.c_int64(E), int(top_k),
                          int(mode), int(renorm), _p(lb, C.c_float), _p(lg, C.c_float), _p(idx, C.c_uint32),
                          _p(sc, C.c_float))
    if rc:
        raise ValueError("router: bad top_k")
    return (idx, sc, lg) if return_logits else (idx, sc)


def permute(idx, n_experts):
    """Stable token->expert sort -> (perm, inv, counts [E], offsets [E+1]); all uint32."""
    flat = _u32(idx).ravel()
    n = flat.size
    perm = np.empty(n, dtype=np.uint32)
    inv = np.empty(n, dtype=np.uint32)
    counts = np.empty(n_experts, dtype=np.uint32)
    offsets = np.empty(n_experts + 1, dtype=np.uint32)
    rc = lib().orc_permute(_p(flat, C.c_uint32), C.c_int64(n), C.c_int64(n_experts), _p(perm, C.c_uint32),
                           _p(inv, C.c_uint32), _p(counts, C.c_uint32), _p(offsets, C.c_uint32))
    if rc:
        raise IndexError("permute: expert index out of range")
    return perm, inv, counts, offsets


def switch_glu(x, idx, gate, up, down, scores=None, group_size=64, bits=4, round_every_op=False, round_out=True):
    """gate/up/down are (wq, scales, biases) triples.  -> [T,H] when `scores` is given
    (weighted combine), else the per-assignment outputs [T,k,H].  `round_out=False` returns
    the float32 accumulation without the final bf16 rounding."""
    x, idx = _f32(x), _u32(idx)
    T, H = x.shape
    k = idx.shape[-1]
    gq, gs_, gb = _u32(gate[0]), _f32(gate[1]), _f32(gate[2])
    uq, us, ub = _u32(up[0]), _f32(up[1]), _f32(up[2])
    dq, ds, db = _u32(down[0]), _f32(down[1]), _f32(down[2])
    E, I = gq.shape[0], gq.shape[1]
    sc = _f32(scores) if scores is not None else None
    out = np.empty((T, H) if sc is not None else (T, k, H), dtype=np.float32)
    rc = lib().orc_switch_glu(_p(x, C.c_float), C.c_int64(T), C.c_int64(H), C.c_int64(E), C.c_int64(I), int(k),
                              _p(idx, C.c_uint32), _p(sc, C.c_float), _p(gq, C.c_uint32), _p(gs_, C.c_float),
                              _p(gb, C.c_float), _p(uq, C.c_uint32), _p(us, C.c_float), _p(ub, C.c_float),
                              _p(dq, C.c_uint32), _p(ds, C.c_float), _p(db, C.c_float), group_size, bits,
                              int(round_every_op), int(round_out), _p(out, C.c_float))
    if rc:
        raise IndexError("switch_glu: expert index out of range")
    return out


def moe_block(x, wr, gate, up, down, top_k, mode=0, renorm=True, logit_bias=None, group_size=64, bits=4,
              round_every_op=False):
    """Whole block -> dict(out, out_f32, idx, scores, perm, inv, counts, offsets); `out_f32` is the
    float32 accumulation before the final bf16 rounding, `out` its bf16 rounding."""
    idx, sc = router(x, wr, top_k, mode, renorm, logit_bias)
    perm, inv, counts, offsets = permute(idx, np.shape(wr)[0])
    out32 = switch_glu(x, idx, gate, up, down, sc, group_size, bits, round_every_op, round_out=False)
    return dict(out=round_bf16(out32), out_f32=out32, idx=idx, scores=sc, perm=perm, inv=inv, counts=counts,
                offsets=offsets)
