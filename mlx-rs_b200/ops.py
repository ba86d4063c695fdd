"""Op surface of the reference, one function per wrapper, same names / argument order / defaults.

quantize / dequantize / quantized_matmul / gather_qmm: mlx-rs/src/ops/quantization.rs:48-230
softmax_axis: mlx-rs/src/ops/arithmetic.rs:1312-1327; argpartition_axis: mlx-rs/src/ops/sort.rs:186-226
take_along_axis: mlx-rs/src/ops/indexing/mod.rs:424-453; rms_norm: mlx-rs/src/fast.rs:178-205

Tensors are torch CUDA tensors (torch only holds the memory).  Index tensors are int32 (same
bits as the reference's uint32 for every valid index).  Calls are eager and stream-ordered.
"""
import ctypes as C

import torch

from . import _lib as L

DEFAULT_GROUP_SIZE = 64
DEFAULT_BITS = 4
_DT = {torch.float32: 0, torch.bfloat16: 1}
_DT3 = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}   # activation dtypes of the matmul ops


def _ctx(ctx):
    return (ctx or L.default_context()).handle


def _req(cond, msg):
    if not cond:
        raise L.B200Error(msg)


def _cuda(*ts):
    for t in ts:
        _req(t is None or (t.is_cuda and t.is_contiguous()), "tensors must be contiguous CUDA tensors")


def quantize(w, group_size=DEFAULT_GROUP_SIZE, bits=DEFAULT_BITS, ctx=None):
    """-> (w_q uint32-as-int32 [..., K*bits/32], scales [..., K/gs], biases [..., K/gs])."""
    _cuda(w)
    _req(w.dtype in _DT, "quantize: float32 or bfloat16 input")
    _req(w.dim() >= 2, "quantize: at least 2 dimensions")  # the reference rejects 1-D input too
    K = w.shape[-1]
    _req(bits in (2, 4, 8) and group_size in (32, 64, 128) and K % group_size == 0,
         f"quantize: unsupported group_size={group_size} bits={bits} for last axis {K}")
    rows = w.numel() // K
    wq = torch.empty(w.shape[:-1] + (K * bits // 32,), dtype=torch.int32, device=w.device)
    s = torch.empty(w.shape[:-1] + (K // group_size,), dtype=w.dtype, device=w.device)
    b = torch.empty_like(s)
    L.check(L.lib().b200_quantize(_ctx(ctx), L.ptr(w), _DT[w.dtype], rows, K, group_size, bits, L.ptr(wq), L.ptr(s),
                                  L.ptr(b), L.stream_ptr()))
    return wq, s, b


def dequantize(w, scales, biases, group_size=DEFAULT_GROUP_SIZE, bits=DEFAULT_BITS, ctx=None):
    _cuda(w, scales, biases)
    _req(scales.dtype in _DT and biases.dtype == scales.dtype, "dequantize: scales/biases float32 or bfloat16")
    K = w.shape[-1] * 32 // bits
    rows = w.numel() // w.shape[-1]
    out = torch.empty(w.shape[:-1] + (K,), dtype=scales.dtype, device=w.device)
    L.check(L.lib().b200_dequantize(_ctx(ctx), L.ptr(w), L.ptr(scales), L.ptr(biases), _DT[scales.dtype], rows, K,
                                    group_size, bits, L.ptr(out), L.stream_ptr()))
    return out


def quantized_matmul(x, w, scales, biases, transpose=False, group_size=DEFAULT_GROUP_SIZE, bits=DEFAULT_BITS, ctx=None):
    """x [..., K] float32 / bfloat16 / float16; scales and biases in the same dtype -> [..., N] in that dtype."""
    _cuda(x, w, scales, biases)
    _req(x.dtype in _DT3 and scales.dtype == x.dtype and biases.dtype == x.dtype,
         "quantized_matmul: float32, bfloat16 or float16 activations with scales and biases of the same dtype")
    K = x.shape[-1]
    M = x.numel() // K
    N = w.shape[0] if transpose else w.shape[1] * 32 // bits
    _req((w.shape[1] * 32 // bits == K) if transpose else (w.shape[0] == K), "quantized_matmul: shape mismatch")
    out = torch.empty(x.shape[:-1] + (N,), dtype=x.dtype, device=x.device)
    L.check(L.lib().b200_quantized_matmul(_ctx(ctx), L.ptr(x), L.ptr(w), L.ptr(scales), L.ptr(biases), int(transpose),
                                          group_size, bits, _DT3[x.dtype], M, K, N, L.ptr(out), L.stream_ptr()))
    return out


def gather_mm(a, b, lhs_indices=None, rhs_indices=None, ctx=None):
    """a [..., M, K], b [..., K, N] (batch dims flattened) -> [*idx.shape, M, N]; bf16, float32 accumulation."""
    _cuda(a, b, lhs_indices, rhs_indices)
    _req(a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "gather_mm: bf16 operands")
    M, K = a.shape[-2], a.shape[-1]
    N = b.shape[-1]
    _req(b.shape[-2] == K, "gather_mm: inner dimensions differ")
    Ba, Bb = a.numel() // (M * K), b.numel() // (K * N)
    idx = lhs_indices if lhs_indices is not None else rhs_indices
    _req(idx is not None, "gather_mm: at least one index array")
    _req(lhs_indices is None or rhs_indices is None or lhs_indices.shape == rhs_indices.shape,
         "gather_mm: index shapes differ")
    out = torch.empty(tuple(idx.shape) + (M, N), dtype=a.dtype, device=a.device)
    L.check(L.lib().b200_gather_mm(_ctx(ctx), L.ptr(a), L.ptr(b), L.ptr(lhs_indices), L.ptr(rhs_indices), Ba, Bb, M, K, N,
                                   idx.numel(), L.ptr(out), L.stream_ptr()))
    return out


def gather_qmm(x, w, scales, biases, lhs_indices=None, rhs_indices=None, transpose=True, group_size=DEFAULT_GROUP_SIZE,
               bits=DEFAULT_BITS, sorted_indices=False, ctx=None):
    """x [..., M, K] (batch dims flattened), w [E, N, K*bits/32] (transpose) or [E, K, N*bits/32] -> [*idx.shape, M, N]."""
    _cuda(x, w, scales, biases, lhs_indices, rhs_indices)
    _req(x.dtype in _DT3 and scales.dtype == x.dtype and biases.dtype == x.dtype,
         "gather_qmm: float32, bfloat16 or float16 activations with scales and biases of the same dtype")
    _req(rhs_indices is not None, "gather_qmm: rhs_indices is required")
    M, K = x.shape[-2], x.shape[-1]
    Bx = x.numel() // (M * K)
    N = w.shape[-2] if transpose else w.shape[-1] * 32 // bits
    E = w.numel() // (w.shape[-2] * w.shape[-1])
    n_idx = rhs_indices.numel()
    _req(lhs_indices is None or lhs_indices.numel() == n_idx, "gather_qmm: index shapes differ")
    _req(lhs_indices is not None or Bx == n_idx, "gather_qmm: without lhs_indices x needs one batch entry per index")
    out = torch.empty(tuple(rhs_indices.shape) + (M, N), dtype=x.dtype, device=x.device)
    L.check(L.lib().b200_gather_qmm(_ctx(ctx), L.ptr(x), L.ptr(w), L.ptr(scales), L.ptr(biases), L.ptr(lhs_indices),
                                    L.ptr(rhs_indices), int(transpose), group_size, bits, int(sorted_indices), _DT3[x.dtype],
                                    Bx, M, K, E, N, n_idx, L.ptr(out), L.stream_ptr()))
    return out


def softmax_axis(a, axis=-1, precise=True, ctx=None):
    _cuda(a)
    _req(axis in (-1, a.dim() - 1) and a.dtype == torch.bfloat16, "softmax_axis: last axis of a bf16 tensor")
    cols = a.shape[-1]
    out = torch.empty_like(a)
    L.check(L.lib().b200_softmax_axis(_ctx(ctx), L.ptr(a), a.numel() // cols, cols, int(precise), L.ptr(out),
                                      L.stream_ptr()))
    return out


def argpartition_axis(a, kth, axis=-1, ctx=None):
    _cuda(a)
    _req(axis in (-1, a.dim() - 1) and a.dtype == torch.bfloat16, "argpartition_axis: last axis of a bf16 tensor")
    cols = a.shape[-1]
    out = torch.empty(a.shape, dtype=torch.int32, device=a.device)
    L.check(L.lib().b200_argpartition_axis(_ctx(ctx), L.ptr(a), a.numel() // cols, cols, int(kth), L.ptr(out),
                                           L.stream_ptr()))
    return out


def take_along_axis(a, indices, axis=-1, ctx=None):
    _cuda(a, indices)
    _req(axis in (-1, a.dim() - 1) and a.element_size() == 2, "take_along_axis: last axis of a 2-byte tensor")
    _req(a.shape[:-1] == indices.shape[:-1], "take_along_axis: leading dimensions differ")
    cols, icols = a.shape[-1], indices.shape[-1]
    out = torch.empty(indices.shape, dtype=a.dtype, device=a.device)
    L.check(L.lib().b200_take_along_axis(_ctx(ctx), L.ptr(a), a.numel() // cols, cols, L.ptr(indices), icols,
                                         L.ptr(out), L.stream_ptr()))
    return out


def take_axis(x, indices, axis=0, ctx=None):
    """take_axis(x, indices, 0) for a 2-D bf16 tensor -> [len(indices), cols]."""
    _req(axis == 0, "take_axis: axis 0")
    return take_rows(x, indices, 1, ctx=ctx)


def argsort_axis(keys, axis=-1, key_bound=256, ctx=None):
    """Stable ascending argsort along the last axis of small unsigned keys (expert indices < key_bound <= 256)."""
    _cuda(keys)
    _req(axis in (-1, keys.dim() - 1) and keys.dtype == torch.int32, "argsort_axis: last axis of an int32 tensor")
    cols = keys.shape[-1]
    out = torch.empty_like(keys)
    L.check(L.lib().b200_argsort_axis(_ctx(ctx), L.ptr(keys), keys.numel() // max(cols, 1), cols, int(key_bound), L.ptr(out),
                                      L.stream_ptr()))
    return out


def topk_axis(a, k, axis=-1, ctx=None):
    """The k largest values along the last axis of a bf16 tensor (ascending)."""
    _cuda(a)
    _req(axis in (-1, a.dim() - 1) and a.dtype == torch.bfloat16, "topk_axis: last axis of a bf16 tensor")
    cols = a.shape[-1]
    out = torch.empty(a.shape[:-1] + (k,), dtype=a.dtype, device=a.device)
    L.check(L.lib().b200_topk_axis(_ctx(ctx), L.ptr(a), a.numel() // cols, cols, int(k), L.ptr(out), L.stream_ptr()))
    return out


def rms_norm(x, weight=None, eps=1e-5, ctx=None):
    _cuda(x, weight)
    cols = x.shape[-1]
    out = torch.empty_like(x)
    L.check(L.lib().b200_rms_norm(_ctx(ctx), L.ptr(x), L.ptr(weight), float(eps), x.numel() // cols, cols, L.ptr(out),
                                  L.stream_ptr()))
    return out


def add_rms_norm(x, residual, weight=None, eps=1e-5, ctx=None):
    """-> (bf16(x + residual), rms_norm of that sum)."""
    _cuda(x, residual, weight)
    cols = x.shape[-1]
    s, out = torch.empty_like(x), torch.empty_like(x)
    L.check(L.lib().b200_add_rms_norm(_ctx(ctx), L.ptr(x), L.ptr(residual), L.ptr(weight), float(eps),
                                      x.numel() // cols, cols, L.ptr(s), L.ptr(out), L.stream_ptr()))
    return s, out


def moe_permute(indices, n_experts, ctx=None):
    """Stable token->expert sort of the flat index list -> (perm, inv_perm, counts [E], offsets [E+1])."""
    _cuda(indices)
    n = indices.numel()
    dev = indices.device
    perm = torch.empty(n, dtype=torch.int32, device=dev)
    inv = torch.empty(n, dtype=torch.int32, device=dev)
    counts = torch.empty(n_experts, dtype=torch.int32, device=dev)
    offsets = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    L.check(L.lib().b200_moe_permute(_ctx(ctx), L.ptr(indices), n, n_experts, L.ptr(perm), L.ptr(inv), L.ptr(counts),
                                     L.ptr(offsets), L.stream_ptr()))
    return perm, inv, counts, offsets


def take_rows(x, indices, div=1, ctx=None):
    """take_axis(x, indices // div, axis=0) for a 2-D bf16 tensor -> [len(indices), cols]."""
    _cuda(x, indices)
    _req(x.dim() == 2 and x.element_size() == 2, "take_rows: 2-D tensor of 2-byte elements")
    out = torch.empty((indices.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    L.check(L.lib().b200_take_rows(_ctx(ctx), L.ptr(x), L.ptr(indices), int(div), indices.numel(), x.shape[0], x.shape[1],
                                   L.ptr(out), L.stream_ptr()))
    return out


def moe_combine(y_sorted, inv_perm, scores, return_f32=False, out=None, ctx=None):
    """out[t] = sum_j scores[t, j] * y_sorted[inv_perm[t*k + j]] (float32 accumulation) -> bf16 [T, H]."""
    _cuda(y_sorted, inv_perm, scores, out)
    T, k = scores.shape
    H = y_sorted.shape[-1]
    if out is None:
        out = torch.empty((T, H), dtype=torch.bfloat16, device=y_sorted.device)
    o32 = torch.empty((T, H), dtype=torch.float32, device=y_sorted.device) if return_f32 else None
    L.check(L.lib().b200_moe_combine(_ctx(ctx), L.ptr(y_sorted), L.ptr(inv_perm), L.ptr(scores), T, k, H, L.ptr(out),
                                     L.ptr(o32), L.stream_ptr()))
    return (out, o32) if return_f32 else out


def _ptr_array(ptrs):
    arr = (C.c_void_p * len(ptrs))(*[int(v) for v in ptrs])
    return arr


def ep_layout(all_counts, rank, capacity_rows, ctx=None):
    """all_counts int32 [G, E] (rows rank s routes to expert e) -> (dst_row0 [E], local_counts [E/G]):
    where this rank's rows of each expert start in the owner's exchange buffers, and how many rows
    arrive here per local expert."""
    _cuda(all_counts)
    G, E = all_counts.shape
    dst_row0 = torch.empty(E, dtype=torch.int32, device=all_counts.device)
    local_counts = torch.empty(E // G, dtype=torch.int32, device=all_counts.device)
    L.check(L.lib().b200_ep_layout(_ctx(ctx), L.ptr(all_counts), G, E, rank, capacity_rows, L.ptr(dst_row0),
                                   L.ptr(local_counts), L.stream_ptr()))
    return dst_row0, local_counts


def ep_return_table(all_counts, rank, peer_y, hidden, n_rows, capacity_rows, ctx=None):
    """-> int64 [n_rows]: for every row this rank receives, the address of its output row in the source
    rank's return buffer (peer_y: device addresses of all ranks' return buffers, capacity_rows rows each)."""
    _cuda(all_counts)
    G, E = all_counts.shape
    addr = torch.empty(max(n_rows, 1), dtype=torch.int64, device=all_counts.device)
    L.check(L.lib().b200_ep_return_table(_ctx(ctx), L.ptr(all_counts), G, E, rank, _ptr_array(peer_y), hidden, n_rows,
                                         capacity_rows, L.ptr(addr), L.stream_ptr()))
    return addr


def ep_dispatch(x, indices, perm, offsets, dst_row0, peer_rows, capacity_rows, n_experts, rank=0, ctx=None):
    """Store every sorted row of this rank into the rows buffer of the rank that owns its expert
    (peer_rows: device addresses of all ranks' buffers, own entry included)."""
    _cuda(x, indices, perm, offsets, dst_row0)
    k = indices.shape[-1]
    L.check(L.lib().b200_ep_dispatch(_ctx(ctx), L.ptr(x), L.ptr(indices), L.ptr(perm), L.ptr(offsets), L.ptr(dst_row0),
                                     perm.numel(), k, x.shape[-1], n_experts, len(peer_rows), rank, _ptr_array(peer_rows),
                                     capacity_rows, L.stream_ptr()))


def ep_combine(peer_y, indices, inv_perm, offsets, dst_row0, scores, hidden, capacity_rows, n_experts, out=None, ctx=None):
    """out[t] = bf16(sum_j scores[t, j] * y row of assignment (t, j) read from its owner's buffer)."""
    _cuda(indices, inv_perm, offsets, dst_row0, scores, out)
    T, k = scores.shape
    if out is None:
        out = torch.empty((T, hidden), dtype=torch.bfloat16, device=scores.device)
    L.check(L.lib().b200_ep_combine(_ctx(ctx), _ptr_array(peer_y), L.ptr(indices), L.ptr(inv_perm), L.ptr(offsets),
                                    L.ptr(dst_row0), L.ptr(scores), T, k, hidden, n_experts, len(peer_y), capacity_rows,
                                    L.ptr(out), L.stream_ptr()))
    return out


def moe_permute_static(indices, n_experts):
    """moe_permute without any device allocation by the library (no context either): the scratch is
    a fixed array inside libb200moe.so.  For callers whose memory pool owns the whole device or whose
    token loop must not meet cudaMalloc's device-wide synchronisation.  The outputs are allocated
    HERE by torch for convenience; a caller that cannot allocate passes its own buffers to the C
    entry point `b200_moe_permute_static`.  Limit: ceil(n/1024) * n_experts <= 65536."""
    _cuda(indices)
    n = indices.numel()
    dev = indices.device
    perm = torch.empty(n, dtype=torch.int32, device=dev)
    inv = torch.empty(n, dtype=torch.int32, device=dev)
    counts = torch.empty(n_experts, dtype=torch.int32, device=dev)
    offsets = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    moe_permute_static_into(indices, n_experts, perm, inv, counts, offsets)
    return perm, inv, counts, offsets


def moe_permute_static_into(indices, n_experts, perm, inv, counts, offsets):
    """The C entry point itself, on caller-provided buffers: nothing is allocated."""
    L.check(L.lib().b200_moe_permute_static(L.ptr(indices), indices.numel(), n_experts, L.ptr(perm), L.ptr(inv),
                                            L.ptr(counts), L.ptr(offsets), L.stream_ptr()))
