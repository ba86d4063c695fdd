"""GPU: every op of the reference surface, through the C ABI, against the CPU oracle."""
import numpy as np
import pytest
import torch

from tests.helpers import bf16_cuda, close_up_to_bf16_rounding, rel_err, u32

pytestmark = pytest.mark.gpu


def np_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int32)).cuda()


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("gs", [32, 64, 128])
@pytest.mark.parametrize("bf16", [True, False])
def test_quantize_bit_exact(pkg, O, bits, gs, bf16):
    rng = np.random.default_rng(bits * 100 + gs)
    w = (rng.standard_normal((3, 37, 256)) * 0.02).astype(np.float32)
    w[0, 0, :gs] = 0.0           # constant group
    w[0, 1, :gs] = np.abs(w[0, 1, :gs])  # one-signed group
    if bf16:
        w = O.round_bf16(w)
    wq, s, b = O.quantize(w, gs, bits, bf16_params=bf16)
    wt = torch.from_numpy(w).cuda()
    dq, ds, db = pkg.ops.quantize(wt.bfloat16() if bf16 else wt, gs, bits)
    assert np.array_equal(u32(dq), wq)
    assert np.array_equal(ds.float().cpu().numpy(), s) and np.array_equal(db.float().cpu().numpy(), b)
    wh = O.dequantize(wq, s, b, gs, bits)
    dh = pkg.ops.dequantize(dq, ds, db, gs, bits).float().cpu().numpy()
    assert np.array_equal(dh, O.round_bf16(wh) if bf16 else wh)


def test_quantize_reference_case(pkg):
    # mlx-rs/src/ops/quantization.rs:297-315 through the CUDA path
    x = (torch.ones(128, 1) * torch.arange(512, dtype=torch.float32)[None]).cuda()
    for bits in (2, 4, 8):
        wq, s, b = pkg.ops.quantize(x, 128, bits)
        assert tuple(wq.shape) == (128, 512 * bits // 32) and tuple(s.shape) == (128, 4) == tuple(b.shape)
        xh = pkg.ops.dequantize(wq, s, b, 128, bits)
        assert (x - xh).abs().max().item() <= 127.0 / (1 << bits)


def test_quantize_rejects_bad_arguments(pkg):
    x = torch.zeros(4, 100, device="cuda")
    with pytest.raises(pkg.B200Error):
        pkg.ops.quantize(x, 64, 4)          # last axis not a multiple of the group size
    with pytest.raises(pkg.B200Error):
        pkg.ops.quantize(torch.zeros(4, 128, device="cuda"), 64, 3)
    with pytest.raises(pkg.B200Error):
        pkg.ops.quantize(torch.zeros(128, device="cuda"), 64, 4)   # 1-D input


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("shape", [(32, 128, 128), (1, 2048, 768), (7, 768, 2048), (100, 64, 40)])
def test_quantized_matmul_transposed(pkg, O, bits, shape):
    m, k, n = shape
    rng = np.random.default_rng(m + n)
    x = O.round_bf16((rng.standard_normal((m, k)) / np.sqrt(k)).astype(np.float32))
    w = O.round_bf16((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32))
    wq, s, b = O.quantize(w, 64, bits)
    ref = O.quantized_matmul(x, wq, s, b, True, 64, bits)
    got = pkg.ops.quantized_matmul(bf16_cuda(x), np_i32(wq), bf16_cuda(s), bf16_cuda(b), True, 64, bits)
    pkg.default_context().check()
    assert tuple(got.shape) == (m, n)
    assert rel_err(got.float().cpu().numpy(), ref) <= 2e-2   # one bf16 rounding of the output


def test_quantized_matmul_reference_case(pkg, O):
    # mlx-rs/src/ops/quantization.rs:317-342 (transpose = false): equals x @ dequantize(w)
    rng = np.random.default_rng(0)
    m, n, k = 32, 128, 128
    x = O.round_bf16((rng.standard_normal((m, k)) / np.sqrt(k)).astype(np.float32))
    w = O.round_bf16((rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32))
    wq, s, b = pkg.ops.quantize(bf16_cuda(w), 64, 4)
    wh = pkg.ops.dequantize(wq, s, b, 64, 4).float().cpu().numpy()
    got = pkg.ops.quantized_matmul(bf16_cuda(x), wq, s, b, False, 64, 4).float().cpu().numpy()
    assert np.abs(got - x @ wh).max() < 1e-2
    ref = O.quantized_matmul(x, u32(wq), s.float().cpu().numpy(), b.float().cpu().numpy(), False, 64, 4)
    assert np.abs(got - ref).max() < 1e-2


@pytest.mark.parametrize("bits", [4, 8])
def test_gather_qmm_reference_cases(pkg, O, bits):
    # mlx-rs/src/ops/quantization.rs:344-423: gather_qmm == gather_mm on the dequantized, transposed weights
    rng = np.random.default_rng(0)
    m, n, k = 32, 64, 64
    w = O.round_bf16(rng.standard_normal((3, n, k)).astype(np.float32))
    wq, s, b = O.quantize(w, 64, bits)
    wh_t = np.swapaxes(O.dequantize(wq, s, b, 64, bits), -1, -2).copy()
    rhs = np.array([2, 1], np.uint32)
    for bx, lhs in ((1, [0, 0]), (5, [0, 2])):
        x = O.round_bf16(rng.standard_normal((bx, m, k)).astype(np.float32))
        lhs = np.array(lhs, np.uint32)
        c1 = O.gather_mm(x, wh_t, lhs, rhs)
        c2 = pkg.ops.gather_qmm(bf16_cuda(x), np_i32(wq), bf16_cuda(s), bf16_cuda(b), np_i32(lhs), np_i32(rhs), True,
                                64, bits)
        pkg.default_context().check()
        assert tuple(c2.shape) == (2, m, n)
        assert rel_err(c2.float().cpu().numpy(), c1) <= 2e-2


def test_gather_qmm_switch_linear_shape(pkg, O):
    # the shape a SwitchLinear issues: x [n,1,K], unsorted expert ids, no lhs
    rng = np.random.default_rng(2)
    n_idx, K, N, E = 300, 256, 192, 16
    x = O.round_bf16(rng.standard_normal((n_idx, 1, K)).astype(np.float32))
    w = O.round_bf16((rng.standard_normal((E, N, K)) * 0.05).astype(np.float32))
    wq, s, b = O.quantize(w)
    rhs = rng.integers(0, E, n_idx).astype(np.uint32)
    ref = O.gather_qmm(x, wq, s, b, None, rhs)
    got = pkg.ops.gather_qmm(bf16_cuda(x), np_i32(wq), bf16_cuda(s), bf16_cuda(b), None, np_i32(rhs))
    pkg.default_context().check()
    assert rel_err(got.float().cpu().numpy(), ref) <= 2e-2
    bad = rhs.copy()
    bad[3] = E + 2                      # out-of-range expert: reported at the next check, nothing written for it
    pkg.ops.gather_qmm(bf16_cuda(x), np_i32(wq), bf16_cuda(s), bf16_cuda(b), None, np_i32(bad))
    with pytest.raises(pkg.B200Error):
        pkg.default_context().check()
    pkg.default_context().check()       # the status word is cleared once reported
    # out-of-range batch index of x: reported the same way (the read is redirected, never out of bounds)
    xb = bf16_cuda(x[:4])
    lhs = np.array([0, 3, 9, 1], np.uint32)     # x has 4 batch entries
    pkg.ops.gather_qmm(xb, np_i32(wq), bf16_cuda(s), bf16_cuda(b), np_i32(lhs), np_i32(rhs[:4]))
    with pytest.raises(pkg.B200Error):
        pkg.default_context().check()
    pkg.default_context().check()


@pytest.mark.parametrize("cols", [8, 128, 200, 256])
def test_softmax_argpartition_take(pkg, O, cols):
    rng = np.random.default_rng(cols)
    a = O.round_bf16(rng.standard_normal((57, cols)).astype(np.float32) * 2)
    a[:, 3] = a[:, 1]                   # ties
    da = bf16_cuda(a)
    p = pkg.ops.softmax_axis(da, -1, True).float().cpu().numpy()
    assert np.array_equal(p, O.f64_to_bf16(O.softmax(a)))
    kth = min(7, cols - 1)
    part = pkg.ops.argpartition_axis(da, kth, -1)
    full = O.argpartition(a, kth)
    got = u32(part)
    assert np.array_equal(got[:, :kth + 1], full[:, :kth + 1])
    for r in range(a.shape[0]):
        assert sorted(got[r].tolist()) == list(range(cols))
        assert a[r, got[r, kth + 1:]].min(initial=np.inf) >= a[r, got[r, kth]]
    taken = pkg.ops.take_along_axis(da, part[:, :kth + 1].contiguous(), -1).float().cpu().numpy()
    assert np.array_equal(taken, O.take_along_axis(a, full[:, :kth + 1]))
    with pytest.raises(pkg.B200Error):
        pkg.ops.argpartition_axis(da, cols, -1)       # kth out of range (mlx-rs/src/ops/sort.rs:266-298)
    pkg.ops.take_along_axis(da, torch.full((57, 1), cols, dtype=torch.int32, device="cuda"), -1)
    with pytest.raises(pkg.B200Error):
        pkg.default_context().check()


def test_rms_norm_and_residual(pkg, O):
    rng = np.random.default_rng(9)
    x = O.round_bf16(rng.standard_normal((33, 2048)).astype(np.float32))
    r = O.round_bf16(rng.standard_normal((33, 2048)).astype(np.float32))
    w = O.round_bf16(rng.standard_normal(2048).astype(np.float32))
    def close(got, ref):   # one bf16 rounding of the output: half an ulp is 2^-9 relative
        return np.all(np.abs(got - ref) <= 2.0 ** -8 * np.abs(ref) + 1e-6)
    got = pkg.ops.rms_norm(bf16_cuda(x), bf16_cuda(w), 1e-6).float().cpu().numpy()
    assert close(got, O.rms_norm(x, w, 1e-6))
    got1 = pkg.ops.rms_norm(bf16_cuda(x), None, 1e-6).float().cpu().numpy()
    assert close(got1, O.rms_norm(x, None, 1e-6))
    s, n = pkg.ops.add_rms_norm(bf16_cuda(x), bf16_cuda(r), None, 1e-6)
    sref = O.round_bf16(x + r)
    assert np.array_equal(s.float().cpu().numpy(), sref)
    assert close(n.float().cpu().numpy(), O.rms_norm(sref, None, 1e-6))


def test_gather_mm_reference_cases(pkg, O):
    # mlx-rs/src/ops/arithmetic.rs:3140-3238: gather = take on the flattened batch + matmul; sorted rhs case
    rng = np.random.default_rng(5)
    a = O.round_bf16((rng.standard_normal((100, 1, 100)) / 10).astype(np.float32))
    b = O.round_bf16((rng.standard_normal((8, 100, 100)) / 10).astype(np.float32))
    rhs = np.sort(rng.integers(0, 8, size=100)).astype(np.uint32)
    ref = O.gather_mm(a, b, None, rhs)
    got = pkg.ops.gather_mm(bf16_cuda(a), bf16_cuda(b), None, torch.from_numpy(rhs.view(np.int32)).cuda())
    pkg.default_context().check()
    assert tuple(got.shape) == (100, 1, 100)
    assert close_up_to_bf16_rounding(got.float().cpu().numpy(), ref, 1e-3)
    # both index arrays, several rows per entry, ragged N
    a = O.round_bf16((rng.standard_normal((5, 11, 300)) / 10).astype(np.float32))
    b = O.round_bf16((rng.standard_normal((3, 300, 200)) / 10).astype(np.float32))
    lhs = rng.integers(0, 5, size=(4, 2)).astype(np.uint32)
    rhs = rng.integers(0, 3, size=(4, 2)).astype(np.uint32)
    ref = O.gather_mm(a, b, lhs, rhs)
    got = pkg.ops.gather_mm(bf16_cuda(a), bf16_cuda(b), torch.from_numpy(lhs.view(np.int32)).cuda(),
                            torch.from_numpy(rhs.view(np.int32)).cuda())
    pkg.default_context().check()
    assert tuple(got.shape) == (4, 2, 11, 200)
    assert close_up_to_bf16_rounding(got.float().cpu().numpy(), ref, 1e-3)
    with pytest.raises(pkg.B200Error):      # an index past the batch is reported, not read
        pkg.ops.gather_mm(bf16_cuda(a), bf16_cuda(b), None, torch.tensor([7, 0, 1, 2, 0], dtype=torch.int32).cuda())
        pkg.default_context().check()


def test_gather_mm_tensor_core_branch(pkg, O):
    """Enough rows for 128-row tiles: the product goes through the grouped tcgen05 kernel (rows sorted by matrix,
    un-quantised bf16 operands).  4096 gathered rows over 8 matrices, ragged N (not a multiple of the 256-column tile),
    skewed use of the matrices with one of them unused, both index arrays."""
    rng = np.random.default_rng(77)
    Ba, Bb, M, K, N, n_idx = 300, 8, 4, 512, 328, 1024
    a = O.round_bf16((rng.standard_normal((Ba, M, K)) / 8).astype(np.float32))
    b = O.round_bf16((rng.standard_normal((Bb, K, N)) / 8).astype(np.float32))
    lhs = rng.integers(0, Ba, size=n_idx).astype(np.uint32)
    p = np.array([0.4, 0.2, 0.0, 0.1, 0.1, 0.1, 0.05, 0.05])
    rhs = rng.choice(Bb, size=n_idx, p=p).astype(np.uint32)
    ref = O.gather_mm(a, b, lhs, rhs)
    ctx = pkg.default_context()
    before = ctx.launch_count()
    got = pkg.ops.gather_mm(bf16_cuda(a), bf16_cuda(b), torch.from_numpy(lhs.view(np.int32)).cuda(),
                            torch.from_numpy(rhs.view(np.int32)).cuda())
    ctx.check()
    assert ctx.launch_count() - before > 1, "expected the sorted tensor-core path, not the single CUDA-core launch"
    assert tuple(got.shape) == (n_idx, M, N)
    assert close_up_to_bf16_rounding(got.float().cpu().numpy(), ref, 1e-3)
    # only rhs indices: entry i of a with matrix rhs[i], 4 matrices x 256 rows
    a2 = O.round_bf16((rng.standard_normal((4, 256, 128)) / 8).astype(np.float32))
    b2 = O.round_bf16((rng.standard_normal((4, 128, 64)) / 8).astype(np.float32))
    got = pkg.ops.gather_mm(bf16_cuda(a2), bf16_cuda(b2), None, torch.tensor([3, 1, 0, 2], dtype=torch.int32).cuda())
    ctx.check()
    ref2 = np.stack([a2[i].astype(np.float64) @ b2[j].astype(np.float64) for i, j in enumerate([3, 1, 0, 2])])
    assert close_up_to_bf16_rounding(got.float().cpu().numpy(), ref2, 1e-3)
    with pytest.raises(pkg.B200Error):      # an index past the batch is reported on this path too
        pkg.ops.gather_mm(bf16_cuda(a), bf16_cuda(b), torch.from_numpy(lhs.view(np.int32)).cuda(),
                          torch.full((n_idx,), 8, dtype=torch.int32).cuda())
        ctx.check()


def f32_cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def test_reference_float32_cases(pkg, O):
    """The reference's own op tests use float32 arrays: quantized_matmul with transpose = false equals
    x @ dequantize(w) within 1e-3 (mlx-rs/src/ops/quantization.rs:317-342) and gather_qmm equals gather_mm on
    the dequantised, transposed weights within 1e-4 (:344-423)."""
    rng = np.random.default_rng(0)
    m, n, k = 32, 128, 128
    x = (rng.standard_normal((m, k)) / np.sqrt(k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    wq, s, b = pkg.ops.quantize(f32_cuda(w), 64, 4)
    assert s.dtype == torch.float32
    wh = pkg.ops.dequantize(wq, s, b, 64, 4).cpu().numpy()
    got = pkg.ops.quantized_matmul(f32_cuda(x), wq, s, b, False, 64, 4).cpu().numpy()
    assert np.abs(got - x @ wh).max() < 1e-3
    m, n, k = 32, 64, 64
    w3 = rng.standard_normal((3, n, k)).astype(np.float32)
    wq, s, b = O.quantize(w3, 64, 4, bf16_params=False)
    wh_t = np.swapaxes(O.dequantize(wq, s, b, 64, 4), -1, -2).copy()
    rhs = np.array([2, 1], np.uint32)
    for bx, lhs in ((1, [0, 0]), (5, [0, 2])):
        xx = rng.standard_normal((bx, m, k)).astype(np.float32)
        lhs = np.array(lhs, np.uint32)
        c1 = O.gather_mm(xx, wh_t, lhs, rhs)
        c2 = pkg.ops.gather_qmm(f32_cuda(xx), np_i32(wq), f32_cuda(s), f32_cuda(b), np_i32(lhs), np_i32(rhs), True, 64, 4)
        pkg.default_context().check()
        assert c2.dtype == torch.float32 and np.abs(c2.cpu().numpy() - c1).max() < 1e-4
    # float16 activations, group 32, 8 bits, and the transpose = false form of gather_qmm (w quantised along N)
    wk = rng.standard_normal((3, k, n)).astype(np.float32) * 0.1
    wq, s, b = O.quantize(wk, 32, 8, bf16_params=False)
    wh = O.dequantize(wq, s, b, 32, 8)
    xx = (rng.standard_normal((4, 8, k)) * 0.5).astype(np.float16)
    rhs = np.array([1, 0, 2, 2], np.uint32)
    ref = np.einsum("bmk,bkn->bmn", xx.astype(np.float32), wh[rhs].astype(np.float16).astype(np.float32))
    got = pkg.ops.gather_qmm(torch.from_numpy(xx).cuda(), np_i32(wq), torch.from_numpy(s.astype(np.float16)).cuda(),
                             torch.from_numpy(b.astype(np.float16)).cuda(), None, np_i32(rhs), False, 32, 8)
    pkg.default_context().check()
    assert got.dtype == torch.float16 and rel_err(got.float().cpu().numpy(), ref) <= 2e-2


@pytest.mark.parametrize("bits", [4, 8])
def test_ops_reach_the_tensor_core_kernel(pkg, O, bits):
    """quantized_matmul and gather_qmm with many rows per weight matrix (the dense quantised Linear, a SwitchLinear
    at prefill size) run the tcgen05 kernel; same bar as the block."""
    rng = np.random.default_rng(5 + bits)
    M, K, N, E = 900, 512, 768, 4
    x = O.round_bf16(rng.standard_normal((M, K)).astype(np.float32))
    w = O.round_bf16((rng.standard_normal((E, N, K)) * 0.05).astype(np.float32))
    wq, s, b = O.quantize(w, 64, bits)
    l0 = pkg.default_context().launch_count()
    got = pkg.ops.quantized_matmul(bf16_cuda(x), np_i32(wq[0]), bf16_cuda(s[0]), bf16_cuda(b[0]), True, 64, bits)
    assert pkg.default_context().launch_count() - l0 == 4      # segments, row tiles, row preparation, tcgen05 product
    ref = O.quantized_matmul(x, wq[0], s[0], b[0], True, 64, bits)
    assert close_up_to_bf16_rounding(got.float().cpu().numpy(), ref, 2e-2)
    rhs = rng.integers(0, E, M).astype(np.uint32)
    lhs = rng.permutation(M).astype(np.uint32)
    ref = O.gather_qmm(x[:, None, :], wq, s, b, lhs, rhs, True, 64, bits)
    got = pkg.ops.gather_qmm(bf16_cuda(x[:, None, :]), np_i32(wq), bf16_cuda(s), bf16_cuda(b), np_i32(lhs), np_i32(rhs),
                             True, 64, bits)
    pkg.default_context().check()
    assert close_up_to_bf16_rounding(got.float().cpu().numpy(), ref, 2e-2)


def test_argsort_take_topk_ops(pkg, O):
    rng = np.random.default_rng(8)
    keys = rng.integers(0, 128, (3, 5000)).astype(np.uint32)
    got = pkg.ops.argsort_axis(np_i32(keys), -1, 128)
    pkg.default_context().check()
    assert np.array_equal(u32(got), O.argsort(keys))
    x = O.round_bf16(rng.standard_normal((50, 64)).astype(np.float32))
    idx = rng.integers(0, 50, 200).astype(np.uint32)
    assert np.array_equal(pkg.ops.take_axis(bf16_cuda(x), np_i32(idx)).float().cpu().numpy(), x[idx])
    a = O.round_bf16(rng.standard_normal((37, 128)).astype(np.float32))
    a[:, 5] = a[:, 9]
    top = pkg.ops.topk_axis(bf16_cuda(a), 8).float().cpu().numpy()
    assert np.array_equal(top, np.sort(a, axis=-1)[:, -8:])
    with pytest.raises(pkg.B200Error):
        pkg.ops.topk_axis(bf16_cuda(a), 500)
