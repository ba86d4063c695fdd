"""CPU: pins the oracle with the relations the reference's own tests hold for this path.

The reference has no golden vectors here (its numeric constants need MLX's RNG); what its tests
pin are shapes, error bounds and equalities between two routes through the library.  Each test
below replays one of them on the oracle (deterministic inputs where the reference's are).
"""
import numpy as np
import pytest


def test_quantize_dequantize_reference_case(O):
    # mlx-rs/src/ops/quantization.rs:297-315: x[r, c] = c, 128 x 512, group 128, bits 2/4/8
    x = np.ones((128, 1), np.float32) * np.arange(512, dtype=np.float32)[None]
    for bits in (2, 4, 8):
        epi = 32 // bits
        wq, s, b = O.quantize(x, 128, bits, bf16_params=False)
        assert wq.shape == (128, 512 // epi) and s.shape == (128, 4) and b.shape == (128, 4)
        xh = O.dequantize(wq, s, b, 128, bits)
        assert np.abs(x - xh).max() <= 127.0 / (1 << bits)


def test_quantize_packing_and_edges(O):
    # element i of a word sits in bits [bits*i, bits*i+bits); the larger-magnitude extreme is exact
    w = np.linspace(-1.0, 0.5, 64, dtype=np.float32)[None]
    wq, s, b = O.quantize(w, 64, 4, bf16_params=False)
    codes = [(int(wq[0, i // 8]) >> (4 * (i % 8))) & 15 for i in range(64)]
    assert codes[0] == 0 and codes[-1] == 15 and codes == sorted(codes)
    wh = O.dequantize(wq, s, b, 64, 4)
    assert wh[0, 0] == w[0, 0]                      # |min| > |max| -> min is representable exactly
    assert np.abs(wh - w).max() <= abs(s[0, 0]) / 2 * 1.0001
    w2 = -w                                          # mirrored: max is the exact edge, scale negative
    wq2, s2, b2 = O.quantize(w2, 64, 4, bf16_params=False)
    assert s2[0, 0] < 0 and O.dequantize(wq2, s2, b2, 64, 4)[0, 0] == w2[0, 0]
    z = np.zeros((2, 64), np.float32)                # constant group: no NaN, exact zero
    wqz, sz, bz = O.quantize(z, 64, 4)
    assert np.all(O.dequantize(wqz, sz, bz, 64, 4) == 0)


def test_quantized_matmul_vs_dequantized(O):
    # mlx-rs/src/ops/quantization.rs:317-342: transpose=false, with biases, < 1e-3
    rng = np.random.default_rng(0)
    m, n, k = 32, 128, 128
    x = (rng.standard_normal((m, k)) / np.sqrt(k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    wq, s, b = O.quantize(w, 64, 4, bf16_params=False)
    wh = O.dequantize(wq, s, b, 64, 4)
    assert np.abs(O.quantized_matmul(x, wq, s, b, False, 64, 4) - x @ wh).max() < 1e-3
    wq, s, b = O.quantize(w.T.copy(), 64, 4, bf16_params=False)
    wh = O.dequantize(wq, s, b, 64, 4)
    assert np.abs(O.quantized_matmul(x, wq, s, b, True, 64, 4) - x @ wh.T).max() < 1e-3


def test_gather_qmm_vs_gather_mm(O):
    # mlx-rs/src/ops/quantization.rs:344-423: both index cases, all_close 1e-4
    rng = np.random.default_rng(0)
    m, n, k = 32, 64, 64
    w = rng.standard_normal((3, n, k)).astype(np.float32)
    wq, s, b = O.quantize(w, 64, 4, bf16_params=False)
    wh_t = np.swapaxes(O.dequantize(wq, s, b, 64, 4), -1, -2).copy()
    rhs = np.array([2, 1], np.uint32)
    for bx, lhs in ((1, np.array([0], np.uint32)), (5, np.array([0, 2], np.uint32))):
        x = rng.standard_normal((bx, m, k)).astype(np.float32)
        lhs_b = np.broadcast_to(lhs, rhs.shape).copy()
        c1 = O.gather_mm(x, wh_t, lhs_b, rhs)
        c2 = O.gather_qmm(x, wq, s, b, lhs_b, rhs, True, 64, 4)
        assert c1.shape == (2, m, n)
        assert np.allclose(c1, c2, rtol=1e-4, atol=1e-4)


def test_gather_mm_vs_take_matmul(O):
    # mlx-rs/src/ops/arithmetic.rs:3140-3238, including the sorted rhs case [100,1,100] x [8,100,100]
    rng = np.random.default_rng(1)
    a = rng.standard_normal((4, 5, 7)).astype(np.float32)
    b = rng.standard_normal((3, 7, 6)).astype(np.float32)
    lhs, rhs = np.array([3, 0, 0, 2], np.uint32), np.array([1, 2, 0, 0], np.uint32)
    assert np.allclose(O.gather_mm(a, b, lhs, rhs), a[lhs] @ b[rhs], atol=1e-5)
    a = rng.standard_normal((100, 1, 100)).astype(np.float32)
    b = rng.standard_normal((8, 100, 100)).astype(np.float32)
    rhs = np.sort(rng.integers(0, 8, 100)).astype(np.uint32)
    assert np.allclose(O.gather_mm(a, b, None, rhs), a @ b[rhs], atol=1e-4)


def test_sort_ops_canonical_rules(O):
    keys = np.array([[3, 1, 3, 0, 1, 1]], np.uint32)
    assert O.argsort(keys).tolist() == [[3, 1, 4, 5, 0, 2]]          # stable
    a = np.array([[0.5, 0.25, 0.5, 0.125]], np.float32)
    part = O.argpartition(-a, 1)
    assert part[0, :2].tolist() == [0, 2]                              # (value desc, index asc)
    assert O.take_along_axis(a, part[:, :2]).tolist() == [[0.5, 0.5]]
    with pytest.raises(IndexError):
        O.take_along_axis(a, np.array([[4]], np.uint32))


def test_f64_to_bf16_single_rounding(O):
    # a value that double rounding (f64 -> f32 -> bf16) gets wrong: just above a bf16 midpoint
    mid = np.float64(1.0 + 2.0 ** -8)           # midpoint between bf16(1.0) and bf16(1.0078125)
    above = mid + 2.0 ** -40                     # rounds to the midpoint in f32, then ties-to-even -> 1.0
    assert O.f64_to_bf16(np.array([above]))[0] == np.float32(1.0078125)
    assert O.f64_to_bf16(np.array([mid]))[0] == np.float32(1.0)
    assert O.f64_to_bf16(np.array([-above]))[0] == np.float32(-1.0078125)


def test_router_modes_and_ties(O):
    rng = np.random.default_rng(3)
    T, H, E, k = 33, 128, 16, 4
    x = O.round_bf16(rng.standard_normal((T, H)).astype(np.float32))
    wr = O.round_bf16((rng.standard_normal((E, H)) * 0.05).astype(np.float32))
    wr[5] = wr[2]                                # exact tie between experts 2 and 5
    idx, sc, lg = O.router(x, wr, k, 0, True, return_logits=True)
    exact = O.round_bf16(x.astype(np.float64) @ wr.astype(np.float64).T)
    assert np.array_equal(lg, O.f64_to_bf16(x.astype(np.float64) @ wr.astype(np.float64).T)) and exact.shape == lg.shape
    p = O.f64_to_bf16(O.softmax(lg))
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-p[t, e], e))[:k]
        assert idx[t].tolist() == order
        if 2 in order or 5 in order:
            assert (2 in order) or (5 not in order)   # the lower index wins a tie
    assert np.allclose(sc.sum(-1), 1.0, atol=2e-2)
    idx1, sc1 = O.router(x, wr, k, 1, False)
    for t in range(T):
        assert idx1[t].tolist() == sorted(range(E), key=lambda e: (-lg[t, e], e))[:k]
    sel = np.take_along_axis(lg, idx1.astype(np.int64), -1).astype(np.float64)
    ref = np.exp(sel - sel.max(-1, keepdims=True))
    assert np.array_equal(sc1, O.f64_to_bf16(ref / ref.sum(-1, keepdims=True)))


def test_permute_is_stable_argsort(O):
    rng = np.random.default_rng(4)
    for n, E in ((0, 4), (1, 1), (7, 3), (4096, 128), (5000, 8)):
        idx = rng.integers(0, E, n).astype(np.uint32)
        perm, inv, counts, offsets = O.permute(idx, E)
        assert np.array_equal(perm, np.argsort(idx, kind="stable").astype(np.uint32))
        assert np.array_equal(inv[perm], np.arange(n, dtype=np.uint32))
        assert np.array_equal(counts, np.bincount(idx, minlength=E).astype(np.uint32))
        assert offsets[0] == 0 and np.array_equal(np.diff(offsets.astype(np.int64)), counts)
    with pytest.raises(IndexError):
        O.permute(np.array([0, 9], np.uint32), 4)


def test_switch_glu_equals_op_composition(O):
    # the block restated op by op with the reference's ops (sorted gather_qmm route) equals the fused oracle
    from tests.helpers import make_block
    blk = make_block(T=9, H=128, E=4, I=64, k=2, seed=5)
    x, k = blk["x"], blk["k"]
    idx, sc = O.router(x, blk["wr"], k)
    flat = idx.reshape(-1)
    order = O.argsort(flat[None])[0]
    inv = O.argsort(order[None])[0]
    xs = x[order // k][:, None, :]
    es = flat[order]
    g = O.gather_qmm(xs, *blk["gate"], None, es)
    u = O.gather_qmm(xs, *blk["up"], None, es)
    h = O.round_bf16(g / (1 + np.exp(-g)) * u)
    y = O.gather_qmm(h, *blk["down"], None, es)[inv].reshape(9, k, -1)
    out = O.round_bf16((y * sc[..., None]).sum(-2))
    fused = O.moe_block(x, blk["wr"], blk["gate"], blk["up"], blk["down"], k)
    assert np.array_equal(fused["idx"], idx) and np.array_equal(fused["perm"], order)
    assert np.abs(out - fused["out"]).max() <= 1e-2 * np.abs(out).max()
    yk = O.switch_glu(x, idx, blk["gate"], blk["up"], blk["down"])
    assert yk.shape == (9, k, 128) and np.abs(yk - O.round_bf16(y)).max() <= 1e-2 * np.abs(y).max()


def test_rms_norm(O):
    rng = np.random.default_rng(6)
    x = rng.standard_normal((5, 64)).astype(np.float32)
    w = rng.standard_normal(64).astype(np.float32)
    ref = w * x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6)
    assert np.allclose(O.rms_norm(x, w, 1e-6), ref, atol=1e-5)
