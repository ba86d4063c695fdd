"""GPU: the routed block through the C ABI against the CPU oracle.

Bars (BASELINE.json): top-k indices, permutation and per-expert counts bit-exact; layer output
max|delta| <= 2e-2 * rms(oracle output) with float32 accumulation.  The output bar is checked on
the float32 result the block produces right before its final rounding (aux `out_f32`) against the
oracle's float32 result, and the bf16 output must equal the rounding of that value exactly: one
bf16 ulp of an output of magnitude 8 rms is 6 % of rms, so no bf16 tensor can be compared at
2e-2 * rms directly."""
import numpy as np
import pytest
import torch

from tests.helpers import bf16_cuda, close_up_to_bf16_rounding, make_block, rel_err, to_device, u32

pytestmark = pytest.mark.gpu
TOL = 2e-2


def check_block(pkg, O, blk, mode=0, renorm=True):
    ref = O.moe_block(blk["x"], blk["wr"], blk["gate"], blk["up"], blk["down"], blk["k"], mode, renorm, blk["bias"],
                      64, blk["bits"])
    dev = to_device(pkg, blk, mode, renorm)
    out, aux = dev.forward(bf16_cuda(blk["x"]), return_aux=True)
    pkg.default_context().check()
    assert np.array_equal(u32(aux["indices"]), ref["idx"]), "top-k indices"
    assert np.array_equal(aux["scores"].float().cpu().numpy(), ref["scores"]), "scores"
    assert np.array_equal(u32(aux["perm"]), ref["perm"]), "perm"
    assert np.array_equal(u32(aux["inv_perm"]), ref["inv"]), "inv"
    assert np.array_equal(u32(aux["counts"]), ref["counts"]), "counts"
    assert np.array_equal(u32(aux["offsets"]), ref["offsets"]), "offsets"
    # the bar applies to the float32 result; the bf16 output must be exactly its rounding
    got32 = aux["out_f32"].cpu().numpy()
    err = rel_err(got32, ref["out_f32"])
    assert np.array_equal(out.float().cpu().numpy(), O.round_bf16(got32)), "bf16 output is not the rounding of out_f32"
    print(f"[parity] T={blk['T']} H={blk['H']} E={blk['E']} I={blk['I']} k={blk['k']} bits={blk['bits']} mode={mode}: "
          f"max|d|/rms = {err:.4f}")
    assert err <= TOL, f"max|d|/rms = {err}"
    return err, dev, ref


@pytest.mark.parametrize("T", [1, 2, 3, 7])
@pytest.mark.parametrize("E,k", [(2, 1), (2, 2), (8, 1), (8, 2)])
def test_tiny_exhaustive(pkg, O, T, E, k):
    check_block(pkg, O, make_block(T, 128, E, 64, k, seed=T * 10 + E + k))


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("T,k", [(1, 8), (5, 3), (8, 12)])
def test_handful_of_tokens_fused_tail(pkg, O, bits, T, k):
    """At most eight tokens: the gate/up CTAs prepare their own activation rows and the down projection finishes
    the block (routing weights and k-way sum in its epilogue).  K = 320 leaves a ragged last block of groups in
    both bit widths; k = 12 makes warps take a second expert slot."""
    check_block(pkg, O, make_block(T, 320, 16, 192, k, bits=bits, seed=T * 7 + k + bits))


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("T,H,E,I,k", [(40, 256, 8, 128, 2),      # 10 rows per expert: two 8-row passes
                                       (100, 512, 8, 320, 2),     # 25 rows per expert; I = 320 leaves a ragged group
                                       (64, 1024, 16, 256, 4)])   # K slices over several blocks
def test_resident_slice_variant(pkg, O, bits, T, H, E, I, k):
    """Register regime beyond a handful of tokens: the variant of the grouped product that copies a CTA's whole
    weight slice into shared memory (both bit widths, several passes per expert, per-expert records), next to
    shapes where only one of the two products can use it."""
    ctx = pkg.default_context()
    ctx.set_qmm_path(ctx.QMM_SMALL)
    try:
        check_block(pkg, O, make_block(T, H, E, I, k, bits=bits, seed=T + H + bits))
    finally:
        ctx.set_qmm_path(ctx.QMM_AUTO)


@pytest.fixture(scope="module")
def config0():
    """BASELINE.json configs[0]: hidden 2048, 128 experts, top-8 renormalised, inter 768, 4-bit, 64 tokens."""
    return make_block(64, 2048, 128, 768, 8, seed=0)


def test_config0_block(pkg, O, config0):
    err, dev, ref = check_block(pkg, O, config0)
    # the un-fused route through the op surface gives the same routing and, within tolerance, the same output
    x = bf16_cuda(config0["x"])
    idx, sc, lg = pkg.nn.router_topk(x, dev.gate_weight, 8, return_logits=True)
    assert np.array_equal(u32(idx), ref["idx"])
    p = pkg.ops.softmax_axis(lg, -1, True)
    neg = (-p.float()).bfloat16()
    part = pkg.ops.argpartition_axis(neg, 7, -1)[:, :8].contiguous()
    assert np.array_equal(u32(part), ref["idx"])       # argpartition(-p, k-1)[:, :k] is the same selection
    yk = dev.switch_mlp.forward(x, idx)
    ref_yk = O.switch_glu(config0["x"], ref["idx"], config0["gate"], config0["up"], config0["down"], round_out=False)
    assert close_up_to_bf16_rounding(yk.float().cpu().numpy(), ref_yk, TOL)


@pytest.mark.parametrize("T", [1, 4, 16])
def test_decode_sweep_first_generation_kernel(pkg, O, config0, T):
    ctx = pkg.default_context()
    ctx.set_qmm_path(ctx.QMM_SMALL)
    try:
        blk = dict(config0)
        blk["x"] = config0["x"][:T].copy()
        blk["T"] = T
        check_block(pkg, O, blk)
    finally:
        ctx.set_qmm_path(ctx.QMM_AUTO)


@pytest.mark.parametrize("T", [1, 4, 16])
def test_decode_sweep(pkg, O, config0, T):
    # BASELINE.json configs[1], decode points (64 is test_config0_block): same weights, fewer tokens
    blk = dict(config0)
    blk["x"] = config0["x"][:T].copy()
    blk["T"] = T
    check_block(pkg, O, blk)


@pytest.fixture(params=["small", "tensor_core"])
def qmm_path(request, pkg):
    """Runs a test once per grouped-product kernel (register-load mma.sync / tcgen05) and restores AUTO."""
    ctx = pkg.default_context()
    ctx.set_qmm_path(dict(small=ctx.QMM_SMALL, tensor_core=ctx.QMM_TENSOR_CORE)[request.param])
    yield request.param
    ctx.set_qmm_path(ctx.QMM_AUTO)


@pytest.mark.parametrize("T", [200, 1500])
def test_more_rows_per_expert(pkg, O, T, qmm_path):
    # experts own many rows: wide/multi-pass variant of the small kernel; ragged 128-row tiles of the tcgen05 kernel
    check_block(pkg, O, make_block(T, 256, 8, 128, 2, seed=T))


@pytest.mark.parametrize("bits", [4, 8])
def test_mixtral_style_skewed(pkg, O, bits, qmm_path):
    # BASELINE.json configs[4] scaled down: 8 experts, top-2, softmax over the selected logits,
    # Zipf(1.2) logit bias; ragged segments including empty experts
    blk = make_block(300, 512, 8, 1024, 2, bits=bits, seed=11, zipf_bias=True)
    err, dev, ref = check_block(pkg, O, blk, mode=1, renorm=False)
    assert ref["counts"].max() > 3 * max(1, ref["counts"].min())


def test_prefill_512_tokens_config0_shape(pkg, O, config0, qmm_path):
    # BASELINE.json configs[1] prefill point T=512 on the config-0 weights, both kernels
    blk = dict(config0)
    g = torch.Generator().manual_seed(7)
    blk["x"] = torch.randn(512, 2048, generator=g).bfloat16().float().numpy()
    blk["T"] = 512
    err, dev, ref = check_block(pkg, O, blk)
    yk = dev.switch_mlp.forward(bf16_cuda(blk["x"]), torch.from_numpy(ref["idx"].view(np.int32)).cuda())
    ref_yk = O.switch_glu(blk["x"], ref["idx"], blk["gate"], blk["up"], blk["down"], round_out=False)
    assert close_up_to_bf16_rounding(yk.float().cpu().numpy(), ref_yk, TOL)


def test_config3_shape_reduced_experts(pkg, O, qmm_path):
    # BASELINE.json configs[3] (Qwen3-235B-A22B layer: hidden 4096, inter 1536, top-8 renormalised, 4-bit)
    # with 16 of its 128 experts so that the CPU oracle finishes in seconds; 300 tokens
    check_block(pkg, O, make_block(300, 4096, 16, 1536, 8, seed=33))


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("T", [3, 400])
def test_config4_shape_reduced_experts(pkg, O, bits, T):
    # BASELINE.json configs[4] (Mixtral layer: hidden 4096, inter 14336, top-2 of 8, softmax over the
    # selected, Zipf(1.2) skew) with 4 experts; K = 14336 in the down projection exceeds what the
    # memory-bound kernels can stage, so both token counts run on the tensor-core kernel
    blk = make_block(T, 4096, 4, 14336, 2, bits=bits, seed=44 + T, zipf_bias=True)
    check_block(pkg, O, blk, mode=1, renorm=False)


def test_no_renorm_and_ties(pkg, O):
    blk = make_block(50, 256, 16, 128, 4, seed=21)
    blk["wr"][7] = blk["wr"][3]          # exact ties between two experts on every token
    blk["wr"][9] = blk["wr"][3]
    check_block(pkg, O, blk, mode=0, renorm=False)
    check_block(pkg, O, blk, mode=1, renorm=False)


def test_empty_input(pkg, O):
    blk = make_block(4, 128, 4, 64, 2, seed=1)
    dev = to_device(pkg, blk)
    out = dev.forward(torch.empty((0, 128), dtype=torch.bfloat16, device="cuda"))
    assert tuple(out.shape) == (0, 128)
    perm, inv, counts, offsets = pkg.ops.moe_permute(torch.empty(0, dtype=torch.int32, device="cuda"), 4)
    pkg.default_context().check()
    assert counts.sum().item() == 0 and offsets.tolist() == [0] * 5


@pytest.mark.parametrize("n,E", [(1, 1), (1000, 128), (1024, 7), (1025, 128), (65536, 128), (100003, 256), (32768, 8)])
def test_permute_bit_exact(pkg, O, n, E):
    rng = np.random.default_rng(n + E)
    p = rng.random(E) ** 3
    idx = rng.choice(E, size=n, p=p / p.sum()).astype(np.uint32)
    perm, inv, counts, offsets = pkg.ops.moe_permute(torch.from_numpy(idx.view(np.int32)).cuda(), E)
    pkg.default_context().check()
    rp, ri, rc, ro = O.permute(idx, E)
    assert np.array_equal(u32(perm), rp) and np.array_equal(u32(inv), ri)
    assert np.array_equal(u32(counts), rc) and np.array_equal(u32(offsets), ro)


def test_router_large_bit_exact(pkg, O):
    # prefill-sized router: all three logit-kernel tilings against the oracle
    rng = np.random.default_rng(5)
    H, E, k = 2048, 128, 8
    wr = O.round_bf16((rng.standard_normal((E, H)) * 0.02).astype(np.float32))
    for T in (3, 100, 1000, 1500, 6200):
        x = O.round_bf16(rng.standard_normal((T, H)).astype(np.float32))
        ridx, rsc, rlg = O.router(x, wr, k, return_logits=True)
        idx, sc, lg = pkg.nn.router_topk(bf16_cuda(x), bf16_cuda(wr), k, return_logits=True)
        assert np.array_equal(lg.float().cpu().numpy(), rlg)
        assert np.array_equal(u32(idx), ridx) and np.array_equal(sc.float().cpu().numpy(), rsc)


def test_bad_config_is_rejected(pkg):
    blk = make_block(4, 128, 4, 64, 2, seed=1)
    dev = to_device(pkg, blk)
    with pytest.raises(pkg.B200Error):
        dev.forward(torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda"))   # wrong hidden size
    with pytest.raises(pkg.B200Error):
        pkg.nn.router_topk(torch.zeros((4, 128), dtype=torch.bfloat16, device="cuda"),
                           torch.zeros((4, 128), dtype=torch.bfloat16, device="cuda"), 5)  # top_k > experts


def test_arena_growth_is_refused_during_stream_capture(pkg):
    """A fresh context has no scratch arena; a block forward inside a stream capture would have to allocate it
    (cudaMalloc + device synchronisation, illegal while capturing): the call fails cleanly, the capture survives,
    and after b200_ctx_reserve the same capture succeeds and replays the eager result."""
    blk = make_block(T=8, H=256, E=8, I=128, k=2, seed=4)
    ctx = pkg.Context()
    block = to_device(pkg, blk)
    block.ctx = block.switch_mlp.ctx = ctx
    x = bf16_cuda(blk["x"])
    s = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        g.capture_begin()
        try:
            with pytest.raises(pkg.B200Error, match="capture"):
                block.forward(x)
        finally:
            g.capture_end()
    torch.cuda.synchronize()
    ctx.reserve(block.config, 8)
    want = block.forward(x)
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2):
        got = block.forward(x)
    g2.replay()
    torch.cuda.synchronize()
    ctx.check()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_stack_of_blocks_with_norm_and_residual(pkg, O):
    # BASELINE.json configs[2] scaled down: 3 pre-RMSNorm (eps 1e-6, unit weight) MoE blocks with residuals
    T, H, E, I, k = 40, 256, 8, 128, 2
    blks = [make_block(T, H, E, I, k, seed=100 + l) for l in range(3)]
    h = blks[0]["x"].copy()
    for b in blks:                                   # oracle: bf16 tensor between ops, float32 inside
        normed = O.round_bf16(O.rms_norm(h, None, 1e-6))
        y = O.moe_block(normed, b["wr"], b["gate"], b["up"], b["down"], k)["out"]
        h = O.round_bf16(h + y)
    stack = pkg.nn.MoeStack([to_device(pkg, b) for b in blks], eps=1e-6)
    got = stack.forward(bf16_cuda(blks[0]["x"])).float().cpu().numpy()
    pkg.default_context().check()
    # a last-bit difference in one layer's output can flip a near-tie in the next layer's routing,
    # which changes that token's output discontinuously: compare token by token
    rms = np.sqrt((h.astype(np.float64) ** 2).mean())
    ok = np.all(np.abs(got - h) <= TOL * rms + 2.0 ** -7 * np.abs(h), axis=1)
    assert ok.mean() >= 0.9, f"only {ok.mean():.2f} of the tokens agree"


@pytest.mark.parametrize("T", [1, 5, 8, 40])
def test_prenorm_entry_point_equals_norm_then_block(pkg, T):
    """b200_moe_block_forward_prenorm against b200_add_rms_norm + b200_moe_block_forward, bit for bit, in the
    handful-of-tokens path and beyond it; with and without a residual and a norm weight."""
    blk = make_block(T, 256, 8, 128, 2, seed=300 + T)
    block = to_device(pkg, blk)
    g = torch.Generator().manual_seed(T)
    h = bf16_cuda(blk["x"])
    res = (torch.randn(T, 256, generator=g) * 0.5).bfloat16().cuda()
    w = (1.0 + 0.1 * torch.randn(256, generator=g)).bfloat16().cuda()
    for residual, weight in ((None, None), (res, None), (res, w)):
        if residual is None:
            s_want, normed = h, pkg.ops.rms_norm(h, weight, 1e-6)
        else:
            s_want, normed = pkg.ops.add_rms_norm(h, residual, weight, 1e-6)
        want = block.forward(normed)
        s_got, got = block.forward_prenorm(h, residual, weight, 1e-6)
        pkg.default_context().check()
        assert torch.equal(s_got.view(torch.int16), s_want.view(torch.int16))
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_host_pipeline_matches_direct_calls(pkg):
    """Five pipelined submits from pinned host buffers (depth 2: slots are reused) return exactly what
    block.forward returns for the same rows."""
    blk = make_block(T=300, H=256, E=8, I=128, k=2, seed=21)
    block = to_device(pkg, blk)
    dev = torch.device("cuda", 0)
    pipe = pkg.nn.HostPipeline(block, 300, 256, dev, depth=2)
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(300 - 17 * i, 256, generator=g).bfloat16().pin_memory() for i in range(5)]
    outs = [torch.empty_like(x).pin_memory() for x in xs]
    for x, o in zip(xs, outs):
        pipe.submit(x, o)
    pipe.drain()
    torch.cuda.synchronize()
    pkg.default_context().check()
    for x, o in zip(xs, outs):
        want = block.forward(x.to(dev)).cpu()
        assert torch.equal(o.view(torch.int16), want.view(torch.int16))


def test_full_size_block_properties(pkg, O, config0):
    """BASELINE.json configs[1] at its largest point (8192 tokens, 128 experts): the oracle cannot run the
    whole block in seconds, so parity is checked through properties that do not depend on size.
    (1) routing of ALL tokens bit-exact against the oracle's router; (2) perm is the stable sort of the
    flat expert list, inv its inverse, counts/offsets its histogram; (3) the bf16 output is exactly the
    rounding of the float32 output; (4) a token's output does not depend on the other tokens in the
    batch, so 96 sampled tokens must match the oracle's block on those tokens alone - this compares
    the tensor-core path at full size with the CPU restatement directly."""
    T, k, E = 8192, 8, 128
    g = torch.Generator().manual_seed(81)
    x = torch.randn(T, 2048, generator=g).bfloat16()
    blk = dict(config0)
    block = to_device(pkg, blk)
    out, aux = block.forward(x.cuda(), return_aux=True)
    pkg.default_context().check()
    xn = x.float().numpy()
    ridx, rsc = O.router(xn, blk["wr"], k)
    idx = u32(aux["indices"])
    assert np.array_equal(idx, ridx) and np.array_equal(aux["scores"].float().cpu().numpy(), rsc)
    flat = idx.reshape(-1)
    perm = u32(aux["perm"])
    assert np.array_equal(perm, np.argsort(flat, kind="stable").astype(np.uint32))
    inv = u32(aux["inv_perm"])
    assert np.array_equal(inv[perm], np.arange(T * k, dtype=np.uint32))
    counts = np.bincount(flat, minlength=E).astype(np.uint32)
    assert np.array_equal(u32(aux["counts"]), counts)
    assert np.array_equal(u32(aux["offsets"]), np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32))
    got32 = aux["out_f32"].cpu().numpy()
    assert np.array_equal(out.float().cpu().numpy(), O.round_bf16(got32))
    sample = np.sort(np.random.default_rng(3).choice(T, size=96, replace=False))
    ref = O.moe_block(xn[sample], blk["wr"], blk["gate"], blk["up"], blk["down"], k)
    assert np.array_equal(ref["idx"], idx[sample])
    rms = np.sqrt((ref["out_f32"].astype(np.float64) ** 2).mean())
    err = float(np.abs(got32[sample] - ref["out_f32"]).max() / rms)
    print(f"[parity] full size T={T}: max|d|/rms over 96 sampled tokens = {err:.4f}")
    assert err <= TOL


def _gpu_block(pkg, H, E, I, k, bits, seed, mode, renorm, zipf):
    """A full-size block whose weights are drawn and quantized on the GPU (the CUDA quantizer is bit-exact
    with the oracle's, tests/test_gpu_ops.py), plus the same packed weights as numpy for the oracle."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    lin, host = [], []
    for r, c in ((I, H), (I, H), (H, I)):
        parts = []
        for e0 in range(0, E, 16):
            w = (torch.randn(min(16, E - e0), r, c, generator=g, device="cuda", dtype=torch.float32) * 0.02).bfloat16()
            parts.append(pkg.ops.quantize(w, 64, bits))
            del w
        wq, sc, bi = (torch.cat([p_[i] for p_ in parts]) for i in range(3))
        lin.append(pkg.nn.QuantizedSwitchLinear(wq, sc, bi, 64, bits))
        host.append((wq.cpu().numpy().view(np.uint32), sc.float().cpu().numpy(), bi.float().cpu().numpy()))
    wr = (torch.randn(E, H, generator=g, device="cuda", dtype=torch.float32) * 0.02).bfloat16()
    bias = (-2.4 * np.log(np.arange(1, E + 1))).astype(np.float32) if zipf else None
    block = pkg.nn.MoeBlock(wr, pkg.nn.SwitchGlu(*lin), k, renorm, mode, torch.from_numpy(bias).cuda() if zipf else None)
    return block, wr.float().cpu().numpy(), host, bias


def _full_size_properties(pkg, O, T, H, E, I, k, bits, mode, renorm, zipf, seed, n_sample=64):
    """The size-independent properties of test_full_size_block_properties for any layer shape."""
    block, wr, host, bias = _gpu_block(pkg, H, E, I, k, bits, seed, mode, renorm, zipf)
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(T, H, generator=g).bfloat16()
    out, aux = block.forward(x.cuda(), return_aux=True)
    pkg.default_context().check()
    xn = x.float().numpy()
    ridx, rsc = O.router(xn, wr, k, mode, renorm, bias)
    idx = u32(aux["indices"])
    assert np.array_equal(idx, ridx), "top-k indices of all tokens"
    assert np.array_equal(aux["scores"].float().cpu().numpy(), rsc), "scores of all tokens"
    flat = idx.reshape(-1)
    perm = u32(aux["perm"])
    assert np.array_equal(perm, np.argsort(flat, kind="stable").astype(np.uint32))
    assert np.array_equal(u32(aux["inv_perm"])[perm], np.arange(T * k, dtype=np.uint32))
    counts = np.bincount(flat, minlength=E).astype(np.uint32)
    assert np.array_equal(u32(aux["counts"]), counts)
    assert np.array_equal(u32(aux["offsets"]), np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32))
    got32 = aux["out_f32"].cpu().numpy()
    assert np.array_equal(out.float().cpu().numpy(), O.round_bf16(got32))
    sample = np.sort(np.random.default_rng(3).choice(T, size=n_sample, replace=False))
    ref = O.moe_block(xn[sample], wr, host[0], host[1], host[2], k, mode, renorm, bias, 64, bits)
    assert np.array_equal(ref["idx"], idx[sample])
    rms = np.sqrt((ref["out_f32"].astype(np.float64) ** 2).mean())
    err = float(np.abs(got32[sample] - ref["out_f32"]).max() / rms)
    print(f"[parity] full size T={T} H={H} E={E} I={I} k={k} bits={bits}: max|d|/rms over {n_sample} sampled tokens = "
          f"{err:.4f}; largest expert share {counts.max() / counts.sum():.3f}")
    assert err <= TOL
    return counts


def test_full_size_config3(pkg, O):
    """BASELINE.json configs[3] at full size: Qwen3-235B-A22B layer (hidden 4096, 128 experts, top-8
    renormalised, inter 1536, 4-bit), 8192 tokens."""
    _full_size_properties(pkg, O, 8192, 4096, 128, 1536, 8, 4, 0, True, False, seed=303)


@pytest.mark.parametrize("bits", [4, 8])
def test_full_size_config4(pkg, O, bits):
    """BASELINE.json configs[4] at full size: Mixtral layer (hidden 4096, 8 experts, top-2 with softmax over
    the selected logits, inter 14336), 16384 tokens, Zipf(1.2)-skewed routing, 4- and 8-bit."""
    counts = _full_size_properties(pkg, O, 16384, 4096, 8, 14336, 2, bits, 1, False, True, seed=404 + bits)
    assert counts.max() > 3 * counts.min()     # the skew is real: the first expert owns several times the last one's rows


@pytest.mark.parametrize("T", [5, 700])
def test_all_tokens_to_the_same_experts(pkg, O, T):
    """Maximum skew: a logit bias sends every token to experts 2 and 5, so six of the eight experts are
    empty and two own T rows each (one long segment per kernel, empty segments around it)."""
    blk = make_block(T, 256, 8, 128, 2, seed=77)
    bias = np.full(8, -40.0, dtype=np.float32)
    bias[[2, 5]] = 40.0
    blk["bias"] = bias
    err, dev, ref = check_block(pkg, O, blk, mode=1, renorm=False)
    assert sorted(np.unique(ref["idx"]).tolist()) == [2, 5]
    assert ref["counts"][2] == T and ref["counts"][5] == T and ref["counts"].sum() == 2 * T
