"""GPU: the allocation-free permutation entry point against the allocating one.

`b200_moe_permute_static` serves callers that must not cause a device allocation (their own pool
owns the device, or their token loop cannot take cudaMalloc's device-wide synchronisation): its
scratch is a fixed array inside the library.  The array keeps the previous call's contents, so the
test makes two calls in a row (a large problem, then a smaller one with other experts) and wants
both to equal the allocating entry point bit for bit.  Collected last on purpose.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _u32(t):
    return t.cpu().numpy().view(np.uint32)


def test_static_permute_matches_allocating_entry_point_twice(pkg, O):
    rng = np.random.default_rng(1234)
    cases = [(200_000, 128), (3_000, 16)]          # multi-chunk first, then fewer chunks and experts
    for n, E in cases:
        p = rng.random(E) ** 2
        idx = torch.from_numpy(rng.choice(E, size=n, p=p / p.sum()).astype(np.int32)).cuda()
        ref = pkg.ops.moe_permute(idx, E)
        # caller-owned outputs, poisoned so that anything left unwritten shows up
        perm = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        inv = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        counts = torch.full((E,), -1, dtype=torch.int32, device="cuda")
        offsets = torch.full((E + 1,), -1, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]     # the driver's view: sees any cudaMalloc, not only torch's
        pkg.ops.moe_permute_static_into(idx, E, perm, inv, counts, offsets)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] >= free_before, "the allocation-free entry point allocated device memory"
        for got, want in zip((perm, inv, counts, offsets), ref):
            assert np.array_equal(_u32(got), _u32(want))
        # and against the CPU restatement of the stable sort, not only against the other GPU entry point
        for got, want in zip((perm, inv, counts, offsets), O.permute(_u32(idx), E)):
            assert np.array_equal(_u32(got), want)
    # single-chunk path (one launch) after the multi-chunk ones
    idx = torch.from_numpy(rng.integers(0, 8, 700).astype(np.int32)).cuda()
    for got, want in zip(pkg.ops.moe_permute_static(idx, 8), pkg.ops.moe_permute(idx, 8)):
        assert np.array_equal(_u32(got), _u32(want))


def test_static_permute_limits(pkg, O):
    """The largest problem the fixed array admits (ceil(n/1024) * n_experts == 65536 exactly, 256 experts),
    and the empty one."""
    E, n = 256, 256 * 1024
    rng = np.random.default_rng(99)
    idx = torch.from_numpy(rng.integers(0, E, n).astype(np.int32)).cuda()
    for got, want in zip(pkg.ops.moe_permute_static(idx, E), O.permute(_u32(idx), E)):
        assert np.array_equal(_u32(got), want)
    empty = torch.empty(0, dtype=torch.int32, device="cuda")
    perm, inv, counts, offsets = pkg.ops.moe_permute_static(empty, 5)
    torch.cuda.synchronize()
    assert perm.numel() == 0 and counts.tolist() == [0] * 5 and offsets.tolist() == [0] * 6


def test_static_permute_rejects_oversized_problems(pkg):
    idx = torch.zeros(1024 * 300, dtype=torch.int32, device="cuda")      # 300 chunks x 256 experts > 65536
    with pytest.raises(pkg.B200Error, match="static scratch"):
        pkg.ops.moe_permute_static(idx, 256)
