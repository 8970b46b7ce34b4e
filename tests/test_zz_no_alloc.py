"""The allocation-free unique-map entry point, for callers that cannot call cudaMalloc (a runtime that owns all device
memory, a plugin handed only its input and output buffers): same output as the entry point with caller-owned scratch.

Collected last on purpose: a run that stops at the first failure has then already run every other test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_workspace_entry_twice(capi, cuda_device):
    rng = np.random.default_rng(77)
    domain = 1_000_000
    for call, n in enumerate((40_000, 25_000)):  # two calls in a row: the second must not see the first call's bits
        ids_np = rng.integers(0, domain, n)
        ids = torch.from_numpy(ids_np).to(cuda_device)
        ref_u, ref_inv, ref_cnt = capi.unique_bitmap(ids, domain)
        # every buffer is made by the caller beforehand; the call itself allocates nothing
        u = torch.full((n,), -7, dtype=torch.int64, device=cuda_device)
        inv = torch.full((n,), -7, dtype=torch.int64, device=cuda_device)
        cnt = torch.full((2,), -7, dtype=torch.int32, device=cuda_device)
        if call == 0:  # warm-up: the first call on a device looks up the scratch array's address (and loads the kernels)
            capi.unique_bitmap_static(ids, domain, u, inv, cnt)
        torch.cuda.synchronize()
        # free bytes as the driver counts them: a cudaMalloc inside the library (which links its own static runtime and is
        # invisible to torch's allocator statistics) would lower it
        free_before = torch.cuda.mem_get_info(cuda_device)[0]
        before = torch.cuda.memory_allocated(cuda_device)
        capi.unique_bitmap_static(ids, domain, u, inv, cnt)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(cuda_device) == before
        assert torch.cuda.mem_get_info(cuda_device)[0] == free_before
        c = int(ref_cnt[0])
        assert cnt.cpu().tolist() == [c, 0] and ref_cnt.cpu().tolist() == [c, 0]
        assert torch.equal(u[:c], ref_u[:c]) and torch.equal(inv, ref_inv)  # integers: exact
        assert np.array_equal(u[:c].cpu().numpy(), np.unique(ids_np))


def test_static_scratch_rejects_oversized_domain(capi, cuda_device):
    ids = torch.zeros(4, dtype=torch.int64, device=cuda_device)
    out = torch.zeros(4, dtype=torch.int64, device=cuda_device)
    cnt = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    with pytest.raises(capi.Ge2Error, match="unsupported"):
        capi.unique_bitmap_static(ids, capi.UNIQUE_STATIC_MAX_DOMAIN + 1, out, out.clone(), cnt)
    capi.unique_bitmap_static(ids, capi.UNIQUE_STATIC_MAX_DOMAIN, out, out.clone(), cnt)  # the limit itself is accepted
    torch.cuda.synchronize()
    assert cnt.cpu().tolist() == [1, 0]
