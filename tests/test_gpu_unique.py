"""GPU parity of the bitmap unique-map (through the C ABI) against the oracle: bit-exact integers."""
import numpy as np
import pytest
import torch

import ge2_oracle as O
import workloads

pytestmark = pytest.mark.gpu


def run(capi, ids_np, domain, device):
    ids = torch.from_numpy(ids_np.astype(np.int64)).to(device)
    u, inv, cnt = capi.unique_bitmap(ids, domain)
    torch.cuda.synchronize()
    count, status = (int(x) for x in cnt.cpu())
    return u.cpu().numpy()[:count], inv.cpu().numpy(), count, status


@pytest.mark.parametrize("n,domain", [(1, 1), (1, 64), (10, 64), (1000, 65), (4096, 63), (22000, 14951), (40000, 1_000_000),
                                      (150000, 1_211_896), (65536, 65536), (70000, 65537)])
def test_matches_oracle(capi, cuda_device, n, domain):
    rng = np.random.default_rng(n * 31 + domain)
    ids = rng.integers(0, domain, n)
    u, inv, count, status = run(capi, ids, domain, cuda_device)
    ou, oinv, _ = O.unique_map_bitmap(ids, domain)
    assert status == 0 and count == ou.size
    assert np.array_equal(u, ou) and np.array_equal(inv, oinv)


def test_skewed_and_degenerate_inputs(capi, cuda_device):
    domain = 1_000_000
    rng = np.random.default_rng(3)
    for ids in (workloads.zipf_ids(rng, 40000, domain, 1.1), np.full(5000, 777_777), np.arange(domain - 3000, domain),
                np.array([0, domain - 1, 0, domain - 1, 63, 64, 65])):
        u, inv, count, status = run(capi, ids, domain, cuda_device)
        ou, oinv = O.unique_map_sort(ids)
        assert status == 0 and np.array_equal(u, ou) and np.array_equal(inv, oinv)


def test_empty_input(capi, cuda_device):
    ids = torch.empty(0, dtype=torch.int64, device=cuda_device)
    u, inv, cnt = capi.unique_bitmap(ids, 100)
    torch.cuda.synchronize()
    assert cnt.cpu().tolist() == [0, 0] and inv.numel() == 0


def test_out_of_range_sets_status_without_faulting(capi, cuda_device):
    ids = np.array([5, 99, 100, -1, 7, 5])
    u, inv, count, status = run(capi, ids, 100, cuda_device)
    assert status & 1
    assert inv[2] == -1 and inv[3] == -1  # the reference's inverse kernel writes -1 there too before falling back to sort
    assert u.tolist() == [5, 7, 99] and inv[[0, 1, 4, 5]].tolist() == [0, 2, 1, 0]


def test_large_domain_properties(capi, cuda_device):
    """Largest configuration: 600 000 ids over a 12.5 M-node domain; checked through properties and the sort restatement."""
    domain, n = 12_500_000, 600_000
    ids = workloads.zipf_ids(np.random.default_rng(8), n, domain, 1.1)
    u, inv, count, status = run(capi, ids, domain, cuda_device)
    assert status == 0 and np.all(np.diff(u) > 0) and np.array_equal(u[inv], ids)
    ou, oinv = O.unique_map_sort(ids)
    assert count == ou.size and np.array_equal(u, ou) and np.array_equal(inv, oinv)


def test_workspace_reuse_back_to_back(capi, cuda_device):
    """The caller-owned workspace is reused across calls; the second call must not see the first call's bits."""
    domain = 100_000
    ws = capi.unique_workspace(domain, cuda_device)
    rng = np.random.default_rng(4)
    for _ in range(3):
        ids_np = rng.integers(0, domain, 20000)
        ids = torch.from_numpy(ids_np).to(cuda_device)
        u, inv, cnt = capi.unique_bitmap(ids, domain, workspace=ws)
        torch.cuda.synchronize()
        ou, oinv = O.unique_map_sort(ids_np)
        c = int(cnt[0])
        assert c == ou.size and np.array_equal(u.cpu().numpy()[:c], ou) and np.array_equal(inv.cpu().numpy(), oinv)
