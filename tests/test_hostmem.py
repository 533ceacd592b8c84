"""Best-effort NUMA placement of pinned memory: the policy call must never break an allocation."""

import pytest
import torch

from churten_b200 import hostmem


def test_policy_is_restored_and_failures_are_silent():
    with hostmem.prefer_node_of(0) as node:
        x = torch.empty(1024)
    assert node is None or isinstance(node, int)
    assert x.numel() == 1024
    # a node that does not exist is refused by the kernel, quietly
    assert hostmem._set_mempolicy(hostmem._MPOL_PREFERRED, 4000) in (False, True)
    assert hostmem._set_mempolicy(hostmem._MPOL_DEFAULT, None) in (False, True)
    info = hostmem.describe(0)
    assert set(info) == {"gpu_numa_node", "host_numa_nodes", "cpus_allowed"}


@pytest.mark.gpu
def test_pinned_near_gives_usable_pinned_memory(cuda):
    host = hostmem.pinned_near(cuda, (256, 33), torch.bfloat16)
    assert host.is_pinned() and host.shape == (256, 33) and host.dtype is torch.bfloat16
    src = torch.randn(256, 33, device=cuda).bfloat16()
    host.copy_(src, non_blocking=True)
    torch.cuda.synchronize()
    assert torch.equal(host, src.cpu())


@pytest.mark.gpu
def test_write_combined_staging_is_pinned_and_feeds_the_device(cuda):
    staging = hostmem.pinned_write_combined(cuda, (5, 7), torch.float32)
    assert staging.shape == (5, 7) and staging.is_pinned()
    values = torch.arange(35, dtype=torch.float32).reshape(5, 7)
    staging.copy_(values)                       # the host only writes it
    on_device = torch.empty(5, 7, device=cuda)
    on_device.copy_(staging, non_blocking=True)
    torch.cuda.synchronize()
    assert torch.equal(on_device.cpu(), values)
