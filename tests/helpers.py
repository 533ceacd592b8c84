"""Shared builders and comparators for the parity tests."""

from __future__ import annotations

import ctypes

import torch


def f32(x: float) -> float:
    """Round a Python float through float32 (hyper-parameters live in fp32 vectors)."""
    return torch.tensor(x, dtype=torch.float32).item()


def bits_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    a = a.detach().cpu().contiguous()
    b = b.detach().cpu().contiguous()
    return a.shape == b.shape and bool(torch.equal(a.view(torch.int32), b.view(torch.int32)))


def assert_bits_equal(name: str, got: torch.Tensor, want: torch.Tensor) -> None:
    if not bits_equal(got, want):
        g, w = got.detach().cpu().float(), want.detach().cpu().float()
        n = int((g.contiguous().view(torch.int32) != w.contiguous().view(torch.int32)).sum())
        diff = (g - w).abs().max().item() if g.shape == w.shape else float("nan")
        raise AssertionError(
            f"{name} is not bit-identical: {n}/{g.numel()} elements differ, max abs diff {diff:.3e}"
        )


def full(n: int, value: float, device) -> torch.Tensor:
    return torch.full((n,), value, dtype=torch.float32, device=device)


def randn(gen: torch.Generator, *shape, device="cpu", scale: float = 1.0) -> torch.Tensor:
    """Seeded on the CPU generator so CPU and CUDA runs see the same numbers."""
    return (torch.randn(*shape, generator=gen) * scale).to(device)


def strided_like(t: torch.Tensor) -> torch.Tensor:
    """Same values in a transposed allocation: shape (R, T), strides (1, R)."""
    out = torch.empty(t.shape[1], t.shape[0], dtype=t.dtype, device=t.device).t()
    out.copy_(t)
    return out


def device_pows(beta1: torch.Tensor, beta2: torch.Tensor, steps: torch.Tensor) -> torch.Tensor:
    """(R, 2) = [beta1^step, beta2^step] computed by the GPU's powf, returned on the CPU."""
    import probe as _probe   # tests/probe: the run-time-mask build of the element math

    probe = _probe.lib()
    dev = torch.device("cuda")
    base = torch.stack([beta1, beta2], dim=1).to(dev, torch.float32).contiguous()
    expo = torch.stack([steps, steps], dim=1).to(dev, torch.float32).contiguous()
    out = torch.empty_like(base)
    rc = probe.cb200_probe_powf(base.data_ptr(), expo.data_ptr(), out.data_ptr(), base.numel(),
                                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    return out.cpu()
