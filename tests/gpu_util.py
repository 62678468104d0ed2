"""Helpers shared by the GPU parity tests."""
import torch

from quik_b200 import _lib


def dev():
    return torch.device("cuda:0")


def assert_device_clean():
    rc = _lib.device_status(clear=True)
    assert rc == 0, f"a bounded device wait ran out (status {rc})"


def make_indices(K, F, order="ascending", seed=0):
    g = torch.Generator().manual_seed(seed)
    fp = torch.randperm(K, generator=g)[:F]
    ints = torch.arange(K)
    ints = ints[~torch.isin(ints, fp)]
    if order == "ascending":
        fp = torch.sort(fp)[0]
    elif order == "shuffled":
        ints = ints[torch.randperm(ints.numel(), generator=g)]
    return ints, fp


def outlier_x(M, K, fp, dtype, seed=0):
    g = torch.Generator().manual_seed(seed + 1000)
    x = torch.randn(M, K, generator=g)
    if fp.numel():
        x[:, fp] *= 20
    return x.to(dtype)


def rel_rms_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / b.pow(2).mean().sqrt().clamp_min(1e-12)).item()
