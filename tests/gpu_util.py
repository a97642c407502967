"""Helpers of the GPU parity tests."""
import torch

from oracle import nha_oracle as orc

# bf16 inputs, fp32 accumulation, against the fp64 oracle: the reference's own "OK" bar
# (scripts/verify_opt_parity.py:753)
TOL_OUT = 2e-2
# gradients, per tensor
TOL_GRAD = 3e-2


def cuda(d):
    return {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in d.items()}


def err(a, b):
    return orc.rel_l2(a.detach().float().cpu(), b.detach().cpu())


def assert_close(got, want, tol, what):
    e = err(got, want)
    assert e == e and e <= tol, f'{what}: rel-L2 {e:.3e} > {tol:.1e}'
    return e
