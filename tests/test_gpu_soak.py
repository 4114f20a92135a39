"""Randomised soak of the public op: forward and backward on random shapes, dtypes and masks (block
masks shared or per head, causal or not, empty rows and columns; dense masks applied element by
element) against the dense fp32 masked softmax of kernel-test.py:37-40 computed by torch on the GPU.
Seeded; each test keeps drawing cases for a fixed number of seconds.
Tolerances (stated by the task): max-abs 2e-2 on O, 5e-2 on dQ, dK, dV."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu
SECONDS = 8.0


def _reference(q, k, v, keep, scale, do):
    q, k, v = (t.float().detach().requires_grad_(True) for t in (q, k, v))
    s = ((q @ k.transpose(-1, -2)) * scale).masked_fill(~keep, float("-inf"))
    p = torch.nan_to_num(torch.softmax(s, -1), nan=0.0)   # rows with nothing kept: zeros
    o = p @ v
    o.backward(do.float())
    return o, q.grad, k.grad, v.grad


def _check(q, k, v, do, mask, keep, what):
    from fa2_custom_mask import flash_attention_custom_mask
    qc, kc, vc = (t.clone().requires_grad_(True) for t in (q, k, v))
    o = flash_attention_custom_mask(qc, kc, vc, mask, 0.125)
    o.backward(do)
    again = flash_attention_custom_mask(q, k, v, mask, 0.125)
    assert torch.equal(o.detach(), again), f"run-to-run difference: {what}"
    ro, rq, rk, rv = _reference(q, k, v, keep, 0.125, do)
    assert (o.detach().float() - ro).abs().max().item() <= 2e-2, what
    for name, got, ref in (("dq", qc.grad, rq), ("dk", kc.grad, rk), ("dv", vc.grad, rv)):
        assert (got.float() - ref).abs().max().item() <= 5e-2, (name, what)


def _draws(seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    ri = lambda a, b: int(torch.randint(a, b, (1,), generator=g, device="cuda"))
    rf = lambda: float(torch.rand(1, generator=g, device="cuda"))
    return g, ri, rf


def test_random_block_masks(lib):
    g, ri, rf = _draws(101)
    t0, n = time.time(), 0
    while time.time() - t0 < SECONDS:
        B, H, nb = ri(1, 3), ri(1, 9), ri(1, 81)
        N = nb * 64
        dtype = torch.float16 if ri(0, 2) else torch.bfloat16
        q, k, v, do = (torch.randn(B, H, N, 64, generator=g, device="cuda").to(dtype) for _ in range(4))
        shape = (1, 1, nb, nb) if ri(0, 3) == 0 else (B, H, nb, nb)
        blk = torch.rand(shape, generator=g, device="cuda") < rf() ** 2
        if ri(0, 2):
            blk |= torch.eye(nb, dtype=torch.bool, device="cuda")
        if ri(0, 3) == 0:
            blk = torch.tril(blk)
        keep = blk.expand(B, H, nb, nb).repeat_interleave(64, -2).repeat_interleave(64, -1)
        _check(q, k, v, do, blk, keep, (B, H, N, dtype, tuple(shape)))
        n += 1
    assert n >= 20


def test_random_dense_masks(lib):
    g, ri, rf = _draws(202)
    t0, n = time.time(), 0
    while time.time() - t0 < SECONDS:
        B, H, nb = ri(1, 3), ri(1, 5), ri(1, 25)
        N = nb * 64
        dtype = torch.float16 if ri(0, 2) else torch.bfloat16
        q, k, v, do = (torch.randn(B, H, N, 64, generator=g, device="cuda").to(dtype) for _ in range(4))
        blk = torch.rand(B, H, nb, nb, generator=g, device="cuda") < rf()
        keep = blk.repeat_interleave(64, -2).repeat_interleave(64, -1)
        kind = ri(0, 3)
        if kind == 0:
            keep = keep & (torch.rand(B, H, N, N, generator=g, device="cuda") < 0.7)
        elif kind == 1:
            keep = torch.tril(keep | torch.eye(N, dtype=torch.bool, device="cuda"))
        _check(q, k, v, do, keep, keep, (B, H, N, dtype, kind))
        n += 1
    assert n >= 20
