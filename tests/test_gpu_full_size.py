"""The five BASELINE.json configurations at FULL size on the GPU.

At these sizes the CPU oracle is too slow for the whole batch, so each case checks
  * 64 paths spread over the batch against the oracle (per-coefficient tolerance as elsewhere), and
  * size-independent properties on the whole batch:
      - Chen's identity: sig(path) = sig(first part) (x) sig(second part), evaluated for the
        first two levels of every path (cheap closed forms of the tensor product);
      - level 1 equals the total increment, level 2's symmetric part equals half its square;
      - backward: linearity in the seeds, zero column sums (translation invariance of the
        signature), and agreement with the oracle on the subset.
"""
import os

import numpy as np
import pytest
import torch

import pysiglib_b200 as psl
from conftest import assert_grad_parity, assert_sig_close
from oracle import oracle

pytestmark = pytest.mark.gpu

CONFIGS = {  # name: B, L, d, N, dtype, law, backward
    "C1": (32, 1000, 10, 5, torch.float64, "iid", False),
    "C2": (1024, 256, 2, 12, torch.float64, "brownian", False),
    "C3": (128, 1024, 5, 7, torch.float32, "brownian", False),
    "C4": (256, 2048, 8, 4, torch.float32, "brownian", True),
    "C5": (4096, 4096, 16, 4, torch.float32, "brownian", True),
}


def make(B, L, d, dtype, law, seed):
    gen = torch.Generator().manual_seed(seed)
    if law == "iid":
        return torch.randn((B, L, d), generator=gen, dtype=dtype)
    inc = torch.randn((B, L - 1, d), generator=gen, dtype=dtype) * (1.0 / L) ** 0.5
    path = torch.zeros((B, L, d), dtype=dtype)
    torch.cumsum(inc, dim=1, out=path[:, 1:])
    return path


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_full_size_config(name):
    B, L, d, N, dtype, law, backward = CONFIGS[name]
    f64 = dtype == torch.float64
    rtol = 1e-10 if f64 else 1e-5
    host = make(B, L, d, dtype, law, 7)
    x = host.cuda()
    s = psl.sig(x, N)
    assert s.shape == (B, sum(d ** k for k in range(1, N + 1)))

    # subset against the oracle: 64 paths spread over the batch (all of them when the batch is smaller)
    pick = sorted(set(np.linspace(0, B - 1, min(B, 64)).astype(int).tolist()))
    threads = os.cpu_count() or 4
    expect = oracle.sig(host[pick].numpy(), N, n_threads=threads)
    assert_sig_close(s[pick].cpu().numpy(), expect, d, N, rtol)

    # whole batch: level 1 = total increment; sym(level 2) = level1 (x) level1 / 2
    tol = 1e-9 if f64 else 2e-4
    total = x[:, -1] - x[:, 0]
    l1, l2 = s[:, :d], s[:, d:d + d * d].reshape(B, d, d)
    scale = total.abs().amax().item() + 1e-30
    assert (l1 - total).abs().max().item() <= tol * max(scale, 1.0)
    sym = 0.5 * (l2 + l2.transpose(1, 2))
    want = 0.5 * total[:, :, None] * total[:, None, :]
    assert (sym - want).abs().max().item() <= tol * max(want.abs().max().item(), 1.0)

    # whole batch: Chen's identity on levels 1 and 2 for a split in the middle
    m = L // 2
    a, b = psl.sig(x[:, :m + 1].contiguous(), N), psl.sig(x[:, m:].contiguous(), N)
    a1, b1 = a[:, :d], b[:, :d]
    a2, b2 = a[:, d:d + d * d].reshape(B, d, d), b[:, d:d + d * d].reshape(B, d, d)
    assert (l1 - (a1 + b1)).abs().max().item() <= tol * max(scale, 1.0)
    chen2 = a2 + b2 + a1[:, :, None] * b1[:, None, :]
    assert (l2 - chen2).abs().max().item() <= tol * max(l2.abs().max().item(), 1.0)

    if not backward:
        return
    gen = torch.Generator(device="cuda").manual_seed(11)
    s1 = torch.randn(s.shape, dtype=dtype, device="cuda", generator=gen)
    s2 = torch.randn(s.shape, dtype=dtype, device="cuda", generator=gen)
    g1 = psl.sig_backprop(x, s, s1, N)
    g2 = psl.sig_backprop(x, s, s2, N)
    g12 = psl.sig_backprop(x, s, 2.0 * s1 - 0.5 * s2, N)
    gscale = g12.abs().amax(dim=(1, 2), keepdim=True)
    assert ((g12 - (2.0 * g1 - 0.5 * g2)).abs() / gscale).max().item() <= 2e-4        # linear in the seeds
    assert (g1.sum(dim=1).abs() / g1.abs().amax(dim=(1, 2))[:, None]).max().item() <= 2e-3  # translation invariance
    p_np = host[pick].numpy()
    seeds_np = s1[pick].cpu().numpy()
    want = oracle.sig_backprop(p_np, expect, seeds_np, N, n_threads=threads)
    p64 = p_np.astype(np.float64)
    truth = oracle.sig_backprop(p64, oracle.sig(p64, N, n_threads=threads), seeds_np.astype(np.float64), N,
                                n_threads=threads)
    assert_grad_parity(g1[pick].cpu().numpy(), want, truth, rtol)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_batch_partitioner_on_two_devices():
    """Reference tests/test_cuda_horner.py:210-222 runs on cuda:0, cuda:1, cuda:0 in turn; here the
    sharded front-end splits one host batch over both devices and must agree with a single device."""
    path = make(37, 64, 4, torch.float32, "brownian", 3).numpy()
    one = psl.sig(path, 4)
    two = psl.sig_sharded(path, 4, devices=[0, 1])
    np.testing.assert_array_equal(one, two)
    seeds = np.ones_like(one)
    g1 = psl.sig_backprop(path, one, seeds, 4)
    g2 = psl.sig_backprop_sharded(path, one, seeds, 4, devices=[0, 1])
    np.testing.assert_allclose(g1, g2, rtol=1e-4, atol=1e-5)
    for dev in ("cuda:0", "cuda:1", "cuda:0"):
        t = torch.tensor(path, device=dev)
        np.testing.assert_array_equal(psl.sig(t, 4).cpu().numpy(), one)


def test_neighbour_operators_at_benchmark_signature_size():
    """sig_join, sig_combine, sig_to_log_sig and corrections on signatures of the C5 shape (d=16,
    degree 4, S=69 904): identities over the whole batch, the oracle on a few entries."""
    B, L, d, N = 700, 24, 16, 4
    path = make(B, L, d, torch.float32, "brownian", 21).cuda()
    s_full = psl.sig(path, N)
    # Chen: joining the two halves / appending the last increment gives the signature of the whole path
    cut = L // 2
    joined = psl.sig_combine(psl.sig(path[:, :cut + 1].contiguous(), N), psl.sig(path[:, cut:].contiguous(), N), d, N)
    assert_sig_close(joined.cpu().numpy(), s_full.cpu().numpy(), d, N, 2e-5)
    head = psl.sig(path[:, :-1].contiguous(), N)
    last = (path[:, -1] - path[:, -2]).contiguous()
    assert_sig_close(psl.sig_join(head, last, d, N).cpu().numpy(), s_full.cpu().numpy(), d, N, 2e-5)
    # Lyndon coordinates are a gather of the expanded logarithm; the logarithm of a straight segment is the segment
    log0 = psl.sig_to_log_sig(s_full, d, N, method=0)
    log1 = psl.sig_to_log_sig(s_full, d, N, method=1)
    idx = torch.tensor(oracle.lyndon_indices(d, N).astype(np.int64) - 1, device="cuda")
    assert torch.equal(log1, log0[:, idx])
    lin = psl.sig_to_log_sig(psl.linear_sig(last, d, N), d, N, method=0)
    assert torch.allclose(lin[:, :d], last, rtol=0, atol=0)
    assert float(lin[:, d:].abs().max()) <= 1e-6 * max(1.0, float(last.abs().max()) ** N)
    sub = [0, 1, B - 1]
    want = oracle.sig_to_log_sig(s_full[sub].cpu().numpy().astype(np.float64), d, N, method=1)
    got = log1[sub].cpu().numpy()
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()
    # zero corrections reproduce the plain signature (scratch is cut into two batch chunks at this size)
    zero = torch.zeros((d * d,), dtype=torch.float32, device="cuda")
    zero[0] = 1e-30  # non-empty, numerically nothing
    corrected = psl.sig(path[:, :6].contiguous(), N, correction=zero)
    assert_sig_close(corrected.cpu().numpy(), psl.sig(path[:, :6].contiguous(), N).cpu().numpy(), d, N, 2e-5)
    corr = (torch.randn((3, 5, d * d), generator=torch.Generator().manual_seed(3)) * 0.05).cuda()
    got = psl.sig(path[[0, 1, B - 1], :6].contiguous(), N, correction=corr).cpu().numpy()
    want = oracle.sig(path[[0, 1, B - 1], :6].cpu().numpy().astype(np.float64), N, correction=corr.cpu().numpy().astype(np.float64))
    assert_sig_close(got, want, d, N, 2e-5)
