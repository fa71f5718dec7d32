"""GPU tests of the runtime around the kernels: recovery from failed scratch allocations
(failures injected on the host, the GPU is never driven out of memory), the library's private
memory pool, the NaN / Inf flag raised by the forward sweep itself, every compiled register-tile
variant of a shape through the test hook that pins one, and device-mismatch rejection."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import cabi
from conftest import assert_grad_parity, assert_sig_close, brownian_paths
from oracle import oracle
from pysiglib_b200 import load_cusig

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _forward(path, degree, **kw):
    code, out = cabi.signature_cuda(path, degree, pad=2, **kw)
    return code, (out[:-2].reshape(path.shape[0], -1) if code == 0 else None)


def _backward(path, sig, derivs, degree, **kw):
    code, out = cabi.sig_backprop_cuda(path, sig, derivs, degree, pad=2, **kw)
    return code, (out[:-2].reshape(path.shape) if code == 0 else None)


@pytest.mark.parametrize("where", ["host", "device"])
@pytest.mark.parametrize("shape", [(9, 70, 8, 4), (5, 40, 19, 3)], ids=["tile", "generic"])
def test_failed_allocations_halve_the_batch_piece(where, shape):
    """The reference halves its batch chunk when cudaMalloc reports out-of-memory
    (siglib/cusig/cu_runtime_utils.h:212-235).  Here the failure is injected on the host: the
    next n scratch / staging requests of the library fail, the call must still succeed with the
    right numbers, and a failure that persists down to a single path surfaces as code 1."""
    B, L, d, N = shape
    path = brownian_paths(3, B, L, d, np.float32)
    expect = oracle.sig(path, N)
    seeds = np.random.default_rng(2).standard_normal(expect.shape).astype(np.float32)
    want = oracle.sig_backprop(path, expect, seeds, N)
    truth = oracle.sig_backprop(path.astype(np.float64), oracle.sig(path.astype(np.float64), N),
                                seeds.astype(np.float64), N)
    to = (lambda a: torch.tensor(a, device="cuda")) if where == "device" else (lambda a: a)
    back = (lambda t: t.cpu().numpy()) if where == "device" else (lambda a: a)
    p, s, g = to(path), to(expect), to(seeds)
    try:
        for failures in (1, 2, 3):
            load_cusig.inject_alloc_failures(failures)
            code, got = _backward(p, s, g, N)
            assert code == 0, load_cusig.last_error_message()
            assert_grad_parity(back(got), want, truth, 1e-5, "backward after %d failed allocations" % failures)
        load_cusig.inject_alloc_failures(0)
        code, got = _forward(p, N)
        assert code == 0
        assert_sig_close(back(got), expect, d, N, 1e-5)
        # every attempt fails: the piece shrinks to one path and the error is reported, not swallowed
        load_cusig.inject_alloc_failures(1000)
        code, _ = _backward(p, s, g, N)
        assert code == 1, (code, load_cusig.last_error_message())
    finally:
        load_cusig.inject_alloc_failures(0)
    code, got = _backward(p, s, g, N)  # and the library still works afterwards
    assert code == 0
    assert_grad_parity(back(got), want, truth, 1e-5)


def test_scratch_comes_from_a_private_pool():
    """Scratch and staging buffers come from a pool the library creates itself; the device's
    default stream-ordered pool (which the host application may use) keeps its settings."""
    from cuda.bindings import runtime as rt
    dev = torch.cuda.current_device()
    err, pool = rt.cudaDeviceGetDefaultMemPool(dev)
    assert int(err) == 0
    err, threshold_before = rt.cudaMemPoolGetAttribute(pool, rt.cudaMemPoolAttr.cudaMemPoolAttrReleaseThreshold)
    path = brownian_paths(1, 64, 200, 8, np.float32)
    sig = oracle.sig(path, 4)
    code, _ = _backward(path, sig, np.ones_like(sig), 4)  # host call: staging slots + scratch
    assert code == 0
    assert load_cusig.pool_reserved_bytes(dev) > 0
    err, threshold_after = rt.cudaMemPoolGetAttribute(pool, rt.cudaMemPoolAttr.cudaMemPoolAttrReleaseThreshold)
    assert int(threshold_after) == int(threshold_before)


@pytest.mark.parametrize("shape", [(4, 30, 8, 4), (3, 25, 19, 3), (2, 300, 8, 4)], ids=["tile", "generic", "segmented"])
@pytest.mark.parametrize("where", ["host", "device"])
def test_nonfinite_flag_is_raised_by_the_forward_pass(shape, where):
    """The NaN / Inf warning of pysiglib.sig (pysiglib/sig.py:299-310) without a pass over the
    output on the host: one overflowing path among finite ones raises the flag, none does not."""
    import pysiglib_b200
    import warnings
    B, L, d, N = shape
    path = brownian_paths(7, B, L, d, np.float32)
    to = (lambda a: torch.tensor(a, device="cuda")) if where == "device" else (lambda a: a)
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        pysiglib_b200.sig(to(path), N)
    bad = path.copy()
    bad[B - 1, L // 2:, 1] = 3e20  # level 2 and above overflow float32
    with pytest.warns(RuntimeWarning, match="NaN or Inf"):
        out = pysiglib_b200.sig(to(bad), N)
    out = out.cpu().numpy() if where == "device" else out
    assert np.isfinite(out[: B - 1]).all() and not np.isfinite(out[B - 1]).all()


def _variants_of(d, N, dtype, backward):
    """(P, G) of every compiled register-tile variant of a shape, read from the generated table."""
    with open(os.path.join(ROOT, "pysiglib_b200", "csrc", "tile_table.h")) as f:
        text = f.read()
    name = "float" if dtype == np.float32 else "double"
    return sorted({(int(p), int(g)) for p, g in
                   re.findall(r"X\(%s, %d, %d, %d, (\d+), (\d+), \d+, \d+\)" % (name, 1 if backward else 0, d, N), text)})


@pytest.mark.parametrize("d,N", [(16, 4), (8, 4), (5, 7), (10, 5), (2, 12), (3, 6)])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_every_compiled_variant_of_a_shape_agrees_with_the_oracle(d, N, dtype):
    B, L = 3, 150
    path = brownian_paths(d * N, B, L, d, dtype)
    expect = oracle.sig(path, N)
    seeds = np.random.default_rng(d).standard_normal(expect.shape).astype(dtype)
    want = oracle.sig_backprop(path, expect, seeds, N)
    p64 = path.astype(np.float64)
    truth = oracle.sig_backprop(p64, oracle.sig(p64, N), seeds.astype(np.float64), N)
    tol = 1e-5 if dtype == np.float32 else 1e-10
    name = "float32" if dtype == np.float32 else "float64"
    fwd, bwd = _variants_of(d, N, dtype, False), _variants_of(d, N, dtype, True)
    assert fwd and bwd
    dpath = torch.tensor(path, device="cuda")
    try:
        for P, G in fwd:
            for segments in (1, 2, 3, 5):   # the join of 3 and 5 segments runs several rounds of the chain kernel
                load_cusig.set_forced_plan(False, P, G, segments)
                plan = load_cusig.describe_plan(B, d, L, N, dtype=name)
                assert "P=%d,G=%d" % (P, G) in plan and "segments=%d" % segments in plan, plan
                code, got = _forward(dpath, N)
                assert code == 0, load_cusig.last_error_message()
                assert_sig_close(got.cpu().numpy(), expect, d, N, tol, what="forward P=%d G=%d x%d" % (P, G, segments))
        load_cusig.set_forced_plan(False, -1, 0, 1)
        for P, G in bwd:
            for segments in (1, 2):
                load_cusig.set_forced_plan(True, P, G, segments)
                code, got = _backward(dpath, torch.tensor(expect, device="cuda"), torch.tensor(seeds, device="cuda"), N)
                assert code == 0, load_cusig.last_error_message()
                assert_grad_parity(got.cpu().numpy(), want, truth, tol, "backward P=%d G=%d x%d" % (P, G, segments))
    finally:
        load_cusig.set_forced_plan(False, -1, 0, 1)
        load_cusig.set_forced_plan(True, -1, 0, 1)


def test_buffers_on_different_devices_are_rejected_on_the_host():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    path = torch.zeros((2, 5, 3), device="cuda:0")
    out = torch.zeros((2 * 39,), device="cuda:1")
    before = load_cusig.launch_count()
    code, _ = cabi.signature_cuda(path, 3, out=out)
    assert code == 2 and "same device" in load_cusig.last_error_message()
    assert load_cusig.launch_count() == before


@pytest.mark.parametrize("resident", [False, True], ids=["scattered", "already_resident"])
def test_sig_multi_device_is_differentiable_and_matches_one_device(resident):
    """The device-resident sharded front-end: scatter with .to(device) (or shards that already
    live on their devices), Sig per shard, optional gather; gradients flow back to the input.
    With one GPU the two shards share it, which still exercises the bookkeeping."""
    import pysiglib_b200
    from pysiglib_b200 import torch_api
    n = torch.cuda.device_count()
    devices = [0, 1] if n >= 2 else [0, 0]
    path_np = brownian_paths(9, 7, 30, 4, np.float64)
    weights = torch.tensor(np.random.default_rng(1).standard_normal((7, 340)), device="cuda:0")
    ref = torch.tensor(path_np, device="cuda:0", requires_grad=True)
    (torch_api.sig(ref, 4) * weights).sum().backward()
    if resident:
        leaves = [torch.tensor(path_np[:4], device="cuda:%d" % devices[0], requires_grad=True),
                  torch.tensor(path_np[4:], device="cuda:%d" % devices[1], requires_grad=True)]
        parts = pysiglib_b200.sig_multi_device(leaves, 4)
        assert [p.device for p in parts] == [l.device for l in leaves]
        out = torch.cat([p.to("cuda:0") for p in parts])
        (out * weights).sum().backward()
        grad = torch.cat([l.grad.to("cuda:0") for l in leaves])
    else:
        x = torch.tensor(path_np, requires_grad=True)  # lives on the host; shards travel to the GPUs
        out = pysiglib_b200.sig_multi_device(x, 4, devices=devices, gather_to="cuda:0")
        assert out.shape == (7, 340) and out.device == torch.device("cuda:0")
        (out * weights).sum().backward()
        grad = x.grad.to("cuda:0")
    np.testing.assert_allclose(out.detach().cpu().numpy(), oracle.sig(path_np, 4), rtol=1e-10, atol=1e-13)
    np.testing.assert_allclose(grad.cpu().numpy(), ref.grad.cpu().numpy(), rtol=1e-12, atol=1e-14)


DEEP_SHAPES = [  # (B, L, d, N, dtype, flags): beyond the three-variant table, one long-chain tile each
    (3, 9, 6, 8, np.float32, {}),
    (2, 6, 16, 6, np.float64, {}),
    (3, 12, 24, 4, np.float64, {}),
    (3, 40, 10, 5, np.float64, {"time_aug": True}),     # C1's shape with time augmentation (d' = 11)
    (2, 30, 2, 12, np.float64, {"lead_lag": True}),     # C2's shape with lead-lag (d' = 4)
    (2, 10, 32, 4, np.float32, {}),
]


@pytest.mark.parametrize("case", DEEP_SHAPES, ids=lambda c: "d%d_N%d_%s%s" % (c[2], c[3], c[4].__name__, "".join("_" + k for k in c[5])))
def test_deep_degree_shapes_run_on_register_tiles(case):
    """Shapes the reference serves with its register 'Tree' kernels (siglib/cusig/
    cu_signature_horner.cuh:267-307, 389-438) and flagged benchmark shapes: served by long-chain
    register tiles here, not by the generic fallback, and equal to the oracle."""
    B, L, d, N, dtype, kw = case
    name = "float32" if dtype == np.float32 else "float64"
    for backward in (False, True):
        assert load_cusig.kernel_family(d, N, dtype=name, backward=backward, **kw) == "tile"
    D = cabi.aug_dim(d, kw.get("time_aug", False), kw.get("lead_lag", False))
    path = brownian_paths(d + N, B, L, d, dtype) * 1.5
    expect = oracle.sig(path, N, **kw)
    tol = 1e-5 if dtype == np.float32 else 1e-10
    dpath = torch.tensor(path, device="cuda")
    code, got = _forward(dpath, N, **kw)
    assert code == 0, load_cusig.last_error_message()
    assert_sig_close(got.cpu().numpy(), expect, D, N, tol)
    seeds = np.random.default_rng(N).standard_normal(expect.shape).astype(dtype)
    want = oracle.sig_backprop(path, expect, seeds, N, **kw)
    p64 = path.astype(np.float64)
    truth = oracle.sig_backprop(p64, oracle.sig(p64, N, **kw), seeds.astype(np.float64), N, **kw)
    code, grad = _backward(dpath, torch.tensor(expect, device="cuda"), torch.tensor(seeds, device="cuda"), N, **kw)
    assert code == 0, load_cusig.last_error_message()
    assert_grad_parity(grad.cpu().numpy(), want, truth, tol)


def test_operators_without_a_stream_argument_wait_for_the_callers_side_stream():
    """sig_combine and friends keep the reference's signatures and run on the legacy default
    stream; an operand still being produced on a torch side stream (non-blocking, so the legacy
    stream does not wait for it) must be finished before they read it."""
    import pysiglib_b200
    d, N, B = 8, 4, 512
    a_np = oracle.sig(brownian_paths(1, 4, 20, d, np.float32), N)
    side = torch.cuda.Stream()
    big = torch.randn((4096, 4096), device="cuda")
    with torch.cuda.stream(side):
        for _ in range(20):
            big = big @ big * 1e-4            # keeps the side stream busy for a while
        a = torch.tensor(np.tile(a_np, (B // 4, 1)), device="cuda") + big[0, 0] * 0.0
        b = a.clone()
        out = pysiglib_b200.sig_combine(a, b, d, N)
        lin = pysiglib_b200.sig_to_log_sig(a, d, N, method=0)
    side.synchronize()
    want = oracle.sig_combine(a_np, a_np, d, N)
    assert_sig_close(out[:4].cpu().numpy(), want, d, N, 1e-5)
    # the same calls once nothing is in flight give bit-identical results
    assert torch.equal(out, pysiglib_b200.sig_combine(a, b, d, N))
    assert torch.equal(lin, pysiglib_b200.sig_to_log_sig(a, d, N, method=0))
