"""GPU parity of ``log_sig`` / ``sig_to_log_sig`` and their backward passes against the
reference's own golden vectors, case by case as the reference tests them
(``tests/test_log_sig.py:105-196``: expanded / time-augmented / lead-lag / Lyndon words /
Lyndon basis, single path and batch, float64 and float32;
``tests/test_log_sig_backprop.py:32-183``: the gradients of all of them with respect to the
path, through autograd).  Tolerances are the reference's ``check_close``: absolute 1e-10 for
float64 forward, 1e-4 for float32 forward, 1e-5 (float64) / 1e-4 (float32) for gradients, and
1e-3 for the float32 batch gradient of the Lyndon basis."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DIM = 3
DTYPES = [np.float64, np.float32]


def _close(expected, got, single_atol=1e-4, double_atol=1e-10):
    got = got.detach().cpu().numpy() if hasattr(got, "cpu") else np.asarray(got)
    expected = np.asarray(expected)
    atol = single_atol if (got.dtype == np.float32 or expected.dtype == np.float32) else double_atol
    diff = np.abs(got.astype(np.float64) - expected.astype(np.float64)).max()
    assert got.shape == expected.shape and diff <= atol, "max diff %.3e > %.1e" % (diff, atol)


@pytest.mark.parametrize("deg", range(1, 6))
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("batched", [False, True])
def test_expanded(golden, deg, dtype, batched):
    from pysiglib_b200 import torch_api
    x = golden["path"].astype(dtype)
    expected = golden["logsig_exp__d%d" % deg]
    if not batched:
        x, expected = x[0], expected[0]
    got = torch_api.log_sig(torch.tensor(x, device="cuda"), deg, method=0)
    assert got.device.type == "cuda"
    _close(expected, got)


@pytest.mark.parametrize("deg", range(1, 6))
@pytest.mark.parametrize("dtype", DTYPES)
def test_expanded_time_aug(golden, deg, dtype):
    from pysiglib_b200 import torch_api
    got = torch_api.log_sig(torch.tensor(golden["path"].astype(dtype), device="cuda"), deg, time_aug=True, method=0)
    _close(golden["logsig_exp_ta__d%d" % deg], got)


@pytest.mark.parametrize("deg", range(1, 5))
@pytest.mark.parametrize("dtype", DTYPES)
def test_expanded_lead_lag(golden, deg, dtype):
    from pysiglib_b200 import torch_api
    got = torch_api.log_sig(torch.tensor(golden["path"][:2].astype(dtype), device="cuda"), deg, lead_lag=True, method=0)
    _close(golden["logsig_exp_ll__d%d" % deg], got)


@pytest.mark.parametrize("deg", range(1, 6))
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("method,key", [(1, "logsig_words"), (2, "logsig_basis")])
@pytest.mark.parametrize("batched", [False, True])
def test_lyndon_coordinates(golden, deg, dtype, method, key, batched):
    import pysiglib_b200
    from pysiglib_b200 import torch_api
    x = golden["path"].astype(dtype)
    expected = golden["%s__d%d" % (key, deg)]
    if not batched:
        x, expected = x[0], expected[0]
    pysiglib_b200.prepare_log_sig(DIM, deg, method)
    got = torch_api.log_sig(torch.tensor(x, device="cuda"), deg, method=method)
    _close(expected, got)
    # NumPy callers reach the same kernels through host pointers
    _close(expected, pysiglib_b200.log_sig(x, deg, method=method))


@pytest.mark.parametrize("deg", range(1, 6))
@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_sig_to_log_sig_backprop_expanded(golden, deg, dtype):
    from pysiglib_b200 import torch_api
    full = torch.tensor(golden["sig_to_logsig_bp_input__d%d" % deg], dtype=dtype, device="cuda")
    x = full[:, 1:].clone().detach().requires_grad_(True)
    ls = torch_api.sig_to_log_sig(x, 1, deg, method=0)
    ls.backward(torch.ones_like(ls))
    _close(golden["sig_to_logsig_bp_expected__d%d" % deg], x.grad, double_atol=1e-5)


@pytest.mark.parametrize("deg", range(1, 6))
@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("name,method,flags", [("exp", 0, {}), ("exp_ta", 0, {"time_aug": True}), ("words", 1, {}),
                                               ("basis", 2, {})])
@pytest.mark.parametrize("batched", [False, True])
def test_log_sig_backprop_through_autograd(golden, deg, dtype, name, method, flags, batched):
    import pysiglib_b200
    from pysiglib_b200 import torch_api
    if name == "exp_ta" and not batched:
        pytest.skip("the reference tests the time-augmented gradient on the batch only")
    path, derivs = golden["path"], golden["logsig_bp_%s_derivs__d%d" % (name, deg)]
    expected = golden["logsig_bp_%s_expected__d%d" % (name, deg)]
    if not batched:
        sl = slice(0, 1) if name == "words" else 0
        path, derivs, expected = path[sl], derivs[sl], expected[sl]
    x = torch.tensor(path, dtype=dtype, device="cuda", requires_grad=True)
    pysiglib_b200.prepare_log_sig(DIM, deg, method)
    ls = torch_api.log_sig(x, deg, method=method, **flags)
    ls.backward(torch.tensor(derivs, dtype=dtype, device="cuda"))
    single = 1e-3 if (name == "basis" and batched) else 1e-4
    _close(expected, x.grad, single_atol=single, double_atol=1e-5)
