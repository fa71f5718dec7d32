"""Pins the log-signature part of the oracle (``oracle/sig_oracle_log.h`` and the Lyndon-basis
projection in ``oracle/oracle.py``) to the reference's own golden vectors.

The vectors come from the reference's fixture (``tests/fixtures/reference_data.npz``, written
there by iisignature / signatory) and are the ones its ``tests/test_log_sig.py:105-196`` and
``tests/test_log_sig_backprop.py:32-183`` compare against: expanded logarithm (plain, time
augmented, lead-lag), Lyndon-word coordinates, Lyndon-basis coordinates, and the gradients of
all of them with respect to the path.  Tolerances are the reference's (1e-10 absolute against
float64 vectors, 1e-5 for the gradient checks, whose expected arrays are mostly float32)."""
import numpy as np
import pytest

from oracle import oracle

DIM = 3


@pytest.mark.parametrize("deg", range(1, 6))
def test_expanded(golden, deg):
    s = oracle.sig(golden["path"], deg)
    got = oracle.sig_to_log_sig(s, DIM, deg, method=0)
    assert np.abs(got - golden["logsig_exp__d%d" % deg]).max() <= 1e-10


@pytest.mark.parametrize("deg", range(1, 6))
def test_expanded_time_aug(golden, deg):
    s = oracle.sig(golden["path"], deg, time_aug=True)
    got = oracle.sig_to_log_sig(s, DIM + 1, deg, method=0)
    assert np.abs(got - golden["logsig_exp_ta__d%d" % deg]).max() <= 1e-10


@pytest.mark.parametrize("deg", range(1, 5))
def test_expanded_lead_lag(golden, deg):
    s = oracle.sig(golden["path"][:2], deg, lead_lag=True)
    got = oracle.sig_to_log_sig(s, 2 * DIM, deg, method=0)
    assert np.abs(got - golden["logsig_exp_ll__d%d" % deg]).max() <= 1e-10


@pytest.mark.parametrize("deg", range(1, 6))
@pytest.mark.parametrize("scalar_term", [False, True])
def test_lyndon_words_and_basis(golden, deg, scalar_term):
    s = oracle.sig(golden["path"], deg, scalar_term=scalar_term)
    words = oracle.sig_to_log_sig(s, DIM, deg, method=1)
    basis = oracle.sig_to_log_sig(s, DIM, deg, method=2)
    assert words.shape == basis.shape == golden["logsig_words__d%d" % deg].shape
    assert np.abs(words - golden["logsig_words__d%d" % deg]).max() <= 1e-10
    assert np.abs(basis - golden["logsig_basis__d%d" % deg]).max() <= 1e-10


@pytest.mark.parametrize("deg", range(1, 6))
@pytest.mark.parametrize("name,method,flags,dim", [("exp", 0, {}, DIM), ("exp_ta", 0, {"time_aug": True}, DIM + 1),
                                                   ("words", 1, {}, DIM), ("basis", 2, {}, DIM)])
def test_backprop_to_the_path(golden, deg, name, method, flags, dim):
    path = golden["path"]
    s = oracle.sig(path, deg, **flags)
    d_log = golden["logsig_bp_%s_derivs__d%d" % (name, deg)]
    d_sig = oracle.sig_to_log_sig_backprop(s, d_log, dim, deg, method=method)
    got = oracle.sig_backprop(path, s, d_sig, deg, **flags)
    expected = golden["logsig_bp_%s_expected__d%d" % (name, deg)]
    atol = 1e-5 if expected.dtype == np.float32 else 1e-10
    assert np.abs(got - expected).max() <= atol


@pytest.mark.parametrize("deg", range(1, 6))
def test_sig_to_log_sig_backprop_one_dimensional(golden, deg):
    # the fixture's input carries the scalar term; the expected gradient is scalar-free
    x = golden["sig_to_logsig_bp_input__d%d" % deg][:, 1:]
    got = oracle.sig_to_log_sig_backprop(x, np.ones_like(x), 1, deg, method=0)
    assert np.abs(got - golden["sig_to_logsig_bp_expected__d%d" % deg]).max() <= 1e-10
    with_scalar = oracle.sig_to_log_sig_backprop(golden["sig_to_logsig_bp_input__d%d" % deg],
                                                 np.ones((1, deg + 1)), 1, deg, method=0)
    assert with_scalar[0, 0] == 0 and np.abs(with_scalar[:, 1:] - got).max() <= 1e-15
