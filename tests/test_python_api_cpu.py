"""Host-side logic of the Python operators (argument contract of the reference's sig /
sig_backprop, pysiglib/sig.py:265-279, pysiglib/sig_backprop.py:210-234), checked without a GPU:
every case here fails or returns before any native compute call."""
import inspect

import numpy as np
import pytest
import torch

import pysiglib_b200 as psl
from pysiglib_b200 import torch_api
from pysiglib_b200.sharded import shard_bounds


def test_signatures_match_the_reference_surface():
    p = inspect.signature(psl.sig).parameters
    assert list(p) == ["path", "degree", "time_aug", "lead_lag", "end_time", "horner", "scalar_term", "correction",
                       "n_jobs"]
    assert all(p[k].kind is inspect.Parameter.KEYWORD_ONLY for k in list(p)[2:])
    assert (p["time_aug"].default, p["lead_lag"].default, p["end_time"].default, p["horner"].default,
            p["scalar_term"].default, p["correction"].default, p["n_jobs"].default) == (False, False, 1., True, False,
                                                                                       None, 1)
    q = inspect.signature(psl.sig_backprop).parameters
    assert list(q) == ["path", "sig", "sig_derivs", "degree", "time_aug", "lead_lag", "end_time", "correction", "n_jobs"]
    assert psl.signature is psl.sig
    # torch_api mirrors the base API (reference tests/test_apis_match.py) and exposes no *_backprop
    assert inspect.signature(torch_api.sig) == inspect.signature(psl.sig)
    assert torch_api.sig.__doc__ == psl.sig.__doc__
    assert not hasattr(torch_api, "sig_backprop")


def test_sig_length():
    assert psl.sig_length(3, 4, scalar_term=True) == 121
    assert psl.sig_length(3, 4) == 120
    assert psl.sig_length(3, 4, time_aug=True, lead_lag=True, scalar_term=True) == 2801
    assert psl.sig_length(1, 5) == 5
    assert psl.sig_length(0, 5, scalar_term=True) == 1
    with pytest.raises(ValueError):
        psl.sig_length(2, 64)
    with pytest.raises(TypeError):
        psl.sig_length(2.0, 3)


def test_argument_type_checks():
    x = np.zeros((2, 5, 3))
    with pytest.raises(TypeError):
        psl.sig(x, 2.0)
    with pytest.raises(ValueError):
        psl.sig(x, -1)
    with pytest.raises(TypeError):
        psl.sig(x, 2, end_time=1)          # an int is not accepted (reference sig.py:270)
    with pytest.raises(TypeError):
        psl.sig(x, 2, time_aug=1)
    with pytest.raises(ValueError):
        psl.sig(x, 2, n_jobs=0)
    with pytest.raises(TypeError):
        psl.sig([[0.0, 1.0]], 2)
    with pytest.raises(TypeError):
        psl.sig(x.astype(np.float16), 2)
    with pytest.raises(ValueError):
        psl.sig(np.zeros(5), 2)
    with pytest.raises(ValueError):
        psl.sig(np.zeros((2, 5, 0)), 2)


def test_correction_argument_contract():
    # reference tests/test_signature.py:191-205: shape, dtype, prefix and lead_lag rules, checked before any native call
    x = np.zeros((2, 2), dtype=np.float64)
    with pytest.raises(ValueError, match="correction shape"):
        psl.sig(x, 2, correction=np.array(1.0, dtype=np.float64))
    with pytest.raises(ValueError, match="same dtype"):
        psl.sig(x, 2, correction=np.zeros((1, 4), dtype=np.float32))
    with pytest.raises(ValueError, match="prefix"):
        psl.sig(x, 3, correction=np.zeros((1, 5), dtype=np.float64))
    with pytest.raises(ValueError, match="lead_lag"):
        psl.sig(x, 2, lead_lag=True, correction=np.zeros((1, 4), dtype=np.float64))
    with pytest.raises(ValueError, match="degree < 2"):
        psl.sig(x, 1, correction=np.zeros(4))
    with pytest.raises(ValueError, match="same array type"):
        psl.sig(x, 2, correction=torch.zeros(4, dtype=torch.float64))
    with pytest.raises(ValueError, match="correction shape"):
        psl.sig(np.zeros((3, 4, 2)), 2, correction=np.zeros((2, 3, 4)))


def test_join_and_transform_argument_contract():
    import inspect
    assert list(inspect.signature(psl.sig_join).parameters) == ["sig", "displacement", "dimension", "degree",
                                                                 "prepend", "n_jobs"]
    assert list(inspect.signature(psl.sig_join_backprop).parameters) == ["d_out", "sig", "displacement", "dimension",
                                                                          "degree", "prepend", "n_jobs"]
    assert list(inspect.signature(psl.linear_sig).parameters) == ["displacement", "dimension", "degree",
                                                                   "scalar_term", "n_jobs"]
    assert list(inspect.signature(psl.transform_path).parameters) == ["path", "time_aug", "lead_lag", "end_time",
                                                                       "n_jobs"]
    s, v = np.zeros((3, 14)), np.zeros((3, 2))
    with pytest.raises(ValueError, match="same batch shape"):
        psl.sig_join(s, np.zeros((2, 2)), 2, 3)
    with pytest.raises(ValueError, match="same dtype"):
        psl.sig_join(s, v.astype(np.float32), 2, 3)
    with pytest.raises(ValueError, match="incorrect length"):
        psl.sig_join(s, np.zeros((3, 3)), 2, 3)
    with pytest.raises(ValueError):
        psl.sig_join(np.zeros((3, 13)), v, 2, 3)
    with pytest.raises(TypeError):
        psl.sig_join(s, v, 2.0, 3)
    with pytest.raises(ValueError, match="both be numpy arrays or both torch tensors"):
        psl.sig_join(s, torch.zeros((3, 2), dtype=torch.float64), 2, 3)
    assert psl.sig_join(np.zeros((0, 14)), np.zeros((0, 2)), 2, 3).shape == (0, 14)
    a, b = psl.sig_join_backprop(np.zeros((0, 14)), np.zeros((0, 14)), np.zeros((0, 2)), 2, 3)
    assert a.shape == (0, 14) and b.shape == (0, 2)
    assert psl.linear_sig(np.zeros((0, 2)), 2, 3).shape == (0, 14)
    x = np.zeros((4, 5, 2))
    assert psl.transform_path(x) is x
    assert psl.transform_path_backprop(x) is x
    with pytest.raises(ValueError, match="length >= 2"):
        psl.transform_path(np.zeros((1, 2)), time_aug=True)
    assert psl.transform_path(np.zeros((0, 5, 2)), time_aug=True, lead_lag=True).shape == (0, 9, 5)
    assert psl.transform_path_backprop(np.zeros((0, 9, 5)), time_aug=True, lead_lag=True).shape == (0, 5, 2)


def test_empty_batch_returns_without_native_call():
    out = psl.sig(np.zeros((0, 5, 3), dtype=np.float32), 3)
    assert out.shape == (0, 39) and out.dtype == np.float32
    out = psl.sig(torch.zeros((0, 4, 5, 2), dtype=torch.float64), 2, scalar_term=True)
    assert tuple(out.shape) == (0, 4, 7)
    g = psl.sig_backprop(np.zeros((0, 5, 3)), np.zeros((0, 39)), np.zeros((0, 39)), 3)
    assert g.shape == (0, 5, 3)


def test_backprop_argument_consistency():
    x = np.zeros((2, 5, 3))
    s = np.zeros((2, 39))
    with pytest.raises(ValueError):
        psl.sig_backprop(x, np.zeros((2, 38)), np.zeros((2, 38)), 3)       # neither layout
    with pytest.raises(ValueError):
        psl.sig_backprop(x, s, np.zeros((2, 41)), 3)                       # derivs of another length
    with pytest.raises(ValueError):
        psl.sig_backprop(x, s, s.astype(np.float32), 3)                    # dtypes differ
    with pytest.raises(ValueError):
        psl.sig_backprop(x, torch.zeros((2, 39), dtype=torch.float64), torch.zeros((2, 39), dtype=torch.float64), 3)
    with pytest.raises(ValueError):
        psl.sig_backprop(x, np.zeros((3, 39)), np.zeros((3, 39)), 3)       # batch shapes differ


def test_shard_bounds_cover_the_batch():
    for batch in (0, 1, 7, 8, 4096, 4099):
        for n in (1, 2, 3, 4, 8):
            b = shard_bounds(batch, n)
            assert b[0][0] == 0 and b[-1][1] == batch
            assert all(x[1] == y[0] for x, y in zip(b, b[1:]))
            sizes = [e - s for s, e in b]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


def test_sig_combine_argument_contract():
    p = inspect.signature(psl.sig_combine).parameters
    assert list(p) == ["sig1", "sig2", "dimension", "degree", "time_aug", "lead_lag", "n_jobs"]
    q = inspect.signature(psl.sig_combine_backprop).parameters
    assert list(q) == ["deriv", "sig1", "sig2", "dimension", "degree", "time_aug", "lead_lag", "n_jobs"]
    a = np.zeros((2, 14))
    with pytest.raises(ValueError):
        psl.sig_combine(a, np.zeros((2, 15)), 2, 3)            # lengths differ
    with pytest.raises(ValueError):
        psl.sig_combine(np.zeros((2, 13)), np.zeros((2, 13)), 2, 3)   # neither layout of (d=2, N=3)
    with pytest.raises(ValueError):
        psl.sig_combine(a, a.astype(np.float32), 2, 3)          # dtypes differ
    with pytest.raises(TypeError):
        psl.sig_combine(a, a, 2.0, 3)
    with pytest.raises(ValueError):
        psl.sig_combine_backprop(np.zeros((3, 14)), a, a, 2, 3)  # batch shapes differ
    assert psl.sig_combine(np.zeros((0, 14)), np.zeros((0, 14)), 2, 3).shape == (0, 14)
    d1, d2 = psl.sig_combine_backprop(np.zeros((0, 15)), np.zeros((0, 15)), np.zeros((0, 15)), 2, 3)
    assert d1.shape == d2.shape == (0, 15)


def test_log_sig_argument_contract():
    import inspect
    assert list(inspect.signature(psl.sig_to_log_sig).parameters) == ["sig", "dimension", "degree", "time_aug",
                                                                       "lead_lag", "method", "n_jobs"]
    assert list(inspect.signature(psl.sig_to_log_sig_backprop).parameters) == [
        "sig", "log_sig_derivs", "dimension", "degree", "time_aug", "lead_lag", "method", "n_jobs"]
    assert list(inspect.signature(psl.log_sig).parameters) == ["path", "degree", "time_aug", "lead_lag", "end_time",
                                                                "method", "scalar_term", "correction", "n_jobs"]
    assert list(inspect.signature(psl.prepare_log_sig).parameters) == ["dimension", "degree", "method", "time_aug",
                                                                        "lead_lag", "use_disk", "device"]
    # Witt's formula (reference tests/test_sig_length.py uses the same closed form)
    assert [psl.log_sig_length(2, n) for n in range(1, 7)] == [2, 3, 5, 8, 14, 23]
    assert psl.log_sig_length(3, 4) == 32 and psl.log_sig_length(2, 3, time_aug=True) == 14
    assert psl.log_sig_length(2, 3, lead_lag=True) == psl.log_sig_length(4, 3) == 4 + 6 + 20
    s = np.zeros((3, 14))
    with pytest.raises(ValueError, match="one of 0, 1, 2 or 3"):
        psl.sig_to_log_sig(s, 2, 3, method=4)
    with pytest.raises(ValueError, match="method=3"):
        psl.sig_to_log_sig(s, 2, 3, method=3)
    with pytest.raises(NotImplementedError):
        psl.log_sig(np.zeros((3, 5, 2)), 3, method=3)
    with pytest.raises(TypeError):
        psl.sig_to_log_sig(s, 2, 3, method=1.0)
    with pytest.raises(ValueError):
        psl.sig_to_log_sig(np.zeros((3, 13)), 2, 3)
    with pytest.raises(ValueError, match="incorrect length"):
        psl.sig_to_log_sig_backprop(s, np.zeros((3, 4)), 2, 3, method=1)
    assert psl.sig_to_log_sig(np.zeros((0, 14)), 2, 3).shape == (0, 5)
    assert psl.sig_to_log_sig(np.zeros((0, 15)), 2, 3, method=0).shape == (0, 15)
    assert psl.sig_to_log_sig_backprop(np.zeros((0, 14)), np.zeros((0, 5)), 2, 3).shape == (0, 14)
    psl.prepare_log_sig(2, 3, 0)


def test_sig_coef_argument_contract():
    import inspect
    assert list(inspect.signature(psl.sig_coef).parameters) == ["path", "words", "time_aug", "lead_lag", "end_time",
                                                                 "prefixes", "n_jobs"]
    assert list(inspect.signature(psl.sig_coef_backprop).parameters) == ["path", "words", "coefs", "derivs", "time_aug",
                                                                          "lead_lag", "end_time", "n_jobs"]
    x = np.zeros((0, 5, 2))
    assert psl.sig_coef(x, [(0,), (1, 0)]).shape == (0, 2)
    assert psl.sig_coef(x, [(0,), (1, 0)], prefixes=True).shape == (0, 3)
    assert psl.sig_coef_backprop(x, [(1, 0)], np.zeros((0, 2)), np.zeros((0, 2))).shape == (0, 5, 2)
    y = np.zeros((3, 5, 2))
    with pytest.raises(ValueError, match="range"):
        psl.sig_coef(y, [(0, 2)])
    with pytest.raises(TypeError):
        psl.sig_coef(y, [[0, 1]])
    with pytest.raises(TypeError):
        psl.sig_coef(y, (0, 1.0))
    with pytest.raises(ValueError, match="non-empty"):
        psl.sig_coef(y, [])
    with pytest.raises(ValueError, match="prefixes=True"):
        psl.sig_coef_backprop(y, [(1, 0)], np.zeros((3, 1)), np.zeros((3, 1)))
    sig = np.arange(14.0)
    np.testing.assert_array_equal(psl.extract_sig_coef(sig, [(0,), (1, 0), (1, 1, 1)], 2), [0.0, 4.0, 13.0])
    np.testing.assert_array_equal(psl.extract_sig_coef(np.arange(15.0), [(), (1,)], 2, scalar_term=True), [0.0, 2.0])
