"""Length of a truncated signature.

Same contract as the reference's ``sig_length`` (``pysiglib/sig_length.py:25-95``, C side
``siglib/cpsig/cp_utils.cpp:91-105``): ``sum_{k=0..N} d'^k`` coefficients with the scalar
term, one less without it; lengths that do not fit 64 bits raise ValueError."""
from .param_checks import check_non_neg, check_type


def aug_dim(dimension, time_aug, lead_lag):
    """Path dimension after lead-lag (doubles it) and time augmentation (adds one)."""
    return (2 * dimension if lead_lag else dimension) + (1 if time_aug else 0)


def _full_length(dim, degree):
    if dim == 0:
        return 1
    if dim == 1:
        return degree + 1
    total = (dim ** (degree + 1) - 1) // (dim - 1)
    if dim ** (degree + 1) >= 1 << 64:
        raise ValueError("Integer overflow encountered in sig_length")
    return total


def sig_length(dimension, degree, *, time_aug=False, lead_lag=False, scalar_term=False):
    """Number of coefficients of the degree-``degree`` signature of a ``dimension``-channel path.

    ``time_aug`` / ``lead_lag`` apply the corresponding change of dimension first.
    ``scalar_term`` counts the leading constant 1 (must match the flag given to ``sig``).
    """
    check_type(dimension, "dimension", int)
    check_type(degree, "degree", int)
    check_non_neg(dimension, "dimension")
    check_non_neg(degree, "degree")
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    return _full_length(aug_dim(dimension, time_aug, lead_lag), degree) - (0 if scalar_term else 1)


def infer_scalar_term(sig, dimension, degree, time_aug=False, lead_lag=False):
    """True when the last axis of ``sig`` includes the scalar term (reference:
    ``pysiglib/sig_length.py:165-182``); ValueError when it matches neither layout."""
    full = sig_length(dimension, degree, time_aug=time_aug, lead_lag=lead_lag, scalar_term=True)
    got = sig.shape[-1]
    if got == full:
        return True
    if got == full - 1:
        return False
    raise ValueError("sig has incompatible length %d for dimension=%d, degree=%d (expected %d or %d)."
                     % (got, dimension, degree, full, full - 1))


def _mobius(k):
    result, p = 1, 2
    while p * p <= k:
        if k % p == 0:
            k //= p
            if k % p == 0:
                return 0
            result = -result
        p += 1
    return -result if k > 1 else result


def log_sig_length(dimension, degree, *, time_aug=False, lead_lag=False):
    """Number of coordinates of the degree-``degree`` log signature in a Lyndon basis: Witt's
    formula ``sum_{i=1..N} (1/i) sum_{x | i} mu(i/x) d^x`` (reference:
    ``pysiglib/sig_length.py:97-163``)."""
    check_type(dimension, "dimension", int)
    check_type(degree, "degree", int)
    check_non_neg(dimension, "dimension")
    check_non_neg(degree, "degree")
    check_type(time_aug, "time_aug", bool)
    check_type(lead_lag, "lead_lag", bool)
    d = aug_dim(dimension, time_aug, lead_lag)
    total = 0
    for i in range(1, degree + 1):
        total += sum(_mobius(i // x) * d ** x for x in range(1, i + 1) if i % x == 0) // i
    return total
