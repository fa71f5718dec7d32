"""The C-ABI library loads without a GPU and exports every symbol include/cusig_b200.h
declares, plus the stubs for the rest of the reference's CUDA surface.  No compute calls."""
import os
import re

import pytest

from pysiglib_b200 import load_cusig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    with open(os.path.join(ROOT, "include", "cusig_b200.h")) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    return sorted(set(re.findall(r"\b([a-z][a-z0-9_]*)\s*\(", text)) - {"defined"})


def test_header_symbols_are_exported():
    lib = load_cusig.library()
    names = declared_symbols()
    assert {"signature_cuda_f", "signature_cuda_d", "sig_backprop_cuda_f", "sig_backprop_cuda_d",
            "cusig_last_error_message", "cusig_shutdown"} <= set(names)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_reference_loader_symbols_are_present():
    # every name the reference's loader resolves at import (pysiglib/load_siglib.py:165-183,420-641)
    lib = load_cusig.library()
    families = ("transform_path transform_path_backprop log_sig_combine log_sig_combine_backprop log_sig_from_path "
                "log_sig_from_path_backprop log_sig_join log_sig_join_backprop logsig_to_sig logsig_to_sig_backprop "
                "sig_combine sig_combine_backprop sig_join sig_join_backprop sig_coef sig_coef_backprop sig_to_log_sig "
                "sig_to_log_sig_backprop sig_kernel sig_kernel_backprop sig_kernel_poly sig_kernel_poly_backprop "
                "linear_sig branched_sig branched_sig_backprop branched_sig_coef branched_sig_coef_backprop "
                "branched_sig_combine branched_sig_combine_backprop branched_sig_kernel branched_sig_kernel_backprop "
                "branched_sig_kernel_poly branched_sig_kernel_poly_backprop branched_sig_to_log_sig "
                "branched_sig_to_log_sig_backprop branched_log_sig_join branched_log_sig_join_backprop "
                "branched_log_sig_from_path branched_log_sig_from_path_backprop signature sig_backprop").split()
    for fam in families:
        for suf in ("f", "d"):
            assert hasattr(lib, "%s_cuda_%s" % (fam, suf)), fam
    for name in ("prepare_log_sig_cuda clear_cache_cuda set_cache_dir_cuda prepare_branched_sig_cuda "
                 "prepare_branched_log_sig_cuda prepare_branched_sig_coef_cuda").split():
        assert hasattr(lib, name), name


def test_stub_reports_a_clean_error_without_a_gpu():
    lib = load_cusig.library()
    assert lib.sig_kernel_cuda_f() == 10
    assert "not part of this build" in load_cusig.last_error_message()
    assert lib.sigb200_sig_length(3, 4) == 121
    assert lib.sigb200_sig_length(2, 64) == 0  # overflow


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(load_cusig, "_lib", None)
    monkeypatch.setattr(load_cusig, "LIBRARY_PATH", "/nonexistent/libcusig.so")
    with pytest.raises(load_cusig.CusigNotBuiltError):
        load_cusig.library()
