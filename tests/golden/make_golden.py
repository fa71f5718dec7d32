"""Extract the hot-path golden vectors of the reference's test fixture.

Source: the reference's ``tests/fixtures/reference_data.npz`` (generated there by
iisignature, see the reference's ``tests/fixtures/generate_fixtures_iisig.py:47-82``
and consumed by its ``tests/test_signature.py:32-110`` and
``tests/test_sig_backprop.py:69-98``, ``tests/test_sig_combine_backprop.py:28-67``,
``tests/test_log_sig.py:105-196`` and ``tests/test_log_sig_backprop.py:32-183``).  Only the
keys that pin ``sig``, ``sig_backprop``, ``sig_combine_backprop``, ``log_sig`` /
``sig_to_log_sig`` and their backward passes are kept; the file written here is what the
tests read, so the suite does not need the reference tree at run time.

Usage (only where the reference tree is mounted):
    python tests/golden/make_golden.py /path/to/reference
"""
import os
import sys

import numpy as np

KEEP_PREFIXES = ("path", "sig__d", "sig_ta__d", "sig_ll__d", "sig_ta_ll__d",
                 "sig_bp_derivs__d", "sig_bp_expected__d", "sig_comb_bp_",
                 "logsig_exp__d", "logsig_exp_ta__d", "logsig_exp_ll__d", "logsig_words__d", "logsig_basis__d",
                 "logsig_bp_", "sig_to_logsig_bp_")


def main(reference_root):
    src = os.path.join(reference_root, "tests", "fixtures", "reference_data.npz")
    data = np.load(src)
    keep = {k: data[k] for k in data.files if k.startswith(KEEP_PREFIXES)}
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_sig_vectors.npz")
    np.savez_compressed(dst, **keep)
    print("wrote", dst, "with", len(keep), "arrays,", sum(v.nbytes for v in keep.values()), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
