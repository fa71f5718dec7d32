"""The drop-in boundary, checked mechanically against the reference's own binding code.

``tests/golden/reference_cuda_abi.json`` holds the ctypes declaration of every symbol the
reference's loader binds in its CUDA library (extracted from ``pysiglib/load_siglib.py`` by
``tests/golden/make_abi_table.py``).  For every one of those symbols this build implements,
the C prototype in ``include/cusig_b200.h`` and the binding in ``pysiglib_b200/load_cusig.py``
must agree with it type for type; every other one must at least be exported (as a stub), because
the reference's loader resolves all of them at import."""
import ctypes
import json
import os
import re

import pytest

from pysiglib_b200 import load_cusig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TABLE = os.path.join(ROOT, "tests", "golden", "reference_cuda_abi.json")

C_TO_CTYPES = {"float": "c_float", "double": "c_double", "uint64_t": "c_uint64", "bool": "c_bool", "int": "c_int",
               "char": "c_char", "void": "None"}


def _ctype_of(c_type):
    c_type = c_type.replace("const", "").strip()
    stars = c_type.count("*")
    base = C_TO_CTYPES[c_type.replace("*", "").strip()]
    if stars == 1 and base == "c_char":
        return "c_char_p"
    for _ in range(stars):
        base = "POINTER(%s)" % base
    return base


def header_prototypes():
    with open(os.path.join(ROOT, "include", "cusig_b200.h")) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    text = re.sub(r"#.*", "", text)
    protos = {}
    for ret, name, args in re.findall(r"([A-Za-z_][\w\s\*]*?)\b([a-z][a-z0-9_]*)\s*\(([^()]*)\)\s*;", text):
        ret = ret.replace('extern "C"', "").strip()
        arg_types = []
        for a in [a.strip() for a in args.split(",") if a.strip() and a.strip() != "void"]:
            m = re.match(r"(.*?)(\b[A-Za-z_]\w*)$", a)  # strip the parameter name
            arg_types.append(_ctype_of(m.group(1) if m and m.group(1).strip() else a))
        protos[name] = {"argtypes": arg_types, "restype": _ctype_of(ret)}
    return protos


@pytest.fixture(scope="module")
def reference_abi():
    with open(TABLE) as f:
        return json.load(f)


def test_table_is_current_with_the_mounted_reference(reference_abi):
    root = os.environ.get("PYSIGLIB_REFERENCE_ROOT", "")
    src = os.path.join(root, "pysiglib", "load_siglib.py")
    if not root or not os.path.exists(src):
        pytest.skip("set PYSIGLIB_REFERENCE_ROOT to the reference tree to re-derive the table")
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_abi_table", os.path.join(ROOT, "tests", "golden", "make_abi_table.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    with open(src) as f:
        assert mod.extract(f.read()) == reference_abi


def test_header_prototypes_match_the_reference_binding(reference_abi):
    protos = header_prototypes()
    served = sorted(set(protos) & set(reference_abi))
    # the path this build serves, with its neighbours
    for must in ("signature_cuda_f", "signature_cuda_d", "sig_backprop_cuda_f", "sig_backprop_cuda_d",
                 "cusig_last_error_message", "cusig_shutdown", "sig_combine_cuda_f", "sig_join_backprop_cuda_d",
                 "transform_path_cuda_f", "sig_to_log_sig_backprop_cuda_d", "sig_coef_cuda_f", "prepare_log_sig_cuda"):
        assert must in served, must
    for name in served:
        assert protos[name] == reference_abi[name], (name, protos[name], reference_abi[name])


def test_every_symbol_the_reference_loader_resolves_is_exported(reference_abi):
    lib = load_cusig.library()
    missing = [name for name in reference_abi if not hasattr(lib, name)]
    assert not missing, missing


def _name_of(ctype):
    if ctype is None:
        return "None"
    if hasattr(ctype, "_type_") and not isinstance(ctype._type_, str):
        return "POINTER(%s)" % _name_of(ctype._type_)
    # ctypes aliases fixed-width names to the platform's types (c_uint64 is c_ulong on LP64)
    for fixed in ("c_uint64", "c_int", "c_bool", "c_float", "c_double", "c_char_p"):
        if ctype is getattr(ctypes, fixed):
            return fixed
    return ctype.__name__


def test_python_binding_matches_the_reference_binding(reference_abi):
    lib = load_cusig.library()
    checked = 0
    for name, decl in reference_abi.items():
        fn = getattr(lib, name)
        if fn.argtypes is None:
            continue  # a stub this package does not bind
        assert [_name_of(t) for t in fn.argtypes] == decl["argtypes"], name
        assert _name_of(fn.restype) == decl["restype"], name
        checked += 1
    assert checked >= 29  # 13 operator families in two precisions + the three lifecycle symbols
