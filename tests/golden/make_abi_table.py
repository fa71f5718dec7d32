"""Extract the ctypes declarations of the reference's CUDA library from its loader, as text.

Source: the reference's ``pysiglib/load_siglib.py`` (``_bind_float_pair(CUSIG, name, lambda T:
(...))`` calls at :420-641 and the explicit ``CUSIG.<name>.argtypes = (...)`` assignments at
:108-110, :165-183, :643-664).  The file is parsed with ``ast``; nothing of the reference is imported
or executed.  The table written here (``reference_cuda_abi.json``: symbol -> argument type
names and result type) is what ``tests/test_abi_matches_reference_loader.py`` holds
``include/cusig_b200.h`` and ``pysiglib_b200/load_cusig.py`` to, so the suite does not need
the reference tree at run time.

Usage (only where the reference tree is mounted):
    python tests/golden/make_abi_table.py /path/to/reference
"""
import ast
import json
import os
import sys


def type_name(node, scalar):
    """ctypes expression -> text, with the lambda's parameter replaced by `scalar`."""
    if isinstance(node, ast.Name):
        return scalar if node.id == "T" else node.id
    if isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id == "POINTER":
        return "POINTER(%s)" % type_name(node.args[0], scalar)
    raise ValueError("unexpected type expression: " + ast.dump(node))


def extract(source):
    table = {}
    tree = ast.parse(source)
    for node in ast.walk(tree):
        # _bind_float_pair(CUSIG, "name", lambda T: (...))
        if (isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id == "_bind_float_pair"
                and isinstance(node.args[0], ast.Name) and node.args[0].id == "CUSIG"):
            name = node.args[1].value
            body = node.args[2].body
            for suffix, scalar in (("f", "c_float"), ("d", "c_double")):
                table["%s_%s" % (name, suffix)] = {"argtypes": [type_name(e, scalar) for e in body.elts],
                                                   "restype": "c_int"}
        # CUSIG.<name>.argtypes = (...)  /  CUSIG.<name>.restype = ...
        if isinstance(node, ast.Assign) and len(node.targets) == 1:
            t = node.targets[0]
            if (isinstance(t, ast.Attribute) and isinstance(t.value, ast.Attribute)
                    and isinstance(t.value.value, ast.Name) and t.value.value.id == "CUSIG"):
                entry = table.setdefault(t.value.attr, {})
                if t.attr == "argtypes":
                    entry["argtypes"] = [type_name(e, None) for e in node.value.elts]
                elif t.attr == "restype":
                    entry["restype"] = "None" if isinstance(node.value, ast.Constant) else type_name(node.value, None)
    return table


def main(reference_root):
    with open(os.path.join(reference_root, "pysiglib", "load_siglib.py")) as f:
        table = extract(f.read())
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_cuda_abi.json")
    with open(dst, "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
        f.write("\n")
    print("wrote", dst, "with", len(table), "symbols")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
