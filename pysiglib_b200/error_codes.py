"""Text for the integer codes returned through the C ABI.

Code table of the reference: ``pysiglib/error_codes.py:16-54`` (codes 1-11 are C++
exception classes, ``100000 + n`` is CUDA error ``n``)."""
from . import load_cusig

CODE_TEXT = {
    1: "Failed to allocate memory",
    2: "Invalid argument",
    3: "Out of range",
    4: "Filesystem error",
    10: "Runtime error",
    11: "Unknown exception",
}


def err_msg(code):
    if code < 100000:
        text = CODE_TEXT.get(code, "Error") + " (" + str(code) + ")"
    else:
        text = "CUDA error (" + str(code - 100000) + ")"
    detail = load_cusig.last_error_message()
    return text + (": " + detail if detail else "")
