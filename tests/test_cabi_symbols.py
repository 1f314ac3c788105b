"""The C-ABI library loads (no GPU needed) and exports every function that include/mok_b200.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "mok_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mokb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = ctypes.CDLL(os.path.join(ROOT, "mixture-of-kittens_b200", "mok", "libmok_b200.so"))
    names = declared_functions()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/mok_b200.h but not exported"


def test_binding_matches_header():
    from mok import _C, _C_mxfp8
    bound = set(_C.EXPORTED) | set(_C_mxfp8.EXPORTED)
    assert bound <= set(declared_functions()), bound - set(declared_functions())
    missing = set(declared_functions()) - bound
    assert not missing, f"declared but not bound in mok/_C.py: {missing}"


def test_argument_errors_without_a_gpu():
    from mok import _C
    lib = _C.lib
    assert lib.mokb_schedule_scratch_bytes(8, 32) > 8 * 32 * 1024 * 4
    assert lib.mokb_layer_scratch_bytes(1024, 4, 1024) > 0
    rc = lib.mokb_mxfp8_quantize(None, 1, 128, 128, None, None, None, None, None)
    assert rc == -1 and b"null input" in _C._last_error()
    rc = lib.mokb_schedule(None, 1, 512, 2, 4, 2048, 0, None, None, None, None, None, None, None)
    assert rc == -1 and b"null pointer" in _C._last_error()
