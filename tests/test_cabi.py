"""No GPU needed: the shared library loads and exports every function that
include/seraph_b200.h declares, and the ctypes mirror covers all of them."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    src = open(os.path.join(ROOT, "include", "seraph_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    names = re.findall(r"\b((?:cuda_|seraph_)[a-z0-9_]+)\s*\(", src)
    return sorted(set(n for n in names if not n.endswith("_t")))


def test_library_exports_every_declared_symbol():
    from seraph_b200 import build
    path = build.build()
    lib = ctypes.CDLL(path)
    names = declared_functions()
    assert len(names) > 80
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_ctypes_mirror_covers_the_header():
    from seraph_b200 import api, build
    build.build()
    lib = api.load()
    assert sorted(declared_functions()) == lib._sig_names


def test_init_without_gpu_fails_loudly():
    import pytest
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from seraph_b200 import api, build
    build.build()
    with pytest.raises(RuntimeError):
        api.Context(0)
