"""LoRA adapter files, host side (no GPU needed): version 2 equals the reference's lora_save byte for byte and is read
back by the reference's lora_load; version 3 keeps the adapters and Adam moments that format drops."""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as O
from oracle_lib import TINY


def make_state(mask, seed, rank=4, alpha=8.0):
    from seraph_b200 import api
    cfg = TINY
    st = api.TrainState(cfg, cfg.init_params(seed))
    n = cfg.lora_tensors(rank, mask)[1]
    st.attach_lora(rank, alpha, mask, (0.05 * np.random.default_rng(seed).standard_normal(n)).astype(np.float32))
    return st


@pytest.mark.parametrize("mask", [0b0000101, 0b1111111, 0b0000001])
def test_version2_is_the_reference_format_byte_for_byte(tmp_path, mask):
    ref = O.ref_lib("cpu")
    if ref is None:
        pytest.skip("oracle/_ref not built (no reference checkout)")
    st = make_state(mask, 3)
    ours, theirs = str(tmp_path / "ours.bin"), str(tmp_path / "theirs.bin")
    assert st.lib.seraph_b200_lora_save(None, st.h, ours.encode(), 2, 0) == 0
    ref.lora_save.restype, ref.lora_save.argtypes = C.c_int, [C.c_void_p, C.c_char_p]
    assert ref.lora_save(st.lora_ptr(), theirs.encode()) == 0
    a, b = open(ours, "rb").read(), open(theirs, "rb").read()
    assert a == b and a[:4] == b"AROL" and int.from_bytes(a[4:8], "little") == 2
    # the reference's own loader reads our file back to the same Q and V adapters
    ref.lora_load.restype, ref.lora_load.argtypes = C.c_void_p, [C.c_char_p]
    m = ref.lora_load(ours.encode())
    assert m
    # our loader: perturb the host adapters, load, and the Q/V adapters are the saved ones again (others untouched)
    before = st.lora_get(0)
    st2 = make_state(mask, 4)
    other = st2.lora_get(0)
    assert st2.lib.seraph_b200_lora_load(None, st2.h, ours.encode()) == 0
    after = st2.lora_get(0)
    tens, _ = TINY.lora_tensors(4, mask)
    for name, shp, off in tens:
        n = int(np.prod(shp))
        in_file = ".q." in name or ".v." in name
        want = before if in_file else other
        assert np.array_equal(after[off:off + n], want[off:off + n]), name
    st.close(); st2.close()


def test_version3_keeps_every_adapter_and_the_moments(tmp_path):
    mask = 0b1111111
    st = make_state(mask, 5)
    path = str(tmp_path / "v3.bin")
    st.set_counters(17, 0)
    assert st.lib.seraph_b200_lora_save(None, st.h, path.encode(), 3, 1) == 0
    st2 = make_state(mask, 6)
    assert st2.lib.seraph_b200_lora_load(None, st2.h, path.encode()) == 0
    for which in range(4):
        if which == 1:
            continue                                   # gradients are not part of a checkpoint
        assert np.array_equal(st.lora_get(which), st2.lora_get(which))
    assert st2.counters()[0] == 17
    # shape or rank mismatch is refused
    st3 = make_state(mask, 7, rank=2)
    assert st3.lib.seraph_b200_lora_load(None, st3.h, path.encode()) != 0
    assert st3.lib.seraph_b200_lora_load(None, st3.h, str(tmp_path / "missing.bin").encode()) != 0
    st.close(); st2.close(); st3.close()
