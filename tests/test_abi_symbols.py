"""The C-ABI library loads without a GPU and exports every symbol its header declares."""

import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from packboost_b200 import build
    build.build()
    from packboost_b200 import backends as B
    return B.lib()


def _declared():
    text = open(os.path.join(ROOT, "include", "packboost_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), n


def test_binding_covers_the_header():
    from packboost_b200 import backends as B
    assert set(_declared()) == set(B.EXPORTED_SYMBOLS)


def test_struct_mirror_and_probes(lib):
    from packboost_b200 import backends as B
    assert lib.pb_train_state_bytes() == C.sizeof(B.TrainState)
    assert lib.pb_abi_version() == 1
    assert lib.pb_ctl_bytes() > 0
    assert lib.pb_device_count() >= 0          # 0 on a box without a GPU, never an exception
    assert B.cpu_available() is False


def test_argument_errors_do_not_need_a_gpu(lib):
    from packboost_b200 import backends as B
    st = B.TrainState()
    with pytest.raises(ValueError):
        B.check(lib.pb_round_begin(C.byref(st), 0, None))
    assert b"n_rows" in lib.pb_last_error()
    with pytest.raises(ValueError):
        B.check(lib.pb_pack_rows(None, 0, 1, 1, None, 0, 5, None, 16, 4, None))
    for fn in (B.find_best_splits_batched_cuda, B.partition_frontier_cuda):
        with pytest.raises(RuntimeError, match="superseded"):
            fn()
    with pytest.raises(RuntimeError, match="unavailable"):
        B.find_best_splits_batched()
