"""The C-ABI library loads on a machine without a GPU and exports every declared symbol."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    names = set()
    for header in (ROOT / "include").glob("*.h"):
        text = re.sub(r"/\*.*?\*/", " ", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b(evox_\w+)\s*\(", text))
    return sorted(names)


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "evox_pso_step" in names and "evox_last_error" in names


@pytest.mark.parametrize("name", declared_symbols())
def test_symbol_exported(name):
    from evox_b200 import _build

    lib = ctypes.CDLL(str(_build.LIB_PATH))
    assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_prototypes_parsed_for_all():
    from evox_b200 import _cabi

    assert set(_cabi.PROTOTYPES) == set(declared_symbols())


def test_error_string_and_argument_check():
    from evox_b200 import _cabi

    # pop_size = 0 is rejected on the host before anything touches a device
    rc = _cabi.lib.evox_pso_fill_uniform(None, 0, 4, 1, 0, 0, 0, None)
    assert rc == -1
    assert b"pop_size" in _cabi.lib.evox_last_error()
    with pytest.raises(_cabi.EvoxKernelError):
        _cabi.check(rc)


def test_no_cpu_path():
    import torch

    from evox_b200 import _cabi
    from evox_b200.problems.numerical import Ackley

    with pytest.raises(_cabi.EvoxKernelError):
        Ackley().evaluate(torch.zeros(3, 4))
