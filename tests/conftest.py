import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pkg():
    """The product package, imported under the name dsv41_b200 (built first if the library is missing)."""
    import __graft_entry__ as g
    if not os.path.exists(os.path.join(g.PKG_DIR, "csrc", "libb200moe.so")):
        g.build()
    return g.load_package()


@pytest.fixture(scope="session")
def mods(pkg):
    import importlib

    class M:
        pass

    m = M()
    for name in ("_lib", "quant", "kernels", "moe_kernels", "fused", "fused2", "cukern", "w8", "ep", "moe", "synth"):
        setattr(m, name.lstrip("_") if name != "_lib" else "lib", importlib.import_module(f"dsv41_b200.{name}"))
    return m


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def dev():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def rel_err(a, b):
    """max |a - b| / max |b|: the error measure of the reference's kernel tests (dsv41/test_kernels.py:18)."""
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).abs().max() / (b.abs().max() + 1e-30)).item()
