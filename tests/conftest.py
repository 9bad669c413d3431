import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    """The package over the in-tree C-ABI library (built on demand; nvcc cross-compiles without a GPU)."""
    mod = entry.load_package()
    if not os.path.exists(mod.LIB_PATH):
        entry.build()
    mod.lib()
    return mod


@pytest.fixture(scope="session")
def orc():
    """The CPU checker."""
    mod = entry.load_oracle()
    try:
        mod.lib()
    except ImportError:
        entry._load_script(os.path.join(ROOT, "oracle", "build_oracle.py"), "tc_oracle_build").build_all()
        mod.lib()
    return mod


# The five benchmark configurations (expression, numpy dtype name, seed).
CONFIGS = [
    ("C [i,64,j,48,k,32] += sum(l,40) * A [l,k,i] * B [j,l];", "float64", 0),
    ("C [a,96,b,96,c,96,d,96] += sum(e,96) * A [a,e,b,d] * B [e,c];", "float64", 1),
    ("C [a,64,b,64,c,64,d,64] += sum(e,64,f,64) * A [e,c,a,f] * B [b,f,d,e];", "float64", 2),
    ("C [a,24,b,24,c,24,i,24,j,24,k,24] += sum(l,24) * A [l,a,i,j] * B [b,c,k,l];", "float32", 3),
    ("C [a,40,b,40,c,40,d,40,e,40,f,40] += sum(g,40) * A [g,a,b,c] * B [d,e,f,g];", "float64", 4),
]

# Tolerances: max|got-ref| / max|ref| (fp64 1e-12, fp32 1e-5, inputs uniform[-1,1)).
TOL = {"float64": 1e-12, "float32": 1e-5}
