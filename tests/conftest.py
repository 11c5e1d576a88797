import os
import sys

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(os.path.join(GOLDEN, name))

    return load


@pytest.fixture(scope="session")
def ref_silu_table():
    """The reference's own silu_table[] (fixture written by tests/golden/make_golden.py)."""
    return np.fromfile(os.path.join(GOLDEN, "silu_table_ref.f32"), dtype=np.float32)


@pytest.fixture(scope="session")
def layer0():
    from tie_b200 import synth, workloads

    return synth.make_layer(workloads.BASE_SEED)


@pytest.fixture(scope="session")
def small_shape():
    from tie_b200 import synth

    return synth.MoeShape(hidden=512, n_expert=32, top_k=4, ffn_dim=256)


@pytest.fixture(scope="session")
def small_layer(small_shape):
    from tie_b200 import synth, workloads

    return synth.make_layer(workloads.BASE_SEED + 1, small_shape)


@pytest.fixture(scope="session")
def port_lib():
    from oracle import port

    port.build()
    return port
