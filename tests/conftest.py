import os
import sys
import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

SEED = 20261125


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def _has_gpu():
    return os.path.exists("/dev/nvidia0") or os.path.exists("/dev/nvidiactl")


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no GPU on this machine")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def clib():
    """The product library through ctypes (host-only entry points work without a GPU)."""
    from maple_runtime_b200 import lib as ml
    if not os.path.exists(ml.LIB_PATH):
        ml.build()
    return ml.load()


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as orc
    return orc.Oracle()


@pytest.fixture(scope="session")
def reference():
    from oracle import oracle as orc
    if not orc.Reference.available():
        pytest.skip("oracle/_ref not built (the reference sources are not on this machine)")
    r = orc.Reference()
    r.threads(min(8, os.cpu_count() or 1))
    return r


class Weights:
    """Synthetic layers from the product's host generator, cached per (seed, layer)."""

    def __init__(self, clib):
        self.clib, self.cache = clib, {}

    def layer(self, L, seed=SEED):
        from maple_runtime_b200 import lib as ml
        k = (seed, L)
        if k not in self.cache:
            self.cache[k] = (ml.synth_router(self.clib, seed, L), ml.synth_norm(self.clib, seed, L),
                             ml.synth_experts(self.clib, seed, L, 0, 256))
        return self.cache[k]

    def hidden(self, stream, nb, seed=SEED):
        from maple_runtime_b200 import lib as ml
        return ml.synth_hidden(self.clib, seed, stream, nb)


@pytest.fixture(scope="session")
def weights(clib):
    return Weights(clib)


@pytest.fixture(scope="session")
def gpu(clib):
    """One initialised library instance for the whole GPU session (the ABI has no teardown)."""
    from maple_runtime_b200 import lib as ml
    g = ml.Gpre(2048)
    g.keep_stages(True)
    # The stage-by-stage tests compare fp32 values bit for bit, which holds on the exact-order router.  The router that batches of
    # 512+ tokens take by default (tensor cores, exact only in its indices) is tested in test_gpu_router_tensor.py and, with every
    # kernel around it, in test_gpu_replay.py; both select it themselves.
    g.set_router(1)
    return g


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint8)


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(bits(a), bits(b))
