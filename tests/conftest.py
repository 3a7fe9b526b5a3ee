import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def pkg():
    from __graft_entry__ import load_package
    return load_package()


@pytest.fixture(scope="session", params=["tcgen05", "mma"])
def ctx(pkg, request):
    """One context per decode path: the tcgen05 streaming kernels and the mma.sync streaming kernels."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    # DSUF_TEST_PDL=1 runs the whole suite with programmatic dependent launch on (every kernel waits for its predecessor
    # with griddepcontrol.wait before it reads anything, so the results must not change)
    c = pkg.Ctx(0, tcgen05=request.param == "tcgen05", pdl=os.environ.get("DSUF_TEST_PDL", "0") == "1")
    yield c
    c.close()


def seeded(seed):
    import torch
    return torch.Generator().manual_seed(seed)


def randn_bf16(gen, *shape, std=1.0):
    """bf16 normal tensor as (torch bf16 tensor, uint16 numpy view)."""
    import torch
    t = (torch.randn(*shape, generator=gen) * std).bfloat16()
    return t, t.view(torch.uint16).numpy()
