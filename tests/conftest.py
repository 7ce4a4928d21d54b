import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch


@pytest.fixture(scope="session")
def pa():
    """The engine's Python mirror; building the library is the job of __graft_entry__.build()."""
    import paged_attention_b200
    return paged_attention_b200


@pytest.fixture(autouse=True)
def fixed_cut(request):
    """Most tests compare outputs bit for bit between entry points or between steps, so they run with the
    adaptive cut (shares that follow measured per-CTA rates) switched off; tests of the adaptive cut itself
    switch it on."""
    if "pa" not in request.fixturenames:
        yield
        return
    pa = request.getfixturevalue("pa")
    before = pa.adaptive_cut()
    pa.set_adaptive_cut(False)
    yield
    pa.set_adaptive_cut(before)
