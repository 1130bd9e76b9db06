import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as ge
    return ge.load_package()


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def ctx(pkg):
    """A context on cuda:0 bound to a non-default stream shared with torch."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    c = pkg.Context(0, stream)
    c.torch_stream = stream
    yield c
    c.close()


@pytest.fixture()
def dev(ctx):
    """Helper to move numpy arrays to the GPU and back, ordered with the context's stream."""
    import numpy as np
    import torch

    class Dev:
        def to(self, a):
            t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
            torch.cuda.synchronize()
            return t

        def empty(self, shape, dtype=torch.float32):
            return torch.empty(shape, dtype=dtype, device="cuda")

        def full(self, shape, val):
            t = torch.full(shape, val, dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()  # the fill ran on torch's stream, not the context's
            return t

        def back(self, t):
            ctx.sync_check()
            return t.cpu().numpy()

    return Dev()
