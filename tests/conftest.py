import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


# the reference's own package (its unmodified BaseWorker, broker and CLI run in some host tests): from the
# local install or the source tree, whichever exists; None where this checkout has neither
REFERENCE = next((p for p in (os.path.join(ROOT, "baseline", "_ref"), "/root/reference")
                  if os.path.isdir(os.path.join(p, "llmq"))), None)
needs_reference = pytest.mark.skipif(REFERENCE is None, reason="the reference llmq package is not available here")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu under gpurun)")


@pytest.fixture(scope="session")
def cuda():
    import torch

    assert torch.cuda.is_available(), "gpu-marked test started without a CUDA device"
    from llmq_b200 import lib

    lib.require_device()  # fails loudly if libb200q.so is missing or the GPU is not sm_100
    return torch.device("cuda", 0)
