import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def free_port() -> int:
    """A TCP port that is free right now (the machine is shared: no fixed rendezvous ports)."""
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def single_rank_group():
    """A 1-rank gloo process group: the layer constructors read rank / world size from it."""
    import torch.distributed as dist
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(free_port()))
        dist.init_process_group("gloo", rank=0, world_size=1)
    yield
    # left initialised for the rest of the session; destroyed at interpreter exit


@pytest.fixture(scope="session")
def built_library():
    """Builds (if stale) and returns the path of libnq_fp8.so."""
    from nano_qwen_b200 import build
    return build.build()
