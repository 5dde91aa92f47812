import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


def pytest_collection_modifyitems(config, items):
    # Tests marked gpu are skipped (not failed) on a machine without CUDA, whatever -m says.
    try:
        import torch
        have = torch.cuda.is_available()
        ndev = torch.cuda.device_count() if have else 0
    except Exception:
        have, ndev = False, 0
    for it in items:
        if "gpu" in it.keywords and not have:
            it.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in it.keywords and ndev < 2:
            it.add_marker(pytest.mark.skip(reason="needs >= 2 CUDA devices"))


@pytest.fixture(scope="session")
def cuda_lib():
    """The CUDA library for tests that only call its HOST functions (no GPU needed): built in tree on first use,
    skipped where there is no nvcc."""
    import shutil

    from fp4_all_reduce_b200 import _native as N
    from fp4_all_reduce_b200 import build as B

    if not N.cuda_library_path().exists():
        if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
            pytest.skip("libfp4ar.so is not built and there is no nvcc to build it")
        B.build_cuda()
        N.cuda.cache_clear()
    return N.cuda()
