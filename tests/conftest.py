import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture()
def ref_models():
    """The reference's ``custom_models.sparse_models`` module, imported from the files staged
    under ``oracle/_ref`` (see oracle/make_ref.py) on top of this repository's drop-in kernel
    modules; tests that need it skip where the files are absent."""
    import contextlib
    import io

    from oracle import make_ref
    make_ref.stage(verbose=False)
    if not make_ref.available():
        pytest.skip("reference callers not staged under oracle/_ref")
    from sparser_faster_llms_b200 import dropin
    keep = ("custom_models", "benchmark_inference", "benchmark_base", "energy_utils")
    saved = {k: v for k, v in sys.modules.items() if k.split(".")[0] in keep}
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, make_ref.import_path())
    dropin.install()
    try:
        with contextlib.redirect_stdout(io.StringIO()):
            from custom_models import sparse_models
        yield sparse_models
    finally:
        sys.path.remove(make_ref.import_path())
        dropin.uninstall()
        for k in [k for k in sys.modules if k.split(".")[0] in keep]:
            del sys.modules[k]
        sys.modules.update(saved)
