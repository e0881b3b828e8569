import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Makes (and caches for the session) random-weight model folders in a temporary place."""
    from tests import helpers

    cache = {}

    def get(name: str, cfgd: dict, seed: int, dtype: str, **kw):
        key = (name, seed, dtype, tuple(sorted(kw.items())))
        if key not in cache:
            out = tmp_path_factory.mktemp(f"{name}-{dtype}-{seed}")
            cache[key] = helpers.make_folder(cfgd, str(out), seed, dtype, **kw)
        return cache[key]

    return get


@pytest.fixture(scope="session", autouse=True)
def sparse_comparisons_compare_enough():
    """After the last test: no bf16 comparison of a model with sparse attention may have passed on near ties alone."""
    yield
    from tests import helpers

    helpers.check_sparse_rows_kept()
