import pathlib
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


def pytest_collection_modifyitems(config, items):
    # GPU tests fail loudly without a device instead of skipping: a silent skip would read as a pass.
    pass


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Factory of model folders with seeded random weights, made once per (config, dtype, flavour)."""
    from helpers import make_model_dir
    made = {}

    def get(name, dtype="float32", flavour="scaled", seed=1):
        key = (name, dtype, flavour, seed)
        if key not in made:
            made[key] = make_model_dir(tmp_path_factory.mktemp(f"{name}_{dtype}_{flavour}"), name, dtype,
                                       flavour, seed)
        return made[key]
    return get
