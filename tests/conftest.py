import os
import sys

import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def tiny_model_dirs(tmp_path_factory):
    """Model folders of the two tiny configurations, written once per session into a temporary folder."""
    import torch
    from ember_b200.weights import write_model_dir
    from tests.tiny_configs import TINY, tiny_config
    out = {}
    for name in TINY:
        d = str(tmp_path_factory.mktemp(f"tiny_{name}"))
        write_model_dir(tiny_config(name), d, seed=TINY[name]["seed"], dtype=torch.bfloat16,
                        std=TINY[name]["std"], norm_std=TINY[name]["norm_std"])
        out[name] = d
    return out
