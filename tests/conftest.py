import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


@pytest.fixture(scope="session")
def golden_small():
    import json
    import numpy as np
    z = np.load(os.path.join(ROOT, "tests", "golden", "small_cases.npz"))
    meta = json.loads(bytes(z["meta"]).decode())
    cases = {}
    for name, m in meta.items():
        cases[name] = {k: z[f"{name}.{k}"] for k in ("values", "rewards", "dones", "importance", "advantages")}
        cases[name]["hyper"] = tuple(m["hyper"])
    return cases


@pytest.fixture(scope="session")
def config_digests():
    import json
    with open(os.path.join(ROOT, "tests", "golden", "config_digests.json")) as f:
        return json.load(f)
