import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on the B200 box only)")


class Fixture:
    """One reference single-op golden case: inputs, outputs (bf16 as uint16 bits), node attributes."""

    def __init__(self, pack, name):
        self.name = name
        self.nodes = json.loads(bytes(pack[f"{name}/nodes"]).decode())
        self.inputs, self.outputs, self.in_dtypes = [], [], []
        i = 0
        while f"{name}/input_{i}" in pack:
            self.inputs.append(pack[f"{name}/input_{i}"])
            self.in_dtypes.append(int(pack[f"{name}/input_{i}/dtype"]))
            i += 1
        i = 0
        while f"{name}/output_{i}" in pack:
            self.outputs.append(pack[f"{name}/output_{i}"])
            i += 1

    def attr(self, key, default=None):
        return self.nodes[0][1].get(key, default)


@pytest.fixture(scope="session")
def single_op():
    pack = np.load(os.path.join(GOLDEN, "single_op.npz"))
    return lambda name: Fixture(pack, name)


@pytest.fixture(scope="session")
def tiny_llama():
    z = np.load(os.path.join(GOLDEN, "tiny_llama_random.npz"))
    cfg = json.loads(bytes(z["config"]).decode())
    meta = {"config", "prompt_ids", "prompt_ids_world", "expected_new_ids"}
    weights = {k: z[k] for k in z.files if k not in meta}
    return cfg, weights, z["prompt_ids"], z["prompt_ids_world"], z["expected_new_ids"]


def eq_with_epsilon(actual, expected, eps):
    """The reference's comparison rule ``CompPolicy::Either``: |a-e| < eps OR |a-e|/|e| < eps per element
    (src/tensor/data.rs:70-101 of the reference)."""
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    diff = np.abs(a - e)
    with np.errstate(divide="ignore", invalid="ignore"):
        rel = diff / np.abs(e)
    ok = (diff < eps) | (rel < eps)
    return bool(ok.all()), float(diff.max()) if diff.size else 0.0
