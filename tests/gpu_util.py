"""Helpers shared by the GPU parity tests (all calls go through the C ABI)."""
import importlib

import numpy as np
import pytest

bridge = importlib.import_module("large-language-model_b200.bridge")
synth = importlib.import_module("large-language-model_b200.synth")

FP32_TOL = 1e-4   # rel-err gate of the fp32 path
BF16_TOL = 2e-2   # rel-err gate for bf16 outputs and gradients


def rel(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-30))


@pytest.fixture(scope="module")
def ctx():
    c = bridge.Context(0)
    yield c
    c.close()
