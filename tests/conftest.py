"""Shared pytest setup: the `gpu` marker, import paths and cached synthetic layers."""
from __future__ import annotations

import importlib
import importlib.util
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PACKAGE_DIR = ROOT / "aima-amd395-qwen36-35b-linux-engine_b200"
PACKAGE_NAME = "aima_moe_b200"

sys.path.insert(0, str(ROOT / "oracle"))
sys.path.insert(0, str(ROOT / "tests"))


def load_package():
    """Imports the package directory (its name is not an identifier) as aima_moe_b200."""
    if PACKAGE_NAME in sys.modules:
        return sys.modules[PACKAGE_NAME]
    spec = importlib.util.spec_from_file_location(
        PACKAGE_NAME, PACKAGE_DIR / "__init__.py", submodule_search_locations=[str(PACKAGE_DIR)])
    module = importlib.util.module_from_spec(spec)
    sys.modules[PACKAGE_NAME] = module
    spec.loader.exec_module(module)
    return module


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def package():
    return load_package()


@pytest.fixture(scope="session")
def synth(package):
    return package.synth


@pytest.fixture(scope="session")
def oracle():
    import moe_oracle

    moe_oracle.build()
    return moe_oracle


@pytest.fixture(scope="session")
def torch_ref():
    import moe_torch_ref

    return moe_torch_ref


@pytest.fixture(scope="session")
def built_library(package):
    """Path of the CUDA shared library, built on demand (nvcc cross-compiles without a GPU)."""
    spec = importlib.util.spec_from_file_location("aima_moe_b200_build", PACKAGE_DIR / "build.py")
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    return build.build()


SEED = 1234


@pytest.fixture(scope="session")
def gpu_layers(package, built_library):
    """Lazily built full synthetic layers: CUDA tensors + a CPU oracle view, keyed by layer."""
    import torch
    import moe_oracle

    cache: dict[int, dict] = {}

    def get(layer: int) -> dict:
        if layer not in cache:
            device = torch.device("cuda", 0)
            cuda = package.synth.layer_weights_cuda(SEED, layer, device)
            cpu = {name: tensor.cpu() for name, tensor in cuda.items()}
            cache[layer] = {"cuda": cuda, "cpu": cpu, "oracle": moe_oracle.OracleLayer(cpu)}
        return cache[layer]

    return get
