"""Test configuration: markers and the automatic skip of GPU tests on machines without CUDA."""

import dataclasses

import pytest
import torch

from moeflow_b200 import MoEConfig


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs one CUDA GPU (B200, sm_100a)")
    config.addinivalue_line("markers", "multigpu: needs >= 2 GPUs; launched as child processes")
    config.addinivalue_line("markers", "slow: full-size shapes (hidden 4096 / 288 experts)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords or "multigpu" in item.keywords:
            item.add_marker(skip)


#: Small layer used by most CPU tests.
SMALL = MoEConfig(hidden_size=64, moe_intermediate_size=32, n_routed_experts=8, top_k=2)
#: Smallest layer the CUDA backend accepts (128-multiples), used by GPU tests.
SMALL_GPU = MoEConfig(hidden_size=256, moe_intermediate_size=128, n_routed_experts=8, top_k=2)


@pytest.fixture
def small_cfg():
    return SMALL


@pytest.fixture
def small_gpu_cfg():
    return SMALL_GPU


def replace(cfg, **kw):
    return dataclasses.replace(cfg, **kw)
