"""Shared pytest set-up: the `gpu` marker, import paths, per-case seeding and the
deterministic `--random-sample=N` sub-sampling the reference's conftest offers
(tests/conftest.py:44-88 in the reference)."""
import os
import random
import sys
import zlib

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "flash-attention-npu_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_addoption(parser):
    parser.addoption("--random-sample", type=int, default=0,
                     help="keep at most N parametrised cases per test function (seeded)")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    n = config.getoption("--random-sample")
    if n and n > 0:
        groups = {}
        for it in items:
            groups.setdefault(it.nodeid.split("[")[0], []).append(it)
        keep = set()
        rng = random.Random(int(os.environ.get("CI_RANDOM_SEED", "0")))
        for _, lst in sorted(groups.items()):
            chosen = lst if len(lst) <= n else rng.sample(lst, n)
            keep.update(id(x) for x in chosen)
        items[:] = [it for it in items if id(it) in keep]
    if not torch.cuda.is_available():
        skip = pytest.mark.skip(reason="no CUDA device")
        for it in items:
            if "gpu" in it.keywords:
                it.add_marker(skip)


@pytest.fixture(autouse=True)
def _seed_per_case(request):
    seed = int(os.environ.get("CI_TORCH_SEED", zlib.crc32(request.node.nodeid.encode()) & 0x7FFFFFFF))
    torch.manual_seed(seed)
    yield
