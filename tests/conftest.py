import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
for p in (ROOT, GOLDEN):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_layers():
    return np.load(os.path.join(GOLDEN, "layers.npz"))


@pytest.fixture(scope="session")
def golden_quantizer():
    return np.load(os.path.join(GOLDEN, "quantizer.npz"))


@pytest.fixture(scope="session")
def golden_unet():
    return np.load(os.path.join(GOLDEN, "unet.npz"))


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def golden_sens():
    return np.load(os.path.join(GOLDEN, "sens.npz"))


# A free-running modulated evaluation is compared with the reference's stored output.  How close
# two exact implementations can be is MEASURED, not guessed: sens.npz holds, per case and
# evaluation, the PSNR between two runs of the reference itself that differ only by a
# perturbation of 1e-4 of the range on the first evaluation's output (tests/golden/cases.py,
# SENS_REL).  The CUDA path's own first-evaluation difference is below that perturbation, so it
# must stay within SENS_MARGIN_DB of the reference's self-agreement at every later evaluation.
SENS_MARGIN_DB = 6.0


def sens_floor(golden_sens, name, k):
    return float(golden_sens[name + "/sens_db"][k]) - SENS_MARGIN_DB
