import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def golden():
    import torch

    return torch.load(os.path.join(ROOT, "tests", "golden", "reference_vectors.pt"), weights_only=False)


@pytest.fixture(scope="session")
def golden_regularized():
    import torch

    return torch.load(os.path.join(ROOT, "tests", "golden", "reference_vectors_regularized.pt"), weights_only=False)


@pytest.fixture(scope="session")
def golden_periodic():
    import torch

    return torch.load(os.path.join(ROOT, "tests", "golden", "reference_vectors_periodic.pt"), weights_only=False)


@pytest.fixture(scope="session")
def golden_attentive():
    import torch

    return torch.load(os.path.join(ROOT, "tests", "golden", "reference_vectors_attentive.pt"), weights_only=False)


@pytest.fixture(scope="session")
def golden_fullwidth():
    import torch

    return torch.load(os.path.join(ROOT, "tests", "golden", "reference_vectors_fullwidth.pt"), weights_only=False)


@pytest.fixture(scope="session")
def golden_condensed_priors():
    import torch

    return torch.load(os.path.join(ROOT, "tests", "golden", "reference_vectors_condensed_priors.pt"), weights_only=False)


@pytest.fixture(scope="session")
def golden_priors_periodic():
    import torch

    return torch.load(os.path.join(ROOT, "tests", "golden", "reference_vectors_priors_periodic.pt"), weights_only=False)
