"""The reference's known-answer cases, run unchanged against the CUDA path."""
import pytest

from golden import reference_cases as rc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", rc.ALL_CASES, ids=lambda c: c.__name__)
def test_cuda_path_matches_reference_literals(case, xp_gpu):
    case(xp_gpu)
