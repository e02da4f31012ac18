"""Pins the CPU oracle to the reference: every known-answer case transcribed from the
reference's test suite (tests/golden/reference_cases.py) must hold for the oracle."""
import pytest

from golden import reference_cases as rc
from oracle_narray import OracleXP


@pytest.mark.parametrize("case", rc.ALL_CASES, ids=lambda c: c.__name__)
def test_oracle_matches_reference_literals(case):
    case(OracleXP)
