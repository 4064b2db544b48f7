"""Pins the CPU oracle against every known-answer constant that the reference's
own tests hold for the hot path (tests/golden/ref_kats.json)."""
import pytest

import kat_runner


@pytest.mark.parametrize("name", kat_runner.CASES)
def test_oracle_matches_reference_kat(zo, name):
    kat_runner.run_case(zo, name)
