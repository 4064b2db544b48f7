"""Pins the CPU oracle against every known-answer constant that the reference's
own tests hold for the hot path (tests/golden/ref_kats.json)."""
import pytest

import kat_runner


@pytest.mark.parametrize("name", kat_runner.CASES)
def test_oracle_matches_reference_kat(zo, name):
    kat_runner.run_case(zo, name)


def test_adam_multi_step_property(zo):
    """src/optim.zig:189-216: weight 1.0 with gradient 0.2 goes down on each of two Adam steps (lr 0.01)."""
    import numpy as np
    w = np.array([1.0], np.float32)
    g = np.array([0.2], np.float32)
    m, v = np.zeros(1, np.float32), np.zeros(1, np.float32)
    zo.adam_step(w, g, m, v, 0.01, 0.9, 0.999, 1e-8, 1.0)
    after1 = float(w[0])
    assert after1 < 1.0
    # first step of Adam moves by lr whatever the gradient's size: 1 - 0.01 up to eps
    assert abs(after1 - 0.99) < 1e-6
    zo.adam_step(w, g, m, v, 0.01, 0.9, 0.999, 1e-8, 2.0)
    assert float(w[0]) < after1
