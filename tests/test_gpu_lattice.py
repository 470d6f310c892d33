"""The regression lattice and a short fuzz run on the device."""
import os
import sys

import pytest

pytestmark = pytest.mark.gpu
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "gates"))


def test_lattice_on_the_device_matches_the_stored_fingerprints_and_equalities():
    import lattice

    assert lattice.main(["--check", "--device", "cuda"]) == 0


def test_fuzz_gate_on_the_device():
    import fuzz

    assert fuzz.main(["--specs", "8", "--seed", "3", "--device", "cuda"]) == 0
