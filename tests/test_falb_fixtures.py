"""The reference's own model fixtures, in both of its formats, through this library.

Each fixture directory holds the same model as LightGBM-style text (``model.txt``) and in the FALB binary
container (``model.falb``), a feature matrix ``X.npy`` and the reference's predictions ``preds.npy``. The
tests skip cleanly when the reference tree is not mounted.
"""
import os
from pathlib import Path

import numpy as np
import pytest

import falcata_b200 as fb

FIXTURES = Path(os.environ.get("FALCATA_REFERENCE_DIR", "/root/reference")) / "tests" / "gates" / "falb_fixtures"
NAMES = sorted(p.name for p in FIXTURES.iterdir() if (p / "model.falb").exists()) if FIXTURES.is_dir() else []
pytestmark = pytest.mark.skipif(not NAMES, reason="reference fixtures are not mounted")


def _expected(d: Path, bst, X):
    want = np.load(d / "preds.npy")
    got = bst.predict(X)
    return got.reshape(want.shape), want


@pytest.mark.parametrize("name", NAMES)
def test_text_fixture_predicts_and_round_trips(name):
    d = FIXTURES / name
    text = (d / "model.txt").read_text()
    bst = fb.Booster(model_file=d / "model.txt")
    got, want = _expected(d, bst, np.load(d / "X.npy"))
    np.testing.assert_array_equal(got, want)
    assert bst.model_to_string() == text


@pytest.mark.parametrize("name", NAMES)
def test_binary_fixture_loads_and_predicts_like_the_reference(name):
    d = FIXTURES / name
    bst = fb.Booster(model_file=d / "model.falb")
    got, want = _expected(d, bst, np.load(d / "X.npy"))
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("name", NAMES)
def test_binary_written_here_matches_the_fixture(name):
    """Same model in, same container out: the file written from the text model is the reference's file
    (same sections, element types, dictionaries and zlib streams), or at least of the same size."""
    d = FIXTURES / name
    ref = (d / "model.falb").read_bytes()
    mine = fb.Booster(model_file=d / "model.txt").model_to_binary()
    assert mine[:32] == ref[:32]                       # header: magic, version, flags, tree and section counts
    assert abs(len(mine) - len(ref)) <= 0.03 * len(ref)
    assert mine == ref[: len(mine)]                    # and in fact every byte of the container (zlib level 6 on the same planes)
    assert ref[len(mine):] == b"\npandas_categorical:null\n"   # what the Python layer appends to a saved file
    back = fb.Booster.from_binary(mine)
    X = np.load(d / "X.npy")
    np.testing.assert_array_equal(back.predict(X), fb.Booster(model_file=d / "model.txt").predict(X))


def test_saved_file_is_the_reference_file(tmp_path):
    d = FIXTURES / NAMES[0]
    out = tmp_path / "m.falb"
    fb.Booster(model_file=d / "model.txt").save_model(out, format="falb")
    assert out.read_bytes() == (d / "model.falb").read_bytes()


def test_unknown_capability_bits_and_reserved_codec_are_refused():
    d = FIXTURES / NAMES[0]
    blob = bytearray((d / "model.falb").read_bytes())
    bad = bytearray(blob); bad[8 + 1] |= 0x80   # a flag bit no reader knows
    with pytest.raises(fb.FalcataError):
        fb.Booster.from_binary(bytes(bad))
    bad = bytearray(blob); bad[32 + 8] = 1      # first section's codec -> the reserved value
    with pytest.raises(fb.FalcataError):
        fb.Booster.from_binary(bytes(bad))
    with pytest.raises(fb.FalcataError):
        fb.Booster.from_binary(bytes(blob[: len(blob) // 2]))   # truncated


def test_contributions_need_the_statistics_section():
    d = FIXTURES / "binary"
    X = np.load(d / "X.npy")
    full = fb.Booster(model_file=d / "model.txt")
    lean = fb.Booster.from_binary(full.model_to_binary())
    with pytest.raises(fb.FalcataError):
        lean.predict(X[:4], pred_contrib=True)
    rich = fb.Booster.from_binary(full.model_to_binary(with_stats=True, with_diagnostics=True))
    np.testing.assert_allclose(rich.predict(X[:16], pred_contrib=True), full.predict(X[:16], pred_contrib=True), rtol=0, atol=1e-12)
    assert rich.model_to_string() == full.model_to_string()
