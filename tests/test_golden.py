"""The plain implementation against the reference's own golden logits (see
tests/golden/make_golden.py for what they are and what they anchor)."""
import json
import os

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE = os.environ.get("FERROX_REFERENCE", "")   # a checkout of the reference, when one is at hand


def _load():
    with open(os.path.join(HERE, "golden", "ferrox_fixture_logits.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("fixture", ["dense", "moe", "mixed"])
def test_committed_plain_logits_match_the_reference_constants(fixture):
    v = _load()[fixture]
    assert len(v["plain_logits"]) == len(v["reference_logits"]) == 32
    # the reference's own tolerance for these constants is 1e-4 (gguf_roundtrip.rs:43)
    assert max(abs(a - b) for a, b in zip(v["plain_logits"], v["reference_logits"])) < 1e-5


@pytest.mark.skipif(not REFERENCE or not os.path.isdir(os.path.join(REFERENCE, "crates/ferrox-models/tests/fixtures")),
                    reason="FERROX_REFERENCE does not name a checkout of the reference")
def test_recomputed_from_the_reference_fixtures():
    import sys

    sys.path.insert(0, os.path.join(HERE, "golden"))
    import make_golden

    fresh, committed = make_golden.compute(REFERENCE), _load()
    for k in committed:
        assert fresh[k]["reference_logits"] == committed[k]["reference_logits"]
        assert max(abs(a - b) for a, b in zip(fresh[k]["plain_logits"], committed[k]["plain_logits"])) < 1e-6
