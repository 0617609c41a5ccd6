"""The host planners still produce the pinned tables (tests/golden/plan_pins.json, written
by tests/golden/make_plan_pins.py): the tables fix every factor entry's summation order."""

import json
import sys
from pathlib import Path

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))


def test_planners_reproduce_the_pinned_tables():
    from make_plan_pins import pins

    want = json.loads((GOLDEN / "plan_pins.json").read_text())
    got = pins()
    assert sorted(got) == sorted(want)
    assert [k for k in want if got[k] != want[k]] == []
