"""The sorting of time stamps into launches (bench.py --timeline), on made-up records."""
import importlib.util
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_for_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_records_of_ctas_become_launches_in_the_order_of_their_wakes():
    b = _bench()
    # (start, wake, first data, end, kind, grid): two launches of a 2-CTA kernel around one of a 3-CTA kernel;
    # the second kernel's CTAs start before the first launch has ended, as they do under programmatic launch
    recs = [(100, 110, 0, 150, 20, 2), (101, 111, 120, 160, 20, 2),
            (140, 170, 0, 180, 10, 3), (141, 171, 0, 185, 10, 3), (142, 169, 0, 181, 10, 3),
            (175, 190, 195, 230, 20, 2), (176, 191, 0, 240, 20, 2)]
    rows = b.timeline_launches(list(reversed(recs)))
    assert [(r["kind"], r["grid"]) for r in rows] == [(20, 2), (10, 3), (20, 2)]
    assert rows[0]["start"] == 100 and rows[0]["wake"] == 110 and rows[0]["data"] == 120 and rows[0]["first_end"] == 150 and rows[0]["end"] == 160
    assert rows[1]["wake"] == 169 and rows[1]["data"] == 0 and rows[1]["end"] == 185
    assert rows[2]["wake"] == 190 and rows[2]["end"] == 240


def test_a_launch_with_records_missing_is_left_out():
    b = _bench()
    recs = [(100, 110, 0, 150, 30, 4), (101, 111, 0, 151, 30, 4), (200, 210, 0, 250, 31, 1)]
    rows = b.timeline_launches(recs)
    assert [(r["kind"], r["grid"]) for r in rows] == [(31, 1)]
