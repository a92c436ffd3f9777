"""Every series a dashboard panel queries is exported by a live (mock-backend) server or by the router."""
import json
import os

from rexl3_b200 import dashboard_check

PANELS = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "dashboard", "panels.json")


def test_panel_catalogue_matches_the_exported_series():
    assert dashboard_check.check(PANELS) == {}


def test_a_panel_with_an_unknown_series_is_reported(tmp_path):
    doc = json.load(open(PANELS))
    doc["panels"].append({"title": "Bogus", "queries": ["rate(rexl3_no_such_series_total[1m])"]})
    p = tmp_path / "panels.json"
    p.write_text(json.dumps(doc))
    assert dashboard_check.check(str(p), exported={"rexl3_requests_total"})["Bogus"] == ["rexl3_no_such_series_total"]
