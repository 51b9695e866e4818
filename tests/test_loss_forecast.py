"""Curve families, binning and the command line of `analysis/loss_forecast.py` (reference ops/loss_curve_forecast.py:27-150)."""
import json
import math

import numpy as np
import pytest

from warpstate_ai_b200.analysis import loss_forecast as LF


def test_log_family_is_exact_on_its_own_curve():
    t = np.array([1.0, 2.0, 4.0, 8.0, 16.0])
    loss = 3.2 - 0.4 * np.log(t)
    p = LF.fit(t, loss, "log")
    assert p["model"] == "log" and p["intercept"] == pytest.approx(3.2) and p["slope"] == pytest.approx(-0.4)
    assert p["rmse"] < 1e-12
    assert LF.predict(p, [32.0])[0] == pytest.approx(3.2 - 0.4 * math.log(32.0))
    assert LF.crossing(p, 2.0) == pytest.approx(math.exp(3.0))              # 3.2 - 0.4 ln t = 2
    rising = LF.fit(t, 3.0 + 0.1 * np.log(t), "log")
    assert LF.crossing(rising, 2.0) is None                                # a curve that goes up never gets there
    slow = LF.fit(t, 3.0 - 1e-3 * np.log(t), "log")
    assert LF.crossing(slow, 2.0) is None                                  # e^1000 tokens: reported as never


@pytest.mark.parametrize("floor, amplitude, alpha", [(1.8, 1.0, 0.3), (0.0, 4.0, 0.08), (2.2, 0.6, 1.1)])
def test_free_power_family_recovers_floor_amplitude_and_exponent(floor, amplitude, alpha):
    t = np.linspace(1.0, 12.0, 45)
    p = LF.fit(t, floor + amplitude * t ** -alpha, "power_free")
    assert p["alpha"] == pytest.approx(alpha, rel=2e-3) and p["floor"] == pytest.approx(floor, abs=2e-3)
    assert p["amplitude"] == pytest.approx(amplitude, rel=5e-3) and p["rmse"] < 1e-5
    assert p["alpha_at_search_boundary"] is False
    target = floor + 0.05
    assert LF.crossing(p, target) == pytest.approx((amplitude / 0.05) ** (1 / alpha), rel=0.05)
    assert LF.crossing(p, floor - 0.01) is None                            # below the floor: never


def test_fixed_floor_is_an_assumption_the_fit_keeps():
    t = np.linspace(1.0, 10.0, 30)
    loss = 1.9 + 0.8 * t ** -0.4
    right = LF.fit(t, loss, "power_fixed:1.9")
    wrong = LF.fit(t, loss, "power_fixed:1.5")
    assert right["model"] == "power_fixed:1.9" and right["floor"] == 1.9 and right["alpha"] == pytest.approx(0.4, rel=1e-3)
    assert wrong["floor"] == 1.5 and wrong["rmse"] > right["rmse"] and wrong["alpha"] < right["alpha"]
    # the further out, the more the assumed floor decides
    near = abs(LF.predict(right, [12.0])[0] - LF.predict(wrong, [12.0])[0])
    far = abs(LF.predict(right, [1000.0])[0] - LF.predict(wrong, [1000.0])[0])
    assert far > 5 * near
    flat = LF.fit(t, np.full_like(t, 2.5), "power_free")
    assert flat["amplitude"] == pytest.approx(0.0, abs=1e-9) or flat["floor"] == pytest.approx(2.5, abs=1e-6)
    assert LF.predict(flat, [50.0])[0] == pytest.approx(2.5, abs=1e-6)


def test_a_window_needs_three_bins():
    with pytest.raises(ValueError, match="at least 3 complete bins"):
        LF.fit([1.0, 2.0], [3.0, 2.9], "log")


def test_bins_are_complete_half_open_intervals():
    rows = [{"tokens": int(t * 1e9), "loss": 4.0 - t} for t in (0.5, 1.0, 1.1, 1.2, 1.25, 1.4, 1.5, 1.6, 1.74, 1.8)]
    bins, end = LF.bin_rows(rows, 0.25, 1.0)
    assert end == 1.75                                                     # 1.8 B reaches the boundary at 1.75, not 2.0
    assert [(b["left_B"], b["right_B"], b["count"]) for b in bins] == [(1.0, 1.25, 3), (1.25, 1.5, 2), (1.5, 1.75, 3)]
    assert bins[0]["tokens_B"] == pytest.approx(1.1) and bins[0]["loss"] == pytest.approx(2.9)
    assert bins[1]["tokens_B"] == pytest.approx(1.325)                     # 1.25 belongs to the bin it starts
    with pytest.raises(ValueError, match="strictly increasing"):
        LF.bin_rows([{"tokens": 5, "loss": 1.0}, {"tokens": 5, "loss": 1.0}], 0.25, 1.0)
    with pytest.raises(ValueError, match="strictly increasing"):
        LF.bin_rows([], 0.25, 1.0)
    sparse = [{"tokens": int(t * 1e9), "loss": 3.0} for t in (1.0, 1.1, 1.6, 1.9)]
    with pytest.raises(ValueError, match="no validation row falls in the bin that starts at 1.25"):
        LF.bin_rows(sparse, 0.25, 1.0)


def test_command_line_writes_a_self_describing_report(tmp_path, capsys):
    rows = [{"tokens": int(t * 1e9), "loss": 2.0 + 1.5 * t ** -0.5} for t in np.arange(1.0, 4.3, 0.1)]
    source = tmp_path / "val.jsonl"
    source.write_text("\n".join(json.dumps(r) for r in rows) + "\n\n")
    out = tmp_path / "reports" / "forecast.json"
    assert LF.main(["--input", str(source), "--output", str(out), "--target-loss", "2.3"]) == 0
    assert "Analyzed 33 validation rows through 4B complete bins" in capsys.readouterr().out
    report = json.loads(out.read_text())
    assert report["source_rows"] == 33 and report["latest_validation"] == rows[-1]
    assert report["source_path"] == str(source) and len(report["source_sha256"]) == 64 and len(report["analysis_sha256"]) == 64
    assert len(report["bins"]) == 12 and report["complete_bins_end_B"] == 4.0
    starts = sorted({f["start_B"] for f in report["fits"]})
    assert starts == [1, 2, 3]                                             # windows from 4 B and 5 B have too few bins
    assert all("cross_2.3_tokens_B" in f for f in report["fits"])
    free = next(f for f in report["fits"] if f["start_B"] == 1 and f["parameters"]["model"] == "power_free")
    assert free["cross_2.3_tokens_B"] == pytest.approx(25.0, rel=0.2)      # 1.5 t^-0.5 = 0.3
    assert set(free["endpoint_losses"]) == {"40B", "268.435456B", "1073.741824B"}
    assert report["holdouts"] == []                                        # no complete billion after 4 B to test on
    with pytest.raises(SystemExit):
        LF.main(["--input", str(source), "--output", str(source)])


def test_the_report_can_be_drawn_without_a_plotting_library(tmp_path):
    import xml.etree.ElementTree as ET
    rows = [{"tokens": int(t * 1e9), "loss": 1.9 + 1.2 * t ** -0.4} for t in np.arange(1.0, 7.31, 0.05)]
    source = tmp_path / "val.jsonl"
    source.write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    out, picture = tmp_path / "forecast.json", tmp_path / "pictures" / "forecast.svg"
    assert LF.main(["--input", str(source), "--output", str(out), "--plot", str(picture)]) == 0
    tree = ET.parse(picture)                                               # well-formed
    space = "{http://www.w3.org/2000/svg}"
    root = tree.getroot()
    assert root.tag == space + "svg" and root.get("width") == "960"
    report = json.loads(out.read_text())
    families = {f["parameters"]["model"] for f in report["fits"] if f["start_B"] == 1}
    lines = root.findall(space + "polyline")
    assert len(lines) == 1 + 2 * len(families)                             # the bin means; each family solid and dashed
    assert sum(1 for line in lines if line.get("stroke-dasharray")) == len(families)
    assert len(root.findall(space + "circle")) == len(report["observed_validation"])
    labels = " ".join(t.text or "" for t in root.findall(space + "text"))
    assert all(name in labels for name in families) and "1073.74" in labels and "not confidence intervals" in labels
    for line in lines:                                                     # every point inside the canvas
        for point in line.get("points").split():
            x, y = map(float, point.split(","))
            assert 0 <= x <= 960 and 0 <= y <= 540
    with pytest.raises(SystemExit):
        LF.main(["--input", str(source), "--output", str(out), "--plot", str(out)])
    with pytest.raises(ValueError, match="nothing to plot"):
        LF.plot({"bins": [], "fits": []}, tmp_path / "empty.svg")
