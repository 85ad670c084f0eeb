"""The histogram calibrator (minml_b200/calibration.py) against the state minml's own Histogram reached on the same seeded
activations (tests/golden/make_calibration.cpp -> tests/golden/calibration_histograms.bin)."""
import os

import numpy as np
import pytest

from minml_b200 import calibration as K
from minml_b200 import checkpoint as C

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "calibration_histograms.bin")
MASK = (1 << 64) - 1


class Lcg:
    """The generator of make_calibration.cpp: exact in fp32, so the batches are bit-identical to the ones minml saw."""

    def __init__(self, seed):
        self.state = seed

    def uniform(self):
        self.state = (self.state * 6364136223846793005 + 1442695040888963407) & MASK
        return np.float32(self.state >> 40) * np.float32(1.0 / 16777216.0)

    def batch(self, count, relu):
        out = np.empty(count, np.float32)
        f = np.float32
        for i in range(count):
            a, b, c, d = self.uniform(), self.uniform(), self.uniform(), self.uniform()
            x = f(f(f(a + b) + f(c + d)) - f(2.0))
            x = f(f(x * f(1.5)) + f(0.25))
            if self.uniform() < f(0.015625):
                x = f(x * f(4.0))
            out[i] = max(x, f(0.0)) if relu else x
        return out


@pytest.fixture(scope="module")
def golden():
    return C.load_file(GOLDEN)


@pytest.mark.parametrize("name", ["relu", "linear"])
def test_histogram_reaches_the_state_minml_reached(golden, name):
    description, blob = golden
    want = description[name]
    h = K.Histogram(want["bins"], want["accuracy"], want["target_bins"])
    if name == "relu":
        h.set_hint("relu")
    g = Lcg(want["seed"])
    batches = 0
    while not h.is_ready() and batches < 400:
        h.collect_statistics(g.batch(want["rows"] * want["cols"], name == "relu").reshape(want["rows"], want["cols"]))
        batches += 1
    assert batches == want["batches"]
    assert h.collected_samples == want["collected_samples"] and h.outliers_count == want["outliers_count"]
    bins = np.frombuffer(blob, np.float64, want["bins"], want["binary_offset"])
    assert np.array_equal(h.data, bins)  # every sample in the same bin
    # the Json text keeps six decimals of the floats
    assert abs(float(h.min_value) - want["min"]) <= 1e-6 and abs(float(h.max_value) - want["max"]) <= 1e-6
    scale, shift = h.get_transform()
    assert abs(scale - want["scale"]) <= 1e-6 and abs(shift - want["shift"]) <= 1e-6
    # fp32 zero sits on the int8 grid
    assert abs(shift / scale - round(shift / scale)) <= 1e-4


def test_exact_ranges_need_no_data():
    h = K.Histogram()
    h.set_hint("sigmoid")
    assert h.is_ready()
    h.optimal_range = h.find_coarse_range()
    scale, shift = h.calculate_transform(h.optimal_range)
    assert h.optimal_range == (0, 2048)
    assert abs(float(scale) - 1.0 / 255.0) <= 1e-7
    assert abs(float(shift) / float(scale) - round(float(shift) / float(scale))) <= 1e-4


def test_range_search_clips_the_tail_of_the_fixture(golden):
    """The ReLU fixture has one value in 64 four times larger than the rest: minml's search (and this one) ends the int8 range
    at 3.3 although values reach 8.9."""
    want = golden[0]["relu"]
    assert 255 * want["scale"] < 0.5 * want["max"]
    h = K.Histogram(want["bins"], want["accuracy"], want["target_bins"])
    h.set_hint("relu")
    g = Lcg(want["seed"])
    for _ in range(want["batches"]):
        h.collect_statistics(g.batch(want["rows"] * want["cols"], True).reshape(want["rows"], want["cols"]))
    lo, hi = h.optimal_range
    assert lo == 0 and hi % want["target_bins"] == 0 and hi < want["bins"]


def test_calibration_table():
    table = K.CalibrationTable(3)
    assert not table.is_ready() and table.completion() == 0.0 and len(table) == 3
    for h in table.histograms:
        h.set_hint("tanh")
    assert table.is_ready() and table.completion() == 1.0 and table[0].get_transform()[0] > 0.0
