"""Activation statistics for int8 quantisation: a restatement of minml's histogram calibrator.

Reference: `src/graph/Histogram.cpp` (collection `:180-236`, range search `:320-346`, transform `:385-399`, helpers
`:32-96`), `src/graph/CalibrationTable.cpp`, used by `Graph::calibrate` (`src/graph/Graph.cpp:420-440`): every node
output gets a histogram; batches are fed until every histogram reports ready; the histogram's `getTransform()` becomes the
node's output transform (int8 -> fp32: x = q * scale + shift).

A histogram first tracks the minimum and maximum until fewer than `accuracy` of the samples seen fall outside the range
found so far, then counts samples into `bins` equal bins of that range until one more batch changes the normalised
histogram by less than `accuracy` (L1 distance divided by batch_rows ** 0.666). The quantisation range is the window of
bins (a multiple of `target_bins` wide, aligned to `target_bins`) whose `target_bins`-level requantised histogram has the
smallest Kullback-Leibler divergence from the full one; scale and shift follow from the window, the shift adjusted so that
fp32 zero is an integer on the int8 grid. Arithmetic types follow the reference (fp32 for the range and the bin index,
fp64 for the histogram), so the bins come out identical to the reference's on the same batches.

This is host code of the calibration step, not part of the GPU path; `networks.py` accepts its transforms in place of the
max-abs rule.
"""
import math

import numpy as np

F = np.float32

ACT_RANGES = {"sigmoid": (0.0, 1.0), "tanh": (-1.0, 1.0), "softmax": (0.0, 1.0)}  # exact ranges: nothing to collect


def _l1_diff(p, q):
    area_p = 1.0 / float(np.add.reduce(p, initial=1e-16))
    area_q = 1.0 / float(np.add.reduce(q, initial=1e-16))
    return float(np.abs(p * area_p - q * area_q).sum())


def _kl_divergence(p, q):
    eps = np.finfo(np.float64).eps
    return float((p * (np.log(eps + p) - np.log(eps + q))).sum())


def _resize(hist, from_bin, to_bin, target_bins):
    """The histogram as `target_bins` levels over [from_bin, to_bin) would see it: mass outside the window is moved to its
    edge bins, every group of merged bins is flattened over its non-empty bins, the result is normalised
    (Histogram.cpp:52-96). Returns a new array."""
    out = hist.copy()
    window = (to_bin - from_bin) // target_bins
    low = float(out[:from_bin].sum())
    out[:from_bin] = 0.0
    out[from_bin] += low
    high = float(out[to_bin:].sum())
    out[to_bin:] = 0.0
    out[to_bin - 1] += high
    groups = out[from_bin:to_bin].reshape(target_bins, window)
    partial = groups.sum(axis=1)
    nonzero = (groups != 0.0).sum(axis=1)
    with np.errstate(invalid="ignore", divide="ignore"):
        avg = partial / nonzero
    flattened = np.where(groups != 0.0, avg[:, None], 0.0)
    out[from_bin:to_bin] = flattened.reshape(-1) * (1.0 / float(partial.sum()))
    return out


class Histogram:
    def __init__(self, number_of_bins=2048, accuracy=0.01, target_bins=256):
        assert number_of_bins % target_bins == 0
        self.data = np.zeros(number_of_bins, np.float64)
        self.min_value = F(np.finfo(np.float32).max)
        self.max_value = F(np.finfo(np.float32).min)
        self.collected_samples = 0
        self.outliers_count = 0
        self.accuracy = F(accuracy)
        self.target_bins = target_bins
        self.is_used = True
        self.is_exact = False
        self.is_ready_flag = False
        self.optimal_range = (0, number_of_bins)
        self.scale = F(1.0)
        self.shift = F(0.0)

    def set_hint(self, activation):
        """The activation that produced the tensor narrows the range in advance (Histogram.cpp:140-170)."""
        if activation in ACT_RANGES:
            lo, hi = ACT_RANGES[activation]
            self.min_value, self.max_value = F(lo), F(hi)
            self.is_ready_flag = True
            self.is_exact = True
        elif activation in ("relu", "exp"):
            self.min_value = F(0.0)

    def is_ready(self):
        return self.is_ready_flag or not self.is_used

    def _enough_for_min_max(self):
        if self.collected_samples == 0:
            return False  # 0 / 0 compares false in the reference
        return self.outliers_count / self.collected_samples < float(self.accuracy)

    def collect_statistics(self, tensor):
        """tensor: a batch, first axis = batch rows (Histogram.cpp:180-236)."""
        if not self.is_used or self.is_exact:
            return
        values = np.ascontiguousarray(tensor, np.float32).reshape(-1)
        if not self._enough_for_min_max():
            self.outliers_count = int(np.count_nonzero((values < self.min_value) | (values > self.max_value)))
            self.min_value = F(min(self.min_value, values.min()))
            self.max_value = F(max(self.max_value, values.max()))
        self.collected_samples += values.size
        if self._enough_for_min_max():
            previous = self.data.copy()
            self._update(values)
            diff = _l1_diff(previous, self.data) / math.pow(float(np.shape(tensor)[0]), float(F(0.666)))
            if diff < float(self.accuracy):
                self.is_ready_flag = True
        if self.is_ready_flag:
            self.optimal_range = self.find_coarse_range()
            self.scale, self.shift = self.calculate_transform(self.optimal_range)

    def _update(self, values):
        size = self.data.size
        tmp = F(size - 1) / (F(self.max_value - self.min_value) + F(1e-16))
        position = (values - self.min_value) * tmp  # fp32
        index = np.where(position < 0, size - 1, np.minimum(position, F(size - 1)).astype(np.int64))  # a negative product wraps to the last bin
        self.data += np.bincount(np.clip(index, 0, size - 1), minlength=size).astype(np.float64)

    def find_coarse_range(self):
        size = self.data.size
        if self.is_exact:
            return (0, size)
        reference = self.data * (1.0 / float(np.add.reduce(self.data, initial=1e-16)))
        best, best_value = (0, size), float("inf")
        for i in range(0, size, self.target_bins):
            for j in range(i + self.target_bins, size + 1, self.target_bins):
                kld = _kl_divergence(reference, _resize(reference, i, j, self.target_bins))
                if kld <= best_value:
                    best, best_value = (i, j), kld
        return best

    def calculate_transform(self, bin_range):
        """(scale, shift) of x = q * scale + shift for the window of bins (Histogram.cpp:385-399)."""
        step = F(self.max_value - self.min_value) / F(self.data.size)
        start = F(self.min_value + F(bin_range[0]) * step)
        end = F(self.min_value + F(bin_range[1]) * step)
        scale = F(end - start) / F(self.target_bins - 1)
        shift = F(0.5) * F(F(end + start) + scale)
        ratio = float(F(-shift) / scale)
        int8_zero = int(math.floor(abs(ratio) + 0.5)) * (1 if ratio >= 0 else -1)  # C round(): half away from zero
        return scale, F(F(-int8_zero) * scale)

    def get_transform(self):
        return float(self.scale), float(self.shift)


class CalibrationTable:
    """One histogram per tensor of interest; ready when all of them are (CalibrationTable.cpp)."""

    def __init__(self, size, number_of_bins=2048, accuracy=0.01, target_bins=256):
        self.histograms = [Histogram(number_of_bins, accuracy, target_bins) for _ in range(size)]

    def __getitem__(self, index):
        return self.histograms[index]

    def __len__(self):
        return len(self.histograms)

    def is_ready(self):
        return len(self.histograms) > 0 and all(h.is_ready() for h in self.histograms)

    def completion(self):
        return sum(h.is_ready() for h in self.histograms) / max(1, len(self.histograms))
