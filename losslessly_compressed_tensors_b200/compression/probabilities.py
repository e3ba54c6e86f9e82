"""Probability of each BF16 exponent under the analytic value distributions.

Restates ``LCT/compression/probabilities.py:10-158`` of the reference: a
magnitude density per family, integrated over every BF16 exponent bin with
``scipy.integrate.quad`` at the same tolerances, centred on the model's mean
exponent, with an optional point mass for exact zeros, and finally re-indexed
so that table index 0 always means "exact zero".  The integrands keep the
reference's arithmetic so the resulting code lengths are the same.
"""
from __future__ import annotations

import math
from typing import Callable

import numpy as np
from scipy.integrate import quad

Pdf = Callable[[float], float]

_EXPONENTS = range(-127, 129)


def _fold(base: Pdf, mean: float) -> Pdf:
    """Magnitude density of a symmetric density ``base`` shifted by ``mean``."""
    mean = float(mean)

    def pdf(value: float) -> float:
        return 0.5 * (base(abs(value - mean)) + base(abs(value + mean)))

    return pdf


def gaussian_probabilities(std: float = 1.0, mean: float = 0.0) -> Pdf:
    sigma = float(std)

    def half_normal(value: float) -> float:
        return 2.0 / (sigma * math.sqrt(2.0 * math.pi)) * math.exp(-0.5 * (value / sigma) ** 2)

    return _fold(half_normal, mean)


def laplace_probabilities(scale: float = 1.0, mean: float = 0.0) -> Pdf:
    s = float(scale)

    def exponential(value: float) -> float:
        return math.exp(-value / s) / s

    return _fold(exponential, mean)


def empirical_probabilities(scale: float = 1.0, mean: float = 0.0) -> Pdf:
    """Exponential body with a power-law tail holding 5 % of the mass (alpha 2.8)."""
    s = float(scale)
    tail_mass, alpha = 0.05, 2.8
    knee = -s * math.log(tail_mass)

    def body_and_tail(value: float) -> float:
        if value <= knee:
            return math.exp(-value / s) / s
        return tail_mass * (alpha - 1.0) / knee * (knee / value) ** alpha

    return _fold(body_and_tail, mean)


def gamma_probabilities(shape: float = 0.82, scale: float = 2.43) -> Pdf:
    """Gamma magnitude density with the reference's fixed activation fit."""
    shape, scale = float(shape), float(scale)
    log_norm = shape * math.log(scale) + math.lgamma(shape)

    def pdf(value: float) -> float:
        value = abs(value)
        return math.exp((shape - 1.0) * math.log(value) - value / scale - log_norm)

    return pdf


def _bin_mass(pdf: Pdf, low: float, high: float) -> float:
    if high == low:
        return 0.0
    return quad(pdf, low, high, epsabs=1e-12, epsrel=1e-10, limit=200)[0]


def _exponent_probabilities(magnitude_pdf: Pdf, zero_prob: float = 0.0) -> np.ndarray:
    """Probabilities of the 256 codec table indices.

    Index 0 is exact zero (exponent -127); the other indices are the exponent's
    distance from the model centre modulo 256, shifted up by one when below the
    zero's own distance.
    """
    by_exponent = np.zeros(256, dtype=np.float64)
    for e in _EXPONENTS:
        low = 0.0 if e == -127 else math.ldexp(1.0, e)
        high = math.inf if e == 128 else math.ldexp(1.0, e + 1)
        by_exponent[e & 255] = _bin_mass(magnitude_pdf, low, high)
    by_exponent /= by_exponent.sum()

    exps = np.arange(-127, 129)
    mean = float(np.dot(exps, by_exponent[exps & 255]))
    center = math.floor(mean + 0.5) if mean >= 0.0 else -math.floor(-mean + 0.5)

    by_delta = np.zeros(256, dtype=np.float64)
    for e in _EXPONENTS:
        by_delta[(e - center) & 255] = by_exponent[e & 255]

    zero_delta = (-127 - center) & 255
    if zero_prob:
        if not (0.0 <= zero_prob <= 1.0):
            raise ValueError("zero_prob must be between 0 and 1")
        by_delta = (1.0 - zero_prob) * by_delta
        by_delta[zero_delta] += zero_prob

    by_index = np.zeros(256, dtype=np.float64)
    for delta in range(256):
        if delta == zero_delta:
            index = 0
        else:
            index = delta + 1 if delta < zero_delta else delta
        by_index[index] += by_delta[delta]
    return by_index
