"""Plackett–Luce skill ratings (Weng & Lin's Bayesian approximation), the model the validator
uses to rank miners from their per-window gradient scores.

The reference takes this from the ``openskill`` package (``PlackettLuce(beta, tau)``, neurons/validator.py:
903-1082); the update rule is re-stated here so that the validator has no dependency on it.
``ordinal()`` is ``mu - 3 sigma``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass
class Rating:
    mu: float = 25.0
    sigma: float = 25.0 / 3.0
    name: str | None = None

    def ordinal(self, z: float = 3.0) -> float:
        return self.mu - z * self.sigma


class PlackettLuce:
    def __init__(self, mu: float = 25.0, sigma: float = 25.0 / 3.0, beta: float = 25.0 / 6.0, kappa: float = 1e-4,
                 tau: float = 25.0 / 300.0):
        self.mu, self.sigma, self.beta, self.kappa, self.tau = mu, sigma, beta, kappa, tau

    def rating(self, mu: float | None = None, sigma: float | None = None, name: str | None = None) -> Rating:
        return Rating(self.mu if mu is None else mu, self.sigma if sigma is None else sigma, name)

    def rate(self, teams: list[list[Rating]], scores: list[float] | None = None, ranks: list[float] | None = None):
        """One-player teams. Higher score = better. Returns new ratings in the same nesting."""
        players = [t[0] for t in teams]
        n = len(players)
        if ranks is None:
            if scores is None:
                ranks = list(range(n))
            else:
                order = sorted(set(scores), reverse=True)
                ranks = [order.index(s) for s in scores]
        sig2 = [p.sigma ** 2 + self.tau ** 2 for p in players]
        c = math.sqrt(sum(s + self.beta ** 2 for s in sig2))
        e = [math.exp(p.mu / c) for p in players]
        sum_q = [sum(e[i] for i in range(n) if ranks[i] >= ranks[q]) for q in range(n)]
        a = [sum(1 for i in range(n) if ranks[i] == ranks[q]) for q in range(n)]
        out = []
        for i, p in enumerate(players):
            omega = delta = 0.0
            for q in range(n):
                if ranks[q] <= ranks[i]:
                    quot = e[i] / sum_q[q]
                    omega += ((1.0 if q == i else 0.0) - quot) / a[q]
                    delta += quot * (1.0 - quot) / a[q]
            omega *= sig2[i] / c
            delta *= sig2[i] / (c * c)
            delta *= math.sqrt(sig2[i]) / c
            out.append([Rating(p.mu + omega, math.sqrt(sig2[i]) * math.sqrt(max(1.0 - delta, self.kappa)), p.name)])
        return out
