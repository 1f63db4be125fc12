"""Sequential search over a categorical launch-parameter space: exhaustive grid or TPE.

The reference tunes its kernels either by timing every combination inline
(``turbo_gnn/_autotune.py:203-246``) or, offline, with an Optuna study whose default sampler is
the tree-structured Parzen estimator (``scripts/kernel_tune.py:105-141``), caching one JSON record
per trial (``src/backends/autotune.py:34-105``).  Optuna is not a dependency here: the estimator
below is the categorical case of the published algorithm (Bergstra et al., "Algorithms for
Hyper-Parameter Optimization", 2011) written for this package.

Every axis is a finite list of values.  After ``n_startup`` random trials the finished trials are
split into the best ``gamma`` fraction and the rest; per axis two smoothed categorical
distributions ``l`` (good) and ``g`` (bad) are estimated; candidates are drawn from ``l`` and the
unseen candidate with the largest ``sum_axis log l(v) / g(v)`` is tried next.  A failed trial
(invalid launch parameters) is recorded with an infinite cost and so counts as bad.
"""

from __future__ import annotations

import hashlib
import itertools
import json
import math
import os
import random
from typing import Any, Hashable, Iterator


def _freeze(cfg: dict[str, Any]) -> tuple:
    return tuple(sorted((k, repr(v)) for k, v in cfg.items()))


class GridSearch:
    """Every combination once, in the order of ``itertools.product`` over the axes."""

    def __init__(self, space: dict[str, list]):
        self.space = {k: list(v) for k, v in space.items()}
        self._it: Iterator = iter(itertools.product(*self.space.values()))
        self.trials: list[tuple[dict, float]] = []

    @property
    def size(self) -> int:
        return math.prod(len(v) for v in self.space.values()) if self.space else 1

    def ask(self) -> dict | None:
        try:
            return dict(zip(self.space, next(self._it)))
        except StopIteration:
            return None

    def tell(self, cfg: dict, cost: float) -> None:
        self.trials.append((dict(cfg), float(cost)))

    def best(self) -> tuple[dict, float] | None:
        done = [t for t in self.trials if math.isfinite(t[1])]
        return min(done, key=lambda t: t[1]) if done else None


class TPESearch(GridSearch):
    """Tree-structured Parzen estimator over categorical axes; never proposes a combination twice."""

    def __init__(self, space: dict[str, list], seed: int = 0, n_startup: int = 8, gamma: float = 0.25,
                 n_candidates: int = 24, prior_weight: float = 1.0):
        super().__init__(space)
        self._rng = random.Random(seed)
        self.n_startup, self.gamma, self.n_candidates, self.prior_weight = n_startup, gamma, n_candidates, prior_weight
        self._seen: set[Hashable] = set()

    def _random_unseen(self) -> dict | None:
        if len(self._seen) >= self.size:
            return None
        for _ in range(64):
            cfg = {k: self._rng.choice(v) for k, v in self.space.items()}
            if _freeze(cfg) not in self._seen:
                return cfg
        for combo in itertools.product(*self.space.values()):  # nearly exhausted: take the first gap
            cfg = dict(zip(self.space, combo))
            if _freeze(cfg) not in self._seen:
                return cfg
        return None

    def _weights(self, trials: list[dict], axis: str) -> list[float]:
        values = self.space[axis]
        counts = [self.prior_weight / len(values)] * len(values)
        for cfg in trials:
            counts[values.index(cfg[axis])] += 1.0
        total = sum(counts)
        return [c / total for c in counts]

    def ask(self) -> dict | None:
        if len(self._seen) >= self.size:
            return None
        if len(self.trials) < self.n_startup:
            cfg = self._random_unseen()
        else:
            ranked = sorted(self.trials, key=lambda t: t[1])
            n_good = max(1, int(math.ceil(self.gamma * len(ranked))))
            good = [t[0] for t in ranked[:n_good]]
            bad = [t[0] for t in ranked[n_good:]] or good
            l_w = {a: self._weights(good, a) for a in self.space}
            g_w = {a: self._weights(bad, a) for a in self.space}
            best_cfg, best_score = None, -math.inf
            for _ in range(self.n_candidates):
                cand = {a: self._rng.choices(vals, weights=l_w[a])[0] for a, vals in self.space.items()}
                if _freeze(cand) in self._seen:
                    continue
                score = sum(math.log(l_w[a][vals.index(cand[a])] / g_w[a][vals.index(cand[a])])
                            for a, vals in self.space.items())
                if score > best_score:
                    best_cfg, best_score = cand, score
            cfg = best_cfg or self._random_unseen()
        if cfg is not None:
            self._seen.add(_freeze(cfg))
        return cfg


def make_search(kind: str, space: dict[str, list], max_trials: int | None = None, seed: int = 0):
    """``"grid"`` or ``"tpe"``; a TPE request falls back to the grid when ``max_trials`` covers every combination."""
    grid = GridSearch(space)
    if kind == "grid" or max_trials is None or grid.size <= max_trials:
        return grid
    if kind != "tpe":
        raise ValueError(f"unknown search '{kind}' (expected 'grid' or 'tpe')")
    return TPESearch(space, seed=seed, n_startup=min(8, max(2, max_trials // 3)))


# ---- per-trial records on disk ---------------------------------------------------------------


def trial_key(kernel: str, feat_dim: int, num_nodes: int, num_edges: int, gpu: str, cfg: dict[str, Any]) -> str:
    """SHA-256 of what identifies one timing: kernel class, problem shape, GPU name and configuration."""
    blob = json.dumps({"kernel": kernel, "feat_dim": feat_dim, "num_nodes": num_nodes, "num_edges": num_edges,
                       "gpu": gpu, "config": {k: repr(v) for k, v in sorted(cfg.items())}}, sort_keys=True)
    return hashlib.sha256(blob.encode()).hexdigest()


class TrialCache:
    """One small JSON file per timed configuration under ``<dir>/trials/``; a miss returns None."""

    def __init__(self, directory: str | None):
        self.dir = os.path.join(directory, "trials") if directory else None

    def load(self, key: str) -> float | None:
        if not self.dir:
            return None
        try:
            with open(os.path.join(self.dir, key + ".json")) as fh:
                ms = json.load(fh)["ms"]
            return float("inf") if ms is None else float(ms)
        except (OSError, ValueError, KeyError, TypeError):
            return None

    def store(self, key: str, record: dict[str, Any], ms: float) -> None:
        if not self.dir:
            return
        os.makedirs(self.dir, exist_ok=True)
        with open(os.path.join(self.dir, key + ".json"), "w") as fh:
            json.dump({**record, "ms": ms if math.isfinite(ms) else None}, fh)
