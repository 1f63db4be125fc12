"""Grid-search autotuning of launch parameters and bucket quantiles.

Mirror of the reference's ``turbo_gnn/_autotune.py`` (``TunableParam`` 18-30,
``AutotuneConfig`` 33-49, ``_InlineAutotuneCache`` 61-100, ``TunableKernel``
103-241, ``with_autotune`` 244-290) with the same names and call semantics,
because user code and the reference's unit tests drive these classes
directly.  What is searched is re-targeted at this library's kernels: warps
per row in the light tier, warps per CTA in the heavy tier, edges per hub
chunk, the hub degree threshold and the light/heavy quantile.

Beyond the reference: ``AutotuneConfig.cache_dir`` is honoured.  When set, the
winning configuration is also written to a JSON file keyed by kernel, graph
size, feature width and GPU name, and read back by later processes.
"""

from __future__ import annotations

import functools
import hashlib
import inspect
import itertools
import json
import logging
import os
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Callable, ClassVar

import torch

from . import _search, _timer

logger = logging.getLogger(__name__)


@dataclass
class TunableParam:
    """One axis of the search grid: attribute ``name`` takes each of ``values``; ``default`` when not tuning."""

    name: str
    values: list
    default: Any


@dataclass
class AutotuneConfig:
    """How a search is timed (``warmup``/``iters`` per candidate), which combinations it visits and
    whether results persist on disk (the winner per problem, and one record per timed trial)."""

    warmup: int = 10
    iters: int = 50
    tune_backward: bool = False
    cache_dir: str | None = None
    use_cache: bool = True
    search: str = "grid"  # "grid": every combination; "tpe": at most max_trials, picked by a Parzen estimator
    max_trials: int | None = None
    seed: int = 0


def _build_combinations(params: list[TunableParam]) -> list[dict[str, Any]]:
    """Cartesian product of the parameter values as a list of {name: value}; ``[{}]`` for no parameters."""
    names = [p.name for p in params]
    return [dict(zip(names, combo)) for combo in itertools.product(*(p.values for p in params))]


def _feature_width(x) -> int:
    return x.shape[-1] if x.ndim > 1 else 1


class _InlineAutotuneCache:
    """In-memory results: graph object identity -> CSR storage identity -> (nodes, edges, feature width).

    A hit needs all three levels to match, so a graph object whose CSR tensors were swapped, or a
    call with another feature width, is tuned again.  Values are
    ``{"kernel_config": dict, "graph_repr": graph}``.
    """

    def __init__(self):
        self._cache: dict[int, dict[int, dict[tuple, dict]]] = {}

    @staticmethod
    def _csr_hash(graph_repr) -> int:
        return hash((graph_repr.forward_indptr.data_ptr(), graph_repr.backward_indptr.data_ptr()))

    @staticmethod
    def _shape_key(graph_repr, feat_dim: int) -> tuple:
        return (graph_repr.forward_indptr.numel() - 1, graph_repr.forward_indices.numel(), feat_dim)

    def lookup(self, graph_repr, feat_dim: int) -> dict | None:
        by_csr = self._cache.get(id(graph_repr))
        if by_csr is None:
            return None
        by_shape = by_csr.get(self._csr_hash(graph_repr))
        if by_shape is None:
            return None
        return by_shape.get(self._shape_key(graph_repr, feat_dim))

    def store(self, graph_repr, feat_dim: int, result: dict) -> None:
        by_csr = self._cache.setdefault(id(graph_repr), {})
        by_shape = by_csr.setdefault(self._csr_hash(graph_repr), {})
        by_shape[self._shape_key(graph_repr, feat_dim)] = result


def _disk_key(kernel_name: str, graph_repr, x) -> str:
    gpu = torch.cuda.get_device_name(x.device) if getattr(x, "is_cuda", False) else "cpu"
    blob = json.dumps(
        [kernel_name, graph_repr.forward_indptr.numel() - 1, graph_repr.forward_indices.numel(), list(x.shape),
         str(x.dtype), gpu]
    )
    return hashlib.sha256(blob.encode()).hexdigest()[:32]


class TunableKernel(ABC):
    """A kernel call with declared tunable attributes.

    Subclasses implement ``_execute(graph, x, **kwargs)`` and list their search axes in the four
    ``get_tunable_*`` methods; names of axes are attribute names set through ``configure``.
    Graph axes are passed to ``graph.repartition``.  Instances are shared per
    (class, constructor kwargs) through ``_get_or_create``.
    """

    _shared_instances: ClassVar[dict[tuple, "TunableKernel"]] = {}

    def __init__(self) -> None:
        self._autotune_enabled: bool = False
        self._is_tuned: bool = False
        self._is_autotuning: bool = False
        self._autotune_config: AutotuneConfig = AutotuneConfig()
        self._inline_cache: _InlineAutotuneCache = _InlineAutotuneCache()

    @abstractmethod
    def _execute(self, graph, x, **kwargs):
        """Run the kernel with the currently configured attributes."""

    # -- cached / tuned execution -----------------------------------------------------

    def _run_tuned(self, graph, x, config, extra_args: tuple, kwargs: dict):
        feat_dim = _feature_width(x)
        found = self._inline_cache.lookup(graph, feat_dim)
        if found is None:
            found = self._inline_autotune(x, graph, config or self._autotune_config, **kwargs)
            self._inline_cache.store(graph, feat_dim, found)
        elif found["kernel_config"]:
            self.configure(**found["kernel_config"])
        return self._execute(found["graph_repr"], x, *extra_args, **kwargs)

    def __call__(self, *args, autotune=False, autotune_config=None, **kwargs):
        if not autotune or self._is_autotuning:
            return self._execute(*args, **kwargs)
        return self._run_tuned(args[0], args[1], autotune_config, tuple(args[2:]), kwargs)

    # -- search space ---------------------------------------------------------------

    def get_tunable_forward_kernel_params(self) -> list[TunableParam]:
        return []

    def get_tunable_forward_graph_params(self) -> list[TunableParam]:
        return []

    def get_tunable_backward_kernel_params(self) -> list[TunableParam]:
        return []

    def get_tunable_backward_graph_params(self) -> list[TunableParam]:
        return []

    def configure(self, **kwargs: Any) -> None:
        """Set tunable attributes by name."""
        for key, value in kwargs.items():
            setattr(self, key, value)

    # -- what gets timed ----------------------------------------------------------------

    def make_forward_bench_fn(self, x: torch.Tensor, graph_repr, **kwargs) -> Callable:
        return lambda: self._execute(graph_repr, x, **kwargs)

    def make_backward_bench_fn(self, x: torch.Tensor, graph_repr, **kwargs) -> Callable:
        forward = self.make_forward_bench_fn(x, graph_repr, **kwargs)
        probe = forward()
        if not isinstance(probe, torch.Tensor):
            raise RuntimeError(
                f"{type(self).__name__}.make_forward_bench_fn must return a tensor "
                "for default make_backward_bench_fn to work"
            )
        upstream = torch.randn_like(probe)

        def _step():
            forward().backward(upstream, retain_graph=True)

        return _step

    # -- search -------------------------------------------------------------------------

    def _disk_path(self, config: AutotuneConfig, graph_repr, x) -> str | None:
        if not config.cache_dir:
            return None
        return os.path.join(config.cache_dir, f"{self.name}_{_disk_key(self.name, graph_repr, x)}.json")

    def _load_from_disk(self, config: AutotuneConfig, graph_repr, x) -> dict | None:
        path = self._disk_path(config, graph_repr, x)
        if not path or not config.use_cache or not os.path.exists(path):
            return None
        try:
            with open(path) as fh:
                saved = json.load(fh)
            graph_cfg, kernel_cfg = saved["graph_config"], saved["kernel_config"]
        except (OSError, ValueError, KeyError):
            return None
        tuned_graph = graph_repr.repartition(**graph_cfg) if graph_cfg else graph_repr
        if kernel_cfg:
            self.configure(**kernel_cfg)
        return {"kernel_config": kernel_cfg, "graph_repr": tuned_graph}

    def _save_to_disk(self, config: AutotuneConfig, graph_repr, x, graph_cfg: dict, kernel_cfg: dict, ms: float):
        path = self._disk_path(config, graph_repr, x)
        if not path:
            return
        os.makedirs(config.cache_dir, exist_ok=True)
        with open(path, "w") as fh:
            json.dump({"kernel": self.name, "graph_config": graph_cfg, "kernel_config": kernel_cfg, "ms": ms}, fh)

    def _inline_autotune(self, x, graph_repr, config=None, **kwargs):
        """Time (graph axes) x (kernel axes) combinations -- all of them, or ``max_trials`` chosen by
        the TPE search -- and return the fastest as a result dict.

        A combination whose run raises ``RuntimeError`` (a launch parameter the library rejects)
        is skipped.  The winning kernel attributes stay configured on return.
        """
        config = config or self._autotune_config
        kernel_axes = self.get_tunable_forward_kernel_params()
        graph_axes = self.get_tunable_forward_graph_params()
        untouched = {"kernel_config": {}, "graph_repr": graph_repr}
        if not kernel_axes and not graph_axes:
            return untouched
        from_disk = self._load_from_disk(config, graph_repr, x)
        if from_disk is not None:
            return from_disk

        best_ms, best, best_graph_cfg = float("inf"), untouched, {}
        graph_names = {p.name for p in graph_axes}
        search = _search.make_search(config.search, {p.name: list(p.values) for p in graph_axes + kernel_axes},
                                     config.max_trials, config.seed)
        trials = _search.TrialCache(config.cache_dir if config.use_cache else None)
        gpu = torch.cuda.get_device_name(x.device) if getattr(x, "is_cuda", False) else "cpu"
        shape = (_feature_width(x), graph_repr.forward_indptr.numel() - 1, graph_repr.forward_indices.numel())
        graphs: dict[tuple, Any] = {}
        self._is_autotuning = True
        try:
            limit = config.max_trials if config.max_trials is not None else search.size
            for _ in range(limit):
                cfg = search.ask()
                if cfg is None:
                    break
                graph_cfg = {k: v for k, v in cfg.items() if k in graph_names}
                kernel_cfg = {k: v for k, v in cfg.items() if k not in graph_names}
                gkey = tuple(sorted((k, repr(v)) for k, v in graph_cfg.items()))
                if gkey not in graphs:
                    graphs[gkey] = graph_repr.repartition(**graph_cfg) if graph_cfg else graph_repr
                candidate_graph = graphs[gkey]
                if kernel_cfg:
                    self.configure(**kernel_cfg)
                key = _search.trial_key(self.name + (":bwd" if config.tune_backward else ""), *shape, gpu, cfg)
                ms = trials.load(key)
                if ms is None:
                    try:
                        fn = (self.make_backward_bench_fn if config.tune_backward else self.make_forward_bench_fn)(
                            x, candidate_graph, **kwargs
                        )
                        ms = _timer.time_callable(fn, warmup=config.warmup, iters=config.iters).ms_per_iter
                    except RuntimeError:
                        logger.debug("Skipping invalid config: graph=%s kernel=%s", graph_cfg, kernel_cfg)
                        ms = float("inf")
                    trials.store(key, {"kernel": self.name, "config": {k: repr(v) for k, v in cfg.items()}}, ms)
                search.tell(cfg, ms)
                if ms < best_ms:
                    best_ms, best_graph_cfg = ms, graph_cfg
                    best = {"kernel_config": kernel_cfg, "graph_repr": candidate_graph}
        finally:
            self._is_autotuning = False
        if best["kernel_config"]:
            self.configure(**best["kernel_config"])
        if best_ms != float("inf"):
            self._save_to_disk(config, graph_repr, x, best_graph_cfg, best["kernel_config"], best_ms)
        self._is_tuned = True
        return best

    # -- shared instances -------------------------------------------------------------------

    @classmethod
    def _get_or_create(cls, **init_kwargs) -> "TunableKernel":
        key = (cls.__name__, tuple(sorted(init_kwargs.items())))
        inst = TunableKernel._shared_instances.get(key)
        if inst is None:
            inst = TunableKernel._shared_instances[key] = cls(**init_kwargs)
        return inst

    @property
    def name(self) -> str:
        return type(self).__name__


def with_autotune(kernel_class, *, init_params=()):
    """Give a kernel function ``autotune=True`` / ``autotune_config=`` keywords.

    Without ``autotune`` the function runs untouched.  With it, the first two parameters of the
    function are taken as (graph, x); keyword names listed in ``init_params`` select the shared
    ``kernel_class`` instance (e.g. one per ``reduce`` mode); the rest are forwarded to
    ``kernel._execute`` after the search (or the cache hit) configured the kernel.
    """

    def decorator(fn):
        signature = inspect.signature(fn)
        graph_name, x_name = list(signature.parameters)[:2]

        @functools.wraps(fn)
        def wrapper(*args, autotune=False, autotune_config=None, **kwargs):
            if not autotune:
                return fn(*args, **kwargs)
            bound = signature.bind(*args, **kwargs)
            bound.apply_defaults()
            call = dict(bound.arguments)
            graph, x = call.pop(graph_name), call.pop(x_name)
            init_kw = {k: call[k] for k in init_params if k in call}
            exec_kw = {k: v for k, v in call.items() if k not in init_params}
            kernel = kernel_class._get_or_create(**init_kw)
            return kernel._run_tuned(graph, x, autotune_config, (), exec_kw)

        return wrapper

    return decorator
