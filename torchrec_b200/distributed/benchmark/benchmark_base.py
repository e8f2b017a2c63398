"""Benchmark harness: ``BenchmarkResult`` (per-iteration device times, host times, peak memory per rank with percentile
accessors), ``benchmark_func`` (CUDA-event timing, warm-up, optional profiler trace) and ``cmd_conf`` — a decorator that
turns the dataclass-typed parameters of a function into command-line flags with YAML / JSON default files
(``torchrec/distributed/benchmark/benchmark_base.py:125-665``)."""
from __future__ import annotations

import argparse
import contextlib
import dataclasses
import inspect
import json
import os
import time
from dataclasses import dataclass, field, fields, is_dataclass, MISSING
from typing import Any, Callable, Dict, List, Optional, Tuple, Union, get_type_hints

import torch


@dataclass
class MemoryStats:
    rank: int
    malloc_retries: int
    max_mem_allocated_mbs: int
    max_mem_reserved_mbs: int

    @classmethod
    def for_device(cls, rank: int) -> "MemoryStats":
        stats = torch.cuda.memory_stats(rank)
        return cls(rank, int(stats.get("num_alloc_retries", 0)), int(stats.get("allocated_bytes.all.peak", 0) // 2 ** 20),
                   int(stats.get("reserved_bytes.all.peak", 0) // 2 ** 20))

    def __str__(self) -> str:
        return f"Rank {self.rank}: retries={self.malloc_retries}, allocated={self.max_mem_allocated_mbs:7}mb, reserved={self.max_mem_reserved_mbs:7}mb"


@dataclass
class BenchmarkResult:
    short_name: str
    gpu_elapsed_time: torch.Tensor  # milliseconds per iteration
    cpu_elapsed_time: torch.Tensor  # milliseconds per iteration
    mem_stats: List[MemoryStats] = field(default_factory=list)
    rank: int = -1

    def __str__(self) -> str:
        gpu = f"GPU Runtime (P90): {self.runtime_percentile(90, device='gpu'):.2f} ms"
        cpu = f"CPU Runtime (P90): {self.runtime_percentile(90, device='cpu'):.2f} ms"
        mem = f"Peak Memory alloc (P90): {self.max_mem_alloc_percentile(90) / 1000:.2f} GB" if self.mem_stats else "Peak Memory: n/a"
        return f"{self.short_name: <{35}} | {gpu} | {cpu} | {mem}"

    def runtime_percentile(self, percentile: int = 50, device: str = "gpu", interpolation: str = "nearest") -> torch.Tensor:
        t = self.gpu_elapsed_time if device == "gpu" else self.cpu_elapsed_time
        return torch.quantile(t.double(), percentile / 100.0, interpolation=interpolation)

    def max_mem_alloc_percentile(self, percentile: int = 50, interpolation: str = "nearest") -> torch.Tensor:
        return self._mem_percentile(percentile, interpolation, lambda m: m.max_mem_allocated_mbs)

    def max_mem_reserved_percentile(self, percentile: int = 50, interpolation: str = "nearest") -> torch.Tensor:
        return self._mem_percentile(percentile, interpolation, lambda m: m.max_mem_reserved_mbs)

    def _mem_percentile(self, percentile: int, interpolation: str, get: Callable[[MemoryStats], int]) -> torch.Tensor:
        data = torch.tensor([get(m) for m in self.mem_stats], dtype=torch.float)
        return torch.quantile(data, percentile / 100.0, interpolation=interpolation)


def benchmark_func(name: str, run_iter: Callable[[], Any], num_iters: int = 10, warmup_iters: int = 3, device: Optional[torch.device] = None,
                   rank: int = -1, profile_dir: str = "", reset_memory_stats: bool = True) -> BenchmarkResult:
    """Time ``run_iter`` per iteration: CUDA events on the current stream (after ``warmup_iters`` untimed runs, synchronised on both
    sides) and host wall clock.  With ``profile_dir`` one extra traced iteration writes a chrome trace there."""
    use_cuda = device is not None and device.type == "cuda" and torch.cuda.is_available()
    for _ in range(warmup_iters):
        run_iter()
    if use_cuda:
        torch.cuda.synchronize(device)
        if reset_memory_stats:
            torch.cuda.reset_peak_memory_stats(device)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(num_iters)] if use_cuda else []
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(num_iters)] if use_cuda else []
    cpu_ms = []
    for i in range(num_iters):
        t0 = time.perf_counter()
        if use_cuda:
            starts[i].record()
        run_iter()
        if use_cuda:
            ends[i].record()
        cpu_ms.append((time.perf_counter() - t0) * 1e3)
    if use_cuda:
        torch.cuda.synchronize(device)
        gpu = torch.tensor([s.elapsed_time(e) for s, e in zip(starts, ends)])
        mem = [MemoryStats.for_device(device.index if device.index is not None else torch.cuda.current_device())]
    else:
        gpu = torch.tensor(cpu_ms)
        mem = []
    if profile_dir:
        os.makedirs(profile_dir, exist_ok=True)
        acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if use_cuda else [])
        with torch.profiler.profile(activities=acts, record_shapes=True, profile_memory=True, with_flops=True, with_modules=True) as prof:
            run_iter()
            if use_cuda:
                torch.cuda.synchronize(device)
        prof.export_chrome_trace(os.path.join(profile_dir, f"trace-{name}-rank{rank}.json"))
    return BenchmarkResult(short_name=name, gpu_elapsed_time=gpu, cpu_elapsed_time=torch.tensor(cpu_ms), mem_stats=mem, rank=rank)


# ---- cmd_conf: dataclass-typed function parameters -> argparse flags with YAML/JSON defaults ----------------------
def _load_config_file(path: str) -> Dict[str, Any]:
    if not path:
        return {}
    with open(path, "r") as f:
        if path.endswith((".yaml", ".yml")):
            import yaml

            return yaml.safe_load(f) or {}
        return json.load(f)


def _convert(tp: Any, value: str) -> Any:
    origin = getattr(tp, "__origin__", None)
    if tp is bool:
        return value.lower() in ("1", "true", "yes", "y")
    if origin in (list, List):
        (elem,) = getattr(tp, "__args__", (str,))
        return [_convert(elem, v) for v in value.split(",") if v != ""]
    if origin is Union:  # Optional[T]
        args = [a for a in tp.__args__ if a is not type(None)]
        return None if value in ("None", "none", "") else _convert(args[0], value)
    if isinstance(tp, type) and issubclass(tp, __import__("enum").Enum):
        return tp[value] if value in tp.__members__ else tp(value)
    if tp in (int, float, str):
        return tp(value)
    return value


def cmd_conf(func: Callable[..., Any]) -> Callable[..., Any]:
    """Calling the decorated function with no arguments parses ``sys.argv``: every field of every dataclass-typed parameter
    becomes ``--<field>``; ``--yaml_config`` / ``--json_config`` name a file of defaults (flat, or nested by parameter name);
    explicit flags win over the file, the file over dataclass defaults."""
    sig = inspect.signature(func)
    hints = get_type_hints(func)

    def wrapper(*args: Any, **kwargs: Any) -> Any:
        if args or kwargs:
            return func(*args, **kwargs)
        pre = argparse.ArgumentParser(add_help=False)
        pre.add_argument("--yaml_config", default="")
        pre.add_argument("--json_config", default="")
        known, _ = pre.parse_known_args()
        defaults = {**_load_config_file(known.json_config), **_load_config_file(known.yaml_config)}
        parser = argparse.ArgumentParser(description=func.__doc__, parents=[pre])
        seen: Dict[str, Tuple[str, Any]] = {}
        for pname, param in sig.parameters.items():
            tp = hints.get(pname, param.annotation)
            if is_dataclass(tp):
                nested = defaults.get(pname, {}) if isinstance(defaults.get(pname), dict) else {}
                fhints = get_type_hints(tp)
                for f in fields(tp):
                    if f.name in seen:
                        continue
                    d = nested.get(f.name, defaults.get(f.name, MISSING))
                    seen[f.name] = (pname, fhints.get(f.name, str))
                    parser.add_argument(f"--{f.name}", default=None, help=f"{tp.__name__}.{f.name}" + ("" if d is MISSING else f" (config: {d})"))
            else:
                seen[pname] = ("", tp)
                parser.add_argument(f"--{pname}", default=None)
        ns = vars(parser.parse_args())
        call: Dict[str, Any] = {}
        for pname, param in sig.parameters.items():
            tp = hints.get(pname, param.annotation)
            if is_dataclass(tp):
                nested = defaults.get(pname, {}) if isinstance(defaults.get(pname), dict) else {}
                fhints = get_type_hints(tp)
                vals = {}
                for f in fields(tp):
                    if ns.get(f.name) is not None:
                        vals[f.name] = _convert(fhints.get(f.name, str), ns[f.name])
                    elif f.name in nested:
                        vals[f.name] = nested[f.name]
                    elif f.name in defaults and not isinstance(defaults[f.name], dict):
                        vals[f.name] = defaults[f.name]
                call[pname] = tp(**vals)
            elif ns.get(pname) is not None:
                call[pname] = _convert(tp, ns[pname]) if tp is not inspect._empty else ns[pname]
            elif pname in defaults:
                call[pname] = defaults[pname]
            elif param.default is not inspect._empty:
                call[pname] = param.default
        return func(**call)

    wrapper.__name__ = func.__name__
    wrapper.__doc__ = func.__doc__
    return wrapper
