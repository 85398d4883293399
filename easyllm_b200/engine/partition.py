"""Pipeline-stage partitioning of a flat layer list.

Parity with the partitioner the reference gets from DeepSpeed's ``PipelineModule``
(``pp_partition_method``: llm/models/mg_models/llama/llama.py:79-95, configs use
``'parameters'``): ``uniform`` balances layer counts, ``parameters`` balances parameter
counts, ``type:<regex>`` balances the number of layers whose class name matches.
Returns ``parts`` with ``parts[s] .. parts[s+1]`` the layer index range of stage ``s``.
"""
from __future__ import annotations

import re
from typing import List, Sequence


def partition_uniform(num_items: int, num_parts: int) -> List[int]:
    parts = [0] * (num_parts + 1)
    if num_items <= num_parts:
        for p in range(num_parts + 1):
            parts[p] = min(p, num_items)
        return parts
    chunk, rem = divmod(num_items, num_parts)
    for p in range(num_parts):
        parts[p + 1] = parts[p] + chunk + (1 if p < rem else 0)
    return parts


def _feasible(weights: Sequence[float], num_parts: int, cap: float):
    """Greedy packing under a per-part capacity; returns boundaries or None."""
    parts, load, used = [0], 0.0, 1
    for i, w in enumerate(weights):
        if w > cap:
            return None
        if load + w > cap:
            used += 1
            if used > num_parts:
                return None
            parts.append(i)
            load = 0.0
        load += w
    while len(parts) < num_parts:
        parts.append(len(weights))
    parts.append(len(weights))
    return parts


def partition_balanced(weights: Sequence[float], num_parts: int) -> List[int]:
    """Contiguous partition minimising the heaviest part (binary search on the bottleneck)."""
    n = len(weights)
    if n <= num_parts:
        return partition_uniform(n, num_parts)
    lo, hi = max(weights), float(sum(weights))
    best = _feasible(weights, num_parts, hi)
    for _ in range(64):
        if hi - lo <= max(1e-9 * hi, 1e-12):
            break
        mid = (lo + hi) / 2
        got = _feasible(weights, num_parts, mid)
        if got is None:
            lo = mid
        else:
            best, hi = got, mid
    # make sure no trailing stage is empty when there are enough weighted layers
    return best


def partition_layers(specs, num_stages: int, method: str = "parameters", param_counts=None) -> List[int]:
    method = (method or "parameters").lower()
    n = len(specs)
    if num_stages == 1:
        return [0, n]
    if method == "uniform":
        return partition_uniform(n, num_stages)
    if method == "parameters":
        if param_counts is None:
            raise ValueError("'parameters' partitioning needs per-layer parameter counts")
        return partition_balanced([float(c) for c in param_counts], num_stages)
    if method.startswith("type:"):
        pat = re.compile(method.split(":", 1)[1], re.IGNORECASE)
        w = [1.0 if pat.search(getattr(s, "typename", type(s).__name__)) else 0.0 for s in specs]
        return partition_balanced(w, num_stages)
    raise NotImplementedError(f"Partitioning method {method} not implemented.")
