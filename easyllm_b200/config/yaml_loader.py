"""YAML config loader with ``!include`` and top-level ``overwrite@`` / ``override@`` patches.

Behavioural parity with the reference loader (llm/utils/general/yaml_loader.py:6-128):

* ``key: !include other.yaml`` inlines another file (path relative to the including file);
  ``!include other.yaml//a.b//0`` additionally walks into the loaded document, where
  ``//`` and ``.`` both separate path components and integer components index lists.
* a top-level ``overwrite@`` (or ``override@``) mapping of ``dotted.path: value`` entries is
  applied to the document after it is built and then removed.  Paths are applied in sorted
  order, missing dict levels are created, list indices may append one element.

The implementation is a post-processing pass over a plain ``yaml.SafeLoader``-style load
instead of a loader subclass with document hooks: includes are represented by a marker
object while parsing and resolved afterwards, which keeps file handling (and the include
cache) outside of PyYAML's constructor machinery.
"""
from __future__ import annotations

import os
import re
from typing import Any, Dict

import yaml

_OVERWRITE_KEYS = ("overwrite@", "override@")
_INCLUDE_CACHE: Dict[str, Any] = {}


class _Include:
    __slots__ = ("spec",)

    def __init__(self, spec: str):
        self.spec = spec


class _Loader(yaml.Loader):
    pass


def _include_ctor(loader, node):
    return _Include(loader.construct_scalar(node))


_Loader.add_constructor("!include", _include_ctor)


def _split_include(spec: str):
    parts = spec.split("//", 1)
    if len(parts) == 1:
        return parts[0], []
    return parts[0], [p for p in re.split(r"//|\.", parts[1]) if p != ""]


def _walk(doc, comps):
    for c in comps:
        doc = doc[int(c)] if isinstance(doc, list) else doc[c]
    return doc


def _resolve_includes(obj, root):
    if isinstance(obj, _Include):
        fname, comps = _split_include(obj.spec)
        path = os.path.normpath(os.path.join(root, fname))
        if path not in _INCLUDE_CACHE:
            _INCLUDE_CACHE[path] = load_yaml(path)
        return _walk(_INCLUDE_CACHE[path], comps)
    if isinstance(obj, dict):
        return {k: _resolve_includes(v, root) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_resolve_includes(v, root) for v in obj]
    return obj


def _path_sort_key(data, dotted):
    cur, out = data, []
    for comp in dotted.split("."):
        if isinstance(cur, list):
            comp = int(comp)
        try:
            cur = cur[comp]
        except Exception:
            cur = {}
        # mixed int/str components sort by (type tag, value)
        out.append((0, comp) if isinstance(comp, int) else (1, comp))
    return tuple(out)


def _assign(data, dotted, value):
    keys = dotted.split(".")
    cur = data
    for i, k in enumerate(keys):
        last = i == len(keys) - 1
        if isinstance(cur, dict):
            if last:
                cur[k] = value
                return
            if k not in cur or cur[k] is None:
                cur[k] = {}
            cur = cur[k]
        elif isinstance(cur, list):
            idx = int(k)
            if idx > len(cur):
                raise IndexError(f"overwrite path {dotted!r}: index {idx} beyond list of {len(cur)}")
            if last:
                if idx < len(cur):
                    cur[idx] = value
                else:
                    cur.append(value)
                return
            if idx == len(cur):
                cur.append({})
            cur = cur[idx]
        else:
            raise ValueError(f"invalid overwrite {dotted!r} -> {value!r}")


def apply_overwrites(data):
    """Apply and strip ``overwrite@``/``override@`` blocks of a loaded document."""
    if not isinstance(data, dict):
        return data
    for key in _OVERWRITE_KEYS:
        if key in data:
            patches = data.pop(key) or {}
            for dotted, v in sorted(patches.items(), key=lambda kv: _path_sort_key(data, kv[0])):
                _assign(data, dotted, v)
    return data


def load_yaml(path: str):
    """Load ``path`` resolving ``!include`` nodes and ``overwrite@`` patches."""
    with open(path, "r") as f:
        raw = yaml.load(f, _Loader)
    data = _resolve_includes(raw, os.path.dirname(os.path.abspath(path)))
    return apply_overwrites(data)


def clear_include_cache():
    _INCLUDE_CACHE.clear()
