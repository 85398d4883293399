"""``--opts k1 v1 k2 v2`` command-line overrides merged into a loaded config.

Parity: llm/utils/general/cfg_helper.py:14-67.  Keys are dotted paths; the special form
``hooks.<type>-kwargs.x`` addresses the entry of the list ``hooks`` whose ``type`` equals
``<type>`` (appending a new entry when none matches).  Values decode to bool / int / float
/ str in that order.
"""
from __future__ import annotations

import copy
import re

_NUM = re.compile(r"^[-+]?(\d+\.\d*|\.\d+|\d+)([eE][-+]?\d+)?$")


def try_decode(val):
    if not isinstance(val, str):
        return val
    up = val.upper()
    if up == "FALSE":
        return False
    if up == "TRUE":
        return True
    if re.fullmatch(r"[-+]?\d+", val):
        return int(val)
    if _NUM.match(val):
        return float(val)
    return val


def _set_path(node, comps, val):
    for k in comps[:-1]:
        nxt = node.get(k)
        if not isinstance(nxt, dict):
            nxt = {}
            node[k] = nxt
        node = nxt
    node[comps[-1]] = val


def merge_opts_into_cfg(opts, cfg):
    cfg = copy.deepcopy(cfg)
    if not opts:
        return cfg
    if len(opts) % 2:
        raise ValueError("--opts expects an even number of tokens: key value [key value ...]")
    for key, raw in zip(opts[0::2], opts[1::2]):
        val = try_decode(raw)
        if "-" in key:
            head, tail = key.split("-", 1)
            *list_path, want_type = head.split(".")
            node = cfg
            for k in list_path[:-1]:
                node = node.setdefault(k, {})
            entries = node.setdefault(list_path[-1], [])
            hit = False
            for entry in entries:
                if entry.get("type") == want_type:
                    _set_path(entry, tail.split("."), val)
                    hit = True
            if not hit:
                fresh = {}
                _set_path(fresh, tail.split("."), val)
                entries.append(fresh)
        else:
            _set_path(cfg, key.split("."), val)
    return cfg
