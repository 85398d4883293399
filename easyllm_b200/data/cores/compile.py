"""Build and load the native index helpers (``libellhelpers.so``, g++ only, no Python headers)."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libellhelpers.so")
_lib = None


def build(force=False):
    src = os.path.join(HERE, "helpers.cpp")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        r = subprocess.run(["make", "-C", HERE, "-B"], capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(f"building helpers.cpp failed:\n{r.stdout}\n{r.stderr}")
    return LIB


compile_helper = build


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.ell_build_location_idx.restype = ctypes.c_int64
        _lib.ell_build_pack_index.restype = ctypes.c_int64
    return _lib


def build_location_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch):
    """int32 ``[num_samples + 1, 2]`` of (doc_idx position, offset) per sample boundary."""
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    doc_idx = np.ascontiguousarray(doc_idx, dtype=np.int32)
    n = (num_epochs * tokens_per_epoch - 1) // seq_length
    out = np.zeros((n + 1, 2), dtype=np.int32)
    got = lib().ell_build_location_idx(sizes.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(len(sizes)),
                                       doc_idx.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(len(doc_idx)),
                                       ctypes.c_int32(seq_length), ctypes.c_int32(num_epochs),
                                       ctypes.c_int64(tokens_per_epoch), out.ctypes.data_as(ctypes.c_void_p))
    if got != n + 1:
        raise ValueError("inconsistent sizes / doc_idx / tokens_per_epoch for build_location_idx")
    return out


def build_pack_index(lengths, capacity):
    lengths = np.ascontiguousarray(lengths, dtype=np.int32)
    bins = np.zeros(len(lengths), dtype=np.int32)
    n = lib().ell_build_pack_index(lengths.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(len(lengths)),
                                   ctypes.c_int32(capacity), bins.ctypes.data_as(ctypes.c_void_p))
    return bins, int(n)
