"""Datasets (registry ``DATASET_REGISTRY``; llm/data/nlp_dataset.py:23-657).

* ``pretrain_bin``      — token shards ``<size>_<i>.npy`` listed in manifest ``.txt`` files; one
                          sample = ``[shard, start, end)`` of ``seq_length`` tokens.
* ``base_nlp_json``     — whole-file or line JSON records held in memory.
* ``mmap_json``         — line JSON read through ``mmap`` with a cached byte-offset table.
* ``mmap_index_json``   — Megatron ``.bin/.idx`` token stream cut into ``seq_length + 1`` token
                          samples through sentence / location / shuffle index maps (cached as .npy),
                          location map built by the native helper or its Python twin.
* ``synthetic_tokens``  — uniform random ids of a fixed seed (benchmarks).
A bad record is replaced by another one instead of failing the job.  Lists of dataset configs
are concatenated.
"""
from __future__ import annotations

import json
import mmap
import os
import random

import numpy as np
import torch
import torch.distributed as dist
from torch.utils.data import ConcatDataset, Dataset

from ..config.registry import DATASET_REGISTRY
from ..parallel.grid import get_grid
from ..utils.log import default_logger as logger
from .index_utils import (MMapIndex, build_data_cache, data_file_path, index_file_path, num_epochs_for, num_tokens)
from .parsers import build_transformer
from .synthetic import SyntheticTokenDataset

IGNORE_INDEX = -100


def _is_builder_rank():
    g = get_grid()
    return g.pp_rank == 0 and g.tp_rank == 0


def _pp_barrier():
    if dist.is_initialized() and get_grid().pp_group is not None:
        dist.barrier(group=get_grid().pp_group)


def _as_list(x):
    return x if isinstance(x, list) else [x]


class _Transformed(Dataset):
    def _init_transformer(self, transformer, tokenizer):
        self.tokenizer = tokenizer
        self.transformer = build_transformer(transformer, tokenizer) if transformer else None

    def _apply(self, meta):
        return self.transformer(meta) if self.transformer is not None else meta


@DATASET_REGISTRY.register("pretrain_bin")
class PretrainBinDataset(_Transformed):
    def __init__(self, txt_files="", folders=None, tokenizer=None, transformer=None, bin_size=256 * 1024,
                 seq_length=4096, data_root=""):
        files = _as_list(txt_files)
        if folders is not None:
            files = [os.path.join(d, f) for d in _as_list(folders) for f in sorted(os.listdir(d)) if "txt" in f]
        self.bin_paths = []
        for fn in files:
            with open(fn) as f:
                self.bin_paths += [l.strip() for l in f if l.strip()]
        self.data_root = data_root
        rows = []
        full = np.arange(0, bin_size + seq_length, seq_length)
        for i, p in enumerate(self.bin_paths):
            size = int(os.path.basename(p).split("_")[0])
            starts = full[:-1] if size == bin_size else np.arange(size // seq_length + 1) * seq_length
            rows.append(np.stack((np.full(len(starts), i), starts, starts + seq_length), 1))
        self.bin_indexs = np.vstack(rows).astype(np.int32) if rows else np.zeros((0, 3), np.int32)
        self._init_transformer(transformer, tokenizer)

    def get_meta(self, idx):
        bi = self.bin_indexs[idx]
        return self._apply({"path": os.path.join(self.data_root, self.bin_paths[bi[0]]), "bin_index": bi})

    def __getitem__(self, idx):
        try:
            meta = self.get_meta(idx)
        except Exception as e:
            logger.warning(f"pretrain_bin: sample {idx} failed ({e}); resampling")
            meta = None
        rng = random.Random(idx + 3 * get_grid().dp_rank)
        tries = 0
        while meta is None:
            tries += 1
            if tries > 100:
                raise RuntimeError("pretrain_bin: no readable sample found")
            j = rng.randint(0, len(self) - 1)
            if j != idx:
                try:
                    meta = self.get_meta(j)
                except Exception:
                    meta = None
        return meta

    def __len__(self):
        return len(self.bin_indexs)


@DATASET_REGISTRY.register("base_nlp_json")
class BaseNLPJsonDataset(_Transformed):
    def __init__(self, json_file, tokenizer=None, transformer=None, json_type="all"):
        files = _as_list(json_file)
        kinds = json_type if isinstance(json_type, list) else [json_type] * len(files)
        self.metas = []
        for fn, kind in zip(files, kinds):
            with open(fn, "r", encoding="utf-8") as f:
                if kind == "all":
                    self.metas.extend(json.load(f))
                elif kind == "line":
                    self.metas.extend(json.loads(l) for l in f if l.strip())
                else:
                    raise ValueError(f"json_type must be 'all' or 'line', got {kind}")
        self._init_transformer(transformer, tokenizer)

    def get_meta(self, idx):
        return self._apply(self.metas[idx])

    def __getitem__(self, idx):
        meta = self.get_meta(idx)
        tries = 0
        while meta is None:
            idx = (idx + 100) % len(self.metas)
            meta = self.get_meta(idx)
            tries += 1
            if tries > len(self.metas):
                raise RuntimeError("base_nlp_json: every record was dropped by the parser")
        return meta

    def __len__(self):
        return len(self.metas)


@DATASET_REGISTRY.register("mmap_json")
class MMapJsonDataset(_Transformed):
    def __init__(self, json_file=None, folder=None, tokenizer=None, transformer=None, json_type="line",
                 cache_dir="./cache", cache_worker=4):
        if folder is not None:
            json_file = [os.path.join(r, n) for r, _, fs in os.walk(folder) for n in sorted(fs)]
        self.files = _as_list(json_file)
        os.makedirs(cache_dir, exist_ok=True)
        self.position_map, self.maps = [], []
        for fi, fn in enumerate(self.files):
            cache = os.path.join(cache_dir, fn.replace("/", "_").split(".")[0] + "_pos.npy")
            if not os.path.exists(cache) and _is_builder_rank():
                offs, at = [], 0
                with open(fn, "rb") as f:
                    for line in f:
                        offs.append((at, at + len(line)))
                        at += len(line)
                np.save(cache + ".tmp.npy", np.asarray(offs, dtype=np.int64))
                os.replace(cache + ".tmp.npy", cache)
            _pp_barrier()
            offs = np.load(cache)
            self.position_map.extend((int(a), int(b), fi) for a, b in offs)
            with open(fn, "r") as f:
                self.maps.append(mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ))
        self._init_transformer(transformer, tokenizer)

    def __getitem__(self, idx):
        a, b, fi = self.position_map[idx]
        return self._apply(json.loads(self.maps[fi][a:b]))

    def __len__(self):
        return len(self.position_map)


def build_location_idx_py(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch):
    """Python twin of ``cores/helpers.cpp::ell_build_location_idx`` (same output)."""
    n = (num_epochs * tokens_per_epoch - 1) // seq_length
    out = np.zeros((n + 1, 2), dtype=np.int32)
    ends = np.cumsum(np.asarray(sizes, dtype=np.int64)[np.asarray(doc_idx)])
    cursors = np.arange(1, n + 1, dtype=np.int64) * seq_length
    pos = np.searchsorted(ends, cursors, side="right")
    begins = np.concatenate(([0], ends))[pos]
    out[1:, 0] = pos
    out[1:, 1] = cursors - begins
    return out


@DATASET_REGISTRY.register("mmap_index_json")
class MMapIndexJsonDataset(_Transformed):
    def __init__(self, data_root, seed, total_samples, max_seq_length, json_file=None, json_type="line",
                 tokenizer=None, transformer=None, cache_dir="train_data_cache", cache_prefix="mmap_sentebnse",
                 cache_worker=4, cache_skip_warmup=True, cache_log_freq=100, cache_splits=1,
                 cache_location_builder="py", ignore_index=IGNORE_INDEX, cutoff_last_epoch=0.95, with_cu_lens=False):
        self._init_transformer(transformer, tokenizer)
        self.ignore_index, self.with_cu_lens = ignore_index, with_cu_lens
        self.cache_location_builder = cache_location_builder
        self.cache_prefix = os.path.join(data_root, cache_dir, cache_prefix)
        if _is_builder_rank() and not self.exists(self.cache_prefix):
            os.makedirs(os.path.join(data_root, cache_dir), exist_ok=True)
            if json_file is None:
                raise FileNotFoundError(f"no cache {self.cache_prefix}.bin/.idx and no json_file to build it from")
            if json_type != "line":
                raise ValueError("Only line type json can build the .bin/.idx cache")
            build_data_cache(self.data_encode, tokenizer, _as_list(json_file), self.cache_prefix, cache_worker,
                             cache_splits, cache_log_freq)
        _pp_barrier()
        self._index = MMapIndex(index_file_path(self.cache_prefix), cache_skip_warmup)
        self._bin = memoryview(np.memmap(data_file_path(self.cache_prefix), mode="r", order="C"))
        ids = np.arange(len(self._index.sizes), dtype=np.int32)
        self.sentenses_idx, self.location_idx, self.shuffle_idx = self.load_index_mappings(
            ids, self._index.sizes, total_samples, max_seq_length, seed, cutoff_last_epoch)

    def data_encode(self, line):
        return self.transformer(json.loads(line))

    @staticmethod
    def exists(prefix):
        return os.path.exists(index_file_path(prefix)) and os.path.exists(data_file_path(prefix))

    @staticmethod
    def _sentence_idx(ids, epochs, rng, separate_last):
        if not separate_last or epochs == 1:
            out = np.tile(ids, epochs).astype(np.int32)
            rng.shuffle(out)
            return out
        first = MMapIndexJsonDataset._sentence_idx(ids, epochs - 1, rng, False)
        last = MMapIndexJsonDataset._sentence_idx(ids, 1, rng, False)
        return np.concatenate((first, last))

    @staticmethod
    def _shuffle_idx(n_first, total, rng):
        dt = np.uint32 if total < np.iinfo(np.uint32).max - 1 else np.int64
        a = np.arange(n_first, dtype=dt)
        rng.shuffle(a)
        if n_first == total:
            return a
        b = np.arange(n_first, total, dtype=dt)
        rng.shuffle(b)
        return np.concatenate((a, b))

    def load_index_mappings(self, ids, sizes, total_samples, seq_length, seed, cutoff_last_epoch):
        tokens_per_epoch = num_tokens(ids, sizes)
        epochs = num_epochs_for(tokens_per_epoch, seq_length, total_samples)
        rng = np.random.RandomState(seed=seed)
        base = f"{self.cache_prefix}_indexmap_{total_samples}ns_{seq_length}sl_{seed}s"
        f_sen, f_loc, f_shf = base + "_sentense_idx.npy", base + "_location_idx.npy", base + "_shuffle_idx.npy"
        if _is_builder_rank() and not all(os.path.isfile(f) for f in (f_sen, f_loc, f_shf)):
            separate_last, n_before_last = False, 0
            if epochs > 1:
                n_before_last = ((epochs - 1) * tokens_per_epoch - 1) // seq_length
                last = total_samples - n_before_last
                per_epoch = (tokens_per_epoch - 1) // seq_length
                if not 0 <= last <= per_epoch:
                    raise ValueError(f"last epoch sample count {last} outside [0, {per_epoch}]")
                separate_last = last < int(cutoff_last_epoch * per_epoch)
            sen = self._sentence_idx(ids, epochs, rng, separate_last)
            sz32 = np.ascontiguousarray(sizes, dtype=np.int32)
            if self.cache_location_builder == "cpp":
                from .cores.compile import build_location_idx
                loc = build_location_idx(sz32, sen, seq_length, epochs, tokens_per_epoch)
            elif self.cache_location_builder == "py":
                loc = build_location_idx_py(sz32, sen, seq_length, epochs, tokens_per_epoch)
            else:
                raise NotImplementedError(self.cache_location_builder)
            shf = self._shuffle_idx(n_before_last if separate_last else loc.shape[0] - 1, loc.shape[0] - 1, rng)
            for fn, arr in ((f_sen, sen), (f_loc, loc), (f_shf, shf)):
                np.save(fn + ".tmp.npy", arr)
                os.replace(fn + ".tmp.npy", fn)
        _pp_barrier()
        return tuple(np.load(f, mmap_mode="r") for f in (f_sen, f_loc, f_shf))

    def _tokens(self, seq, offset=0, length=None):
        ptr, size = self._index[int(seq)]
        length = size - offset if length is None else length
        return np.frombuffer(self._bin, dtype=self._index.dtype, count=length,
                             offset=ptr + offset * np.dtype(self._index.dtype).itemsize)

    def __len__(self):
        return self.location_idx.shape[0] - 1

    def __getitem__(self, idx):
        i = int(self.shuffle_idx[idx])
        (d0, o0), (d1, o1) = self.location_idx[i], self.location_idx[i + 1]
        if d0 == d1:
            sample = self._tokens(self.sentenses_idx[d0], o0, o1 - o0 + 1)
        else:
            parts = [self._tokens(self.sentenses_idx[d0], o0)]
            parts += [self._tokens(self.sentenses_idx[d]) for d in range(d0 + 1, d1)]
            parts.append(self._tokens(self.sentenses_idx[d1], 0, o1 + 1))
            sample = np.concatenate(parts)
        ids = torch.from_numpy(sample.astype(np.int64))
        out = {"input_ids": ids, "labels": ids.clone()}
        if self.with_cu_lens:
            ends = (np.where(sample == self.tokenizer.eos_token_id)[0] + 1).tolist()
            if not ends or ends[-1] != len(sample):
                ends.append(len(sample))
            cu = [0] + ends
            out["cu_seqlens"] = torch.LongTensor(cu)
            out["position_ids"] = torch.LongTensor([p for a, b in zip(cu[:-1], cu[1:]) for p in range(b - a)])
        return out


@DATASET_REGISTRY.register("synthetic_tokens")
class SyntheticTokens(SyntheticTokenDataset):
    def __init__(self, vocab_size=None, seq_length=4096, num_samples=1 << 20, seed=0, tokenizer=None, **_):
        super().__init__(vocab_size or len(tokenizer), seq_length + 1, num_samples, seed)

    def __getitem__(self, idx):
        g = torch.Generator().manual_seed(self.seed * 1000003 + idx)
        ids = torch.randint(0, self.vocab_size - 1, (self.seq_length,), generator=g, dtype=torch.int64)
        return {"input_ids": ids, "labels": ids.clone()}


def build_dataset(cfg_dataset, tokenizer):
    if isinstance(cfg_dataset, list):
        return ConcatDataset([build_dataset(c, tokenizer) for c in cfg_dataset])
    cfg = {"type": cfg_dataset["type"], "kwargs": dict(cfg_dataset.get("kwargs") or {})}
    cfg["kwargs"]["tokenizer"] = tokenizer
    return DATASET_REGISTRY.build(cfg)
