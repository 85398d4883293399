"""Megatron ``.bin`` / ``.idx`` indexed token datasets (llm/data/data_utils.py:14-387).

``.idx`` layout: magic ``MMIDIDX\\0\\0``, uint64 version 1, uint8 dtype code, uint64 number of
sequences, uint64 number of document boundaries, then ``sizes`` int32[n], ``pointers``
int64[n] (byte offsets into ``.bin``) and ``doc_idx`` int64[d].  ``.bin`` is the raw token
stream.  Provides the reader, a streaming builder with merge, and the multi-worker
tokenise-to-cache driver used by the ``mmap_index_json`` dataset and the offline builder tool.
"""
from __future__ import annotations

import os
import shutil
import struct
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from ..utils.log import default_logger as logger

DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}
MAGIC = b"MMIDIDX\x00\x00"


def index_file_path(prefix):
    return prefix + ".idx"


def data_file_path(prefix):
    return prefix + ".bin"


def best_fitting_dtype(vocab_size=None):
    return np.uint16 if vocab_size is not None and vocab_size < 65500 else np.int32


def dtype_code(dtype):
    for k, v in DTYPES.items():
        if v == dtype:
            return k
    raise ValueError(dtype)


def num_tokens(documents, sizes):
    return int(np.sum(np.asarray(sizes)[documents]))


def num_epochs_for(tokens_per_epoch, seq_length, num_samples):
    """Epochs needed so that ``(epochs · tokens − 1) // seq_length >= num_samples`` (each sample
    reads seq_length + 1 tokens, the last shared with its successor)."""
    need = num_samples * seq_length + 1
    return max(1, -(-need // tokens_per_epoch))


class MMapIndex:
    def __init__(self, path, skip_warmup=True):
        with open(path, "rb") as f:
            if f.read(9) != MAGIC:
                raise ValueError(f"{path} is not an MMIDIDX index file")
            (version,) = struct.unpack("<Q", f.read(8))
            if version != 1:
                raise ValueError(f"unsupported index version {version}")
            (code,) = struct.unpack("<B", f.read(1))
            self.dtype = DTYPES[code]
            (self._len,) = struct.unpack("<Q", f.read(8))
            (self._doc_count,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self._mmap = np.memmap(path, mode="r", order="C")
        buf = memoryview(self._mmap)
        self.sizes = np.frombuffer(buf, dtype=np.int32, count=self._len, offset=offset)
        self.pointers = np.frombuffer(buf, dtype=np.int64, count=self._len, offset=offset + self.sizes.nbytes)
        self.doc_idx = np.frombuffer(buf, dtype=np.int64, count=self._doc_count,
                                     offset=offset + self.sizes.nbytes + self.pointers.nbytes)

    def __getitem__(self, i):
        return int(self.pointers[i]), int(self.sizes[i])

    def __len__(self):
        return self._len

    @staticmethod
    def write(path, dtype, sizes, doc_idx):
        sizes = np.asarray(sizes, dtype=np.int32)
        pointers = np.zeros(len(sizes), dtype=np.int64)
        if len(sizes) > 1:
            np.cumsum(sizes[:-1].astype(np.int64) * np.dtype(dtype).itemsize, out=pointers[1:])
        with open(path, "wb") as f:
            f.write(MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<B", dtype_code(dtype)))
            f.write(struct.pack("<Q", len(sizes)))
            f.write(struct.pack("<Q", len(doc_idx)))
            f.write(sizes.tobytes(order="C"))
            f.write(pointers.tobytes(order="C"))
            f.write(np.asarray(doc_idx, dtype=np.int64).tobytes(order="C"))


class MMapIndexedDatasetBuilder:
    def __init__(self, out_file, dtype=np.int64):
        self._f = open(out_file, "wb")
        self.dtype = dtype
        self.sizes, self.doc_idx = [], [0]

    def add_item(self, tokens):
        arr = np.asarray(tokens.numpy() if hasattr(tokens, "numpy") else tokens, dtype=self.dtype)
        self._f.write(arr.tobytes(order="C"))
        self.sizes.append(arr.size)

    def end_document(self):
        self.doc_idx.append(len(self.sizes))

    def merge_file_(self, other_prefix):
        idx = MMapIndex(index_file_path(other_prefix))
        if idx.dtype != self.dtype:
            raise ValueError("cannot merge index files of different dtypes")
        base = len(self.sizes)
        self.sizes.extend(int(s) for s in idx.sizes)
        self.doc_idx.extend(int(d) + base for d in idx.doc_idx[1:])
        with open(data_file_path(other_prefix), "rb") as f:
            shutil.copyfileobj(f, self._f)

    def finalize(self, index_file):
        self._f.close()
        MMapIndex.write(index_file, self.dtype, self.sizes, self.doc_idx)


def build_data_cache(encode_fn, tokenizer, json_files, cache_prefix, workers=4, cache_splits=1, log_freq=1000):
    """Tokenise line-JSON files into ``<cache_prefix>.bin/.idx`` (one part per worker, then merged)."""
    dtype = best_fitting_dtype(len(tokenizer))
    lines = []
    for jf in json_files:
        with open(jf, "r", encoding="utf-8") as f:
            lines.extend(l for l in f if l.strip())
    workers = max(1, min(workers, len(lines)))
    chunks = [lines[i::workers] for i in range(workers)]

    def work(args):
        wid, chunk = args
        prefix = f"{cache_prefix}_part{wid}"
        b = MMapIndexedDatasetBuilder(data_file_path(prefix), dtype)
        for n, line in enumerate(chunk):
            item = encode_fn(line)
            if item is None:
                continue
            ids = item["input_ids"] if isinstance(item, dict) else item[0]
            b.add_item(ids)
            b.end_document()
            if log_freq > 0 and (n + 1) % log_freq == 0:
                logger.info(f"worker {wid}: {n + 1} documents tokenised")
        b.finalize(index_file_path(prefix))
        return prefix

    with ThreadPoolExecutor(max_workers=workers) as ex:
        parts = list(ex.map(work, enumerate(chunks)))
    out = MMapIndexedDatasetBuilder(data_file_path(cache_prefix), dtype)
    for p in parts:
        out.merge_file_(p)
        os.remove(data_file_path(p))
        os.remove(index_file_path(p))
    out.finalize(index_file_path(cache_prefix))
    return cache_prefix
