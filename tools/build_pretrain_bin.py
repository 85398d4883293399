"""jsonl (``content`` field) → token shards ``<size>_<i>.npy`` + a ``.txt`` manifest for the
``pretrain_bin`` dataset (tools/build_pretrain_bin.py:30-194 of the reference).

    python tools/build_pretrain_bin.py --tokenizer_path tok --jsonl data.jsonl --out_dir bins \
        --bin_size 262144 [--workers 8] [--tokenizer_type LlamaTokenizer]

Long documents are split on newlines / sentence punctuation before tokenisation (tokenizer
speed), every document ends with EOS, tokens are concatenated and cut into shards of
``bin_size`` tokens (the last shard keeps its real size in its file name).
"""
import argparse
import json
import os
import re
import sys
from concurrent.futures import ThreadPoolExecutor

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

_SPLIT = re.compile(r"(?<=[\n。！？!?\.])")


def split_text(text, max_chars=4000):
    if len(text) <= max_chars:
        return [text]
    out, cur = [], ""
    for piece in _SPLIT.split(text):
        if len(cur) + len(piece) > max_chars and cur:
            out.append(cur)
            cur = ""
        cur += piece
    if cur:
        out.append(cur)
    return out


def encode_doc(tokenizer, text):
    ids = []
    for i, part in enumerate(split_text(text)):
        ids.extend(tokenizer(part, add_special_tokens=(i == 0))["input_ids"])
    return ids + [tokenizer.eos_token_id]


def main(argv=None):
    from easyllm_b200.data import build_tokenizer
    p = argparse.ArgumentParser()
    p.add_argument("--tokenizer_path", default=None)
    p.add_argument("--tokenizer_type", default="LlamaTokenizer")
    p.add_argument("--jsonl", required=True, nargs="+")
    p.add_argument("--out_dir", required=True)
    p.add_argument("--bin_size", type=int, default=256 * 1024)
    p.add_argument("--workers", type=int, default=8)
    p.add_argument("--content_key", default="content")
    a = p.parse_args(argv)
    kw = {"tokenizer_name_or_path": a.tokenizer_path} if a.tokenizer_path else {}
    tok = build_tokenizer({"type": a.tokenizer_type, "kwargs": kw})
    os.makedirs(a.out_dir, exist_ok=True)
    docs = []
    for fn in a.jsonl:
        with open(fn, encoding="utf-8") as f:
            docs += [json.loads(l)[a.content_key] for l in f if l.strip()]
    with ThreadPoolExecutor(max_workers=a.workers) as ex:
        encoded = list(ex.map(lambda t: encode_doc(tok, t), docs))
    stream = np.fromiter((t for d in encoded for t in d), dtype=np.int64)
    dtype = np.uint16 if len(tok) < 65500 else np.int32
    paths = []
    for i, start in enumerate(range(0, len(stream), a.bin_size)):
        chunk = stream[start:start + a.bin_size].astype(dtype)
        path = os.path.join(a.out_dir, f"{len(chunk)}_{i}.npy")
        np.save(path, chunk)
        paths.append(os.path.abspath(path))
    manifest = os.path.join(a.out_dir, "bins.txt")
    with open(manifest, "w") as f:
        f.write("\n".join(paths) + "\n")
    print(f"{len(docs)} documents, {len(stream)} tokens, {len(paths)} shards -> {manifest}")


if __name__ == "__main__":
    main()
