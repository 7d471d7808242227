#!/usr/bin/env python
"""Tokenize a text corpus into the ``.bin`` shards that ``dion_b200.models.data`` reads.

Each shard is a 256 x int32 header (magic 20240520, version 1, token count) followed by uint16
GPT-2 tokens; every document is preceded by the end-of-text token; shard 0 is the validation
split (``fineweb_val_000000.bin``), later shards are ``fineweb_train_%06d.bin``.  This is the
role of data/fineweb.py in the reference; here the tokenizer workers stream documents through a
bounded queue and a single writer packs them, so memory stays at one shard.

Sources (``--source``):
  hf:<dataset>[:<config>]   a Hugging Face dataset with a ``text`` column (needs ``datasets``
                            and network access), e.g. ``hf:HuggingFaceFW/fineweb-edu``
  txt:<glob>                local text files, one document per file
  jsonl:<glob>              local JSON-lines files with a ``text`` field

    python data/prepare_fineweb.py --source hf:HuggingFaceFW/fineweb-edu --out data/FineWebEdu
"""
from __future__ import annotations

import argparse
import glob
import json
import multiprocessing as mp
import os
import sys
from typing import Iterable, Iterator

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from dion_b200.models.data import write_datafile  # noqa: E402

_ENC = None


def _encoder():
    global _ENC
    if _ENC is None:
        try:
            import tiktoken
        except ImportError as exc:  # pragma: no cover - optional dependency
            raise SystemExit("tiktoken is required for tokenization: pip install tiktoken") from exc
        _ENC = tiktoken.get_encoding("gpt2")
    return _ENC


def tokenize_document(text: str) -> np.ndarray:
    enc = _encoder()
    ids = [enc.eot_token]
    ids.extend(enc.encode_ordinary(text))
    arr = np.asarray(ids, dtype=np.int64)
    if arr.max(initial=0) >= 2 ** 16:
        raise ValueError("token id does not fit uint16")
    return arr.astype(np.uint16)


def documents(source: str) -> Iterator[str]:
    kind, _, spec = source.partition(":")
    if kind == "hf":
        try:
            from datasets import load_dataset
        except ImportError as exc:  # pragma: no cover - optional dependency
            raise SystemExit("the `datasets` package is required for hf: sources") from exc
        name, _, config = spec.partition(":")
        ds = load_dataset(name, name=config or "default", split="train", streaming=True)
        for row in ds:
            yield row["text"]
    elif kind == "txt":
        for path in sorted(glob.glob(spec)):
            with open(path, encoding="utf-8") as f:
                yield f.read()
    elif kind == "jsonl":
        for path in sorted(glob.glob(spec)):
            with open(path, encoding="utf-8") as f:
                for line in f:
                    if line.strip():
                        yield json.loads(line)["text"]
    else:
        raise SystemExit(f"unknown source {source!r}")


class ShardWriter:
    """Packs token arrays into fixed-size shards; a document that straddles a boundary is cut
    and its tail opens the next shard."""

    def __init__(self, out_dir: str, shard_size: int, prefix: str = "fineweb"):
        self.out_dir, self.shard_size, self.prefix = out_dir, shard_size, prefix
        self.buf = np.empty(shard_size, dtype=np.uint16)
        self.fill = 0
        self.index = 0
        self.files = []
        os.makedirs(out_dir, exist_ok=True)

    def _flush(self, count: int) -> None:
        split = "val" if self.index == 0 else "train"
        path = os.path.join(self.out_dir, f"{self.prefix}_{split}_{self.index:06d}.bin")
        write_datafile(path, self.buf[:count])
        self.files.append(path)
        self.index += 1
        self.fill = 0

    def add(self, tokens: np.ndarray) -> None:
        pos = 0
        while pos < len(tokens):
            take = min(len(tokens) - pos, self.shard_size - self.fill)
            self.buf[self.fill:self.fill + take] = tokens[pos:pos + take]
            self.fill += take
            pos += take
            if self.fill == self.shard_size:
                self._flush(self.shard_size)

    def close(self):
        if self.fill:
            self._flush(self.fill)
        return self.files


def build_shards(docs: Iterable[str], out_dir: str, shard_size: int, workers: int,
                 tokenize=tokenize_document):
    writer = ShardWriter(out_dir, shard_size)
    if workers <= 1:
        for doc in docs:
            writer.add(tokenize(doc))
    else:
        with mp.Pool(workers) as pool:
            for tokens in pool.imap(tokenize, docs, chunksize=16):
                writer.add(tokens)
    return writer.close()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--source", default="hf:HuggingFaceFW/fineweb-edu")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(__file__), "FineWebEdu"))
    ap.add_argument("-s", "--shard_size", type=int, default=10 ** 8, help="tokens per shard")
    ap.add_argument("--workers", type=int, default=max(1, (os.cpu_count() or 2) - 2))
    args = ap.parse_args()
    files = build_shards(documents(args.source), args.out, args.shard_size, args.workers)
    print(f"wrote {len(files)} shard(s) to {args.out}")


if __name__ == "__main__":
    main()
