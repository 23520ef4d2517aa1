#!/usr/bin/env python
"""Pack text into the fixed-length uint16 token files the data loader reads.

    python -m dawn_srw_b200.tools.pretokenize --input a.txt b.jsonl --output data/c4_train
        [--seq-len 512] [--shard-tokens 100000000] [--tokenizer bert-base-uncased]
        [--text-key text] [--max-tokens N] [--resume]

Documents (one per line of a ``.txt`` file, or the ``--text-key`` field of each
``.jsonl`` record) are tokenised, terminated by the separator token and packed
back to back into rows of ``seq_len`` tokens with no padding; the tail that does
not fill a row is dropped.  Output: ``<output>_000.bin``, ``<output>_001.bin``, ...
(uint16, row-major) and ``<output>_meta.json`` listing the shards - the layout
of the reference's C4 preparation (scripts/pretokenize_c4.py:98-383), which
streams the corpus from the Hugging Face hub instead of local files.
``--resume`` keeps completed shards and continues after the documents they
consumed.

The tokenizer must be in the local Hugging Face cache (there is no download
here); ``--tokenizer bytes`` selects a dependency-free byte-level fallback
(ids 0..255, separator 256) for smoke tests.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Iterator, List

import numpy as np


class ByteTokenizer:
    vocab_size, sep_token_id = 257, 256

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8"))


class HFTokenizer:
    def __init__(self, name: str):
        from transformers import AutoTokenizer
        self.tok = AutoTokenizer.from_pretrained(name, local_files_only=True)
        self.vocab_size = len(self.tok)
        self.sep_token_id = self.tok.sep_token_id if self.tok.sep_token_id is not None \
            else self.tok.eos_token_id
        if self.vocab_size > 65536:
            raise SystemExit(f"vocabulary of {name} ({self.vocab_size}) does not fit uint16")

    def encode(self, text: str) -> List[int]:
        return self.tok.encode(text, add_special_tokens=False)


def documents(paths: List[str], text_key: str) -> Iterator[str]:
    for p in paths:
        with open(p, "r", encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                if p.endswith(".jsonl") or p.endswith(".json"):
                    try:
                        line = json.loads(line).get(text_key, "")
                    except json.JSONDecodeError:
                        continue
                if line:
                    yield line


def meta_path(output: str) -> str:
    return output + "_meta.json"


def write_meta(output: str, meta: dict) -> None:
    tmp = meta_path(output) + ".tmp"
    with open(tmp, "w") as f:
        json.dump(meta, f, indent=2)
    os.replace(tmp, meta_path(output))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", nargs="+", required=True)
    ap.add_argument("--output", required=True, help="prefix of the shard files")
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--shard-tokens", type=int, default=100_000_000)
    ap.add_argument("--tokenizer", default="bert-base-uncased")
    ap.add_argument("--text-key", default="text")
    ap.add_argument("--max-tokens", type=int, default=0)
    ap.add_argument("--resume", action="store_true")
    args = ap.parse_args(argv)
    tok = ByteTokenizer() if args.tokenizer == "bytes" else HFTokenizer(args.tokenizer)
    S = args.seq_len
    rows_per_shard = max(1, args.shard_tokens // S)
    os.makedirs(os.path.dirname(os.path.abspath(args.output)), exist_ok=True)
    meta = {"seq_len": S, "vocab_size": tok.vocab_size, "tokenizer": args.tokenizer, "dtype": "uint16",
            "shards": [], "documents": 0, "complete": False}
    skip_docs = 0
    if args.resume and os.path.exists(meta_path(args.output)):
        with open(meta_path(args.output)) as f:
            old = json.load(f)
        if old.get("seq_len") == S and old.get("tokenizer") == args.tokenizer:
            meta["shards"] = [s for s in old["shards"] if os.path.exists(
                os.path.join(os.path.dirname(os.path.abspath(args.output)), os.path.basename(s["path"])))]
            skip_docs = meta["shards"][-1]["documents_end"] if meta["shards"] else 0
            meta["documents"] = skip_docs
    buf: List[int] = []
    rows: List[np.ndarray] = []
    total = sum(s["tokens"] for s in meta["shards"])
    n_docs = 0

    def flush():
        nonlocal rows, total
        if not rows:
            return
        idx = len(meta["shards"])
        path = f"{args.output}_{idx:03d}.bin"
        arr = np.stack(rows).astype(np.uint16)
        tmp = path + ".tmp"
        arr.tofile(tmp)
        os.replace(tmp, path)
        meta["shards"].append({"path": os.path.basename(path), "tokens": int(arr.size),
                               "sequences": int(arr.shape[0]), "documents_end": n_docs})
        meta["documents"] = n_docs
        total += int(arr.size)
        write_meta(args.output, meta)
        rows = []

    done = False
    for doc in documents(args.input, args.text_key):
        n_docs += 1
        if n_docs <= skip_docs:
            continue
        buf.extend(tok.encode(doc))
        buf.append(tok.sep_token_id)
        while len(buf) >= S:
            rows.append(np.asarray(buf[:S], dtype=np.uint16))
            buf = buf[S:]
            if len(rows) == rows_per_shard:
                # a shard ends on a document boundary of the packed stream: the unfinished
                # row restarts with the next document after a resume
                flush()
            if args.max_tokens and total + len(rows) * S >= args.max_tokens:
                done = True
                break
        if done:
            break
    flush()
    meta["complete"] = True
    write_meta(args.output, meta)
    print(json.dumps({"shards": len(meta["shards"]), "tokens": total, "documents": meta["documents"],
                      "meta": meta_path(args.output)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
