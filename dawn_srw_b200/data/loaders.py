"""Token data sources.

File formats are the reference's (utils/data_jax.py:129-517):

* ``BinDataset``: a flat little-endian ``uint16`` token file, memory-mapped and
  viewed as ``[n_seq, seq_len]`` (trailing tokens that do not fill a sequence
  are dropped).
* ``ShardedBinDataset``: a directory / prefix with ``_meta.json`` =
  ``{"shards": [{"path", "sequences", "tokens"}, ...], "vocab_size",
  "num_shards"}``; one shard is resident at a time.
* ``SyntheticDataset``: uniform-random token ids from a seed (benchmarks and
  tests; there is no dataset on the benchmark machines).

``BinDataLoader`` yields ``(input_ids, attention_mask)`` int32 batches in
sequential order.  Every rank reads only its slice of each global batch
(``batch_index`` of ``batch_replicas``), ``reset(start_step)`` repositions the
stream for a mid-epoch resume, and batches are staged in pinned host memory so
the host-to-device copy can be asynchronous.
"""
from __future__ import annotations

import json
import os
from typing import Iterator, List, Optional, Tuple

import numpy as np
import torch

from ..utils.fileio import fetch_to_local, is_remote


class BinDataset:
    def __init__(self, path: str, seq_len: int, max_tokens: Optional[int] = None):
        self.path, self.seq_len = path, seq_len
        self.data = np.memmap(path, dtype=np.uint16, mode="r")
        n_tok = len(self.data) if not max_tokens else min(len(self.data), int(max_tokens))
        self.n_seq = n_tok // seq_len
        self.vocab_size = None

    def __len__(self):
        return self.n_seq

    def rows(self, lo: int, hi: int) -> np.ndarray:
        s = self.seq_len
        return np.asarray(self.data[lo * s: hi * s]).reshape(hi - lo, s)


class ShardedBinDataset:
    def __init__(self, meta_path: str, seq_len: int, max_tokens: Optional[int] = None):
        if os.path.isdir(meta_path):
            meta_path = os.path.join(meta_path, "_meta.json")
        with open(meta_path) as f:
            meta = json.load(f)
        base = os.path.dirname(meta_path)
        self.seq_len = seq_len
        self.vocab_size = meta.get("vocab_size")
        self.shards: List[Tuple[str, int]] = []
        budget = int(max_tokens) if max_tokens else None
        for sh in meta["shards"]:
            n_seq = int(sh.get("sequences", sh["tokens"] // seq_len))
            if budget is not None:
                n_seq = min(n_seq, budget // seq_len)
                budget -= n_seq * seq_len
            if n_seq <= 0:
                break
            p = sh["path"]
            self.shards.append((p if os.path.isabs(p) else os.path.join(base, os.path.basename(p)), n_seq))
        self.offsets = np.cumsum([0] + [n for _, n in self.shards])
        self.n_seq = int(self.offsets[-1])
        self._resident = (-1, None)

    def __len__(self):
        return self.n_seq

    def _shard(self, i: int) -> np.ndarray:
        if self._resident[0] != i:
            path, n = self.shards[i]
            self._resident = (i, np.memmap(path, dtype=np.uint16, mode="r"))
        return self._resident[1]

    def rows(self, lo: int, hi: int) -> np.ndarray:
        out = np.empty((hi - lo, self.seq_len), dtype=np.uint16)
        pos = lo
        while pos < hi:
            si = int(np.searchsorted(self.offsets, pos, side="right") - 1)
            a = pos - int(self.offsets[si])
            take = min(hi - pos, self.shards[si][1] - a)
            s = self.seq_len
            out[pos - lo: pos - lo + take] = np.asarray(self._shard(si)[a * s:(a + take) * s]).reshape(take, s)
            pos += take
        return out


class SyntheticDataset:
    """Uniform-random tokens; row ``i`` depends only on (seed, i)."""

    def __init__(self, n_seq: int, seq_len: int, vocab_size: int, seed: int = 0):
        self.n_seq, self.seq_len, self.vocab_size, self.seed = n_seq, seq_len, vocab_size, seed

    def __len__(self):
        return self.n_seq

    def rows(self, lo: int, hi: int) -> np.ndarray:
        out = np.empty((hi - lo, self.seq_len), dtype=np.int64)
        for i in range(lo, hi):
            out[i - lo] = np.random.default_rng((self.seed, i)).integers(0, self.vocab_size, self.seq_len)
        return out


class BinDataLoader:
    def __init__(self, dataset, global_batch: int, batch_index: int = 0, batch_replicas: int = 1,
                 pin: bool = True, prefetch: int = 2):
        if global_batch % batch_replicas != 0:
            raise ValueError(f"global batch {global_batch} is not divisible by "
                             f"{batch_replicas} batch shards")
        self.ds, self.global_batch = dataset, global_batch
        self.local_batch = global_batch // batch_replicas
        self.batch_index = batch_index
        self.steps = len(dataset) // global_batch
        self.start_step = 0
        self.pin = pin and torch.cuda.is_available()
        self.prefetch = max(0, int(prefetch))     # batches prepared ahead by a background thread

    def __len__(self):
        return self.steps

    def reset(self, start_step: int = 0):
        self.start_step = int(start_step)

    def batch(self, step: int) -> Tuple[torch.Tensor, torch.Tensor]:
        lo = step * self.global_batch + self.batch_index * self.local_batch
        rows = self.ds.rows(lo, lo + self.local_batch)
        ids = torch.from_numpy(rows.astype(np.int32))
        mask = torch.ones_like(ids)
        if self.pin:
            ids, mask = ids.pin_memory(), mask.pin_memory()
        return ids, mask

    def __iter__(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        """Batches ``start_step .. steps-1`` in order.  With ``prefetch > 0`` a
        background thread reads, converts and pins up to that many batches ahead
        of the consumer (file reads and pinning overlap the training step); the
        sequence of batches is the same as without it."""
        first, self.start_step = self.start_step, 0
        if self.prefetch == 0 or self.steps - first <= 1:
            for step in range(first, self.steps):
                yield self.batch(step)
            return
        import queue
        import threading
        q: "queue.Queue" = queue.Queue(maxsize=self.prefetch)
        stop = threading.Event()

        def produce():
            try:
                for step in range(first, self.steps):
                    if stop.is_set():
                        return
                    item = self.batch(step)
                    while not stop.is_set():
                        try:
                            q.put(item, timeout=0.1)
                            break
                        except queue.Full:
                            continue
                q.put(None)
            except BaseException as e:            # surfaces in the consumer, never lost in the thread
                q.put(e)

        th = threading.Thread(target=produce, daemon=True, name="dawn-data-prefetch")
        th.start()
        try:
            while True:
                item = q.get()
                if item is None:
                    return
                if isinstance(item, BaseException):
                    raise item
                yield item
        finally:
            stop.set()


def load_data(data_cfg, seq_len: int, global_batch: int, vocab_size: int, *, batch_index=0,
              batch_replicas=1, seed=0):
    """(train_loader, val_loader, vocab_size) from the ``data`` config section."""
    def open_ds(path, max_tokens):
        if path is None:
            return None
        if is_remote(path):
            # token files are memory-mapped: fetch a remote one into the local cache first
            cache = getattr(data_cfg, "local_cache_dir", None)
            if not cache:
                raise ValueError(f"{path}: set data.local_cache_dir so the remote token file can be "
                                 "copied next to the trainer (token files are memory-mapped)")
            path = fetch_to_local(path, cache)
        if os.path.isdir(path) or path.endswith("_meta.json") or os.path.exists(path + "_meta.json"):
            meta = path if not os.path.exists(path + "_meta.json") else path + "_meta.json"
            return ShardedBinDataset(meta, seq_len, max_tokens)
        return BinDataset(path, seq_len, max_tokens)

    if getattr(data_cfg, "synthetic", False) or data_cfg.bin_train is None:
        n = max(getattr(data_cfg, "synthetic_sequences", 4096), global_batch)
        train = SyntheticDataset(n, seq_len, vocab_size, seed)
        val = SyntheticDataset(max(global_batch, n // 8), seq_len, vocab_size, seed + 1)
    else:
        train = open_ds(data_cfg.bin_train, data_cfg.max_train_tokens)
        val = open_ds(data_cfg.bin_val, data_cfg.max_val_tokens)
        if getattr(train, "vocab_size", None):
            vocab_size = int(train.vocab_size)
    tl = BinDataLoader(train, global_batch, batch_index, batch_replicas)
    vl = BinDataLoader(val, global_batch, batch_index, batch_replicas) if val is not None else None
    return tl, vl, vocab_size
