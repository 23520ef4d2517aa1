"""File access for configs, logs and checkpoints: local paths directly, URL
paths (``gs://``, ``s3://``, ``memory://`` ...) through fsspec when the matching
filesystem package is installed.

The reference wraps the same five operations over local files and GCS
(scripts/train_jax.py:221-361: ``_open_file``, ``_file_exists``,
``_list_files``, ``_delete_file``, ``_makedirs``).  Token ``.bin`` files are
memory-mapped and therefore must be local; ``fetch_to_local`` copies a remote
one into a cache directory first (the reference's ``local_cache_dir``).
"""
from __future__ import annotations

import glob
import os
import shutil
from typing import List


def is_remote(path: str) -> bool:
    return "://" in str(path) and not str(path).startswith("file://")


def _fs(path: str):
    try:
        import fsspec
    except ImportError as e:                      # pragma: no cover
        raise RuntimeError(f"{path}: URL paths need the fsspec package") from e
    try:
        return fsspec.core.url_to_fs(path)
    except (ImportError, ValueError) as e:
        raise RuntimeError(f"{path}: no filesystem driver for this URL scheme is installed "
                           f"({e}); copy the files locally or install the driver") from e


def open_file(path: str, mode: str = "r"):
    if is_remote(path):
        fs, p = _fs(path)
        return fs.open(p, mode)
    if any(c in mode for c in "wa"):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    return open(path, mode)


def file_exists(path: str) -> bool:
    if is_remote(path):
        fs, p = _fs(path)
        return fs.exists(p)
    return os.path.exists(path)


def list_files(pattern: str) -> List[str]:
    """Glob; remote results keep their URL scheme."""
    if is_remote(pattern):
        fs, p = _fs(pattern)
        scheme = pattern.split("://", 1)[0]
        return sorted(f"{scheme}://{q.lstrip('/')}" if not str(q).startswith(scheme) else q
                      for q in fs.glob(p))
    return sorted(glob.glob(pattern))


def delete_file(path: str) -> None:
    if is_remote(path):
        fs, p = _fs(path)
        fs.rm(p)
    elif os.path.exists(path):
        os.remove(path)


def makedirs(path: str) -> None:
    if is_remote(path):
        fs, p = _fs(path)
        fs.makedirs(p, exist_ok=True)
    else:
        os.makedirs(path, exist_ok=True)


def fetch_to_local(path: str, cache_dir: str) -> str:
    """Local path of ``path``: itself when local, else a copy under ``cache_dir``
    (downloaded once; a partial download never becomes visible)."""
    if not is_remote(path):
        return path
    os.makedirs(cache_dir, exist_ok=True)
    dst = os.path.join(cache_dir, path.split("://", 1)[1].replace("/", "_"))
    if not os.path.exists(dst):
        with open_file(path, "rb") as src, open(dst + ".part", "wb") as out:
            shutil.copyfileobj(src, out, length=16 << 20)
        os.replace(dst + ".part", dst)
    return dst
