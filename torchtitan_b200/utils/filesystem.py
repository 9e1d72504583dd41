"""Path helpers that work on local paths and on fsspec URIs (``s3://bucket/run``, ``gs://...``, ``memory://...``).

A path is remote when it starts with ``<protocol>://``; everything else goes to ``os`` / ``shutil`` so that local
runs never import fsspec.  Used by the checkpoint manager for step discovery, retention and folder creation; the
checkpoint payload itself is written by ``torch.distributed.checkpoint``, which picks its fsspec storage from the
same kind of URI.

Parity: torchtitan/tools/filesystem.py:22-114.
"""

from __future__ import annotations

import os
import re
import shutil

__all__ = ["is_remote", "exists", "isdir", "isfile", "listdir", "rmtree", "join", "makedirs", "open_file"]

_URI = re.compile(r"^[A-Za-z][A-Za-z0-9+.\-]*://")


def is_remote(path: str) -> bool:
    return bool(_URI.match(str(path))) and not str(path).startswith("file://")


def _resolve(path: str):
    """``(filesystem, path inside it)`` of a remote path."""
    try:
        import fsspec
    except ImportError as e:      # pragma: no cover - fsspec ships with the image
        raise RuntimeError(f"'{path}' needs the fsspec package") from e
    fs, inner = fsspec.core.url_to_fs(path)
    return fs, inner


def _local(path: str) -> str:
    return path[len("file://"):] if str(path).startswith("file://") else path


def exists(path: str) -> bool:
    if is_remote(path):
        fs, p = _resolve(path)
        return fs.exists(p)
    return os.path.exists(_local(path))


def isdir(path: str) -> bool:
    if is_remote(path):
        fs, p = _resolve(path)
        return fs.isdir(p)
    return os.path.isdir(_local(path))


def isfile(path: str) -> bool:
    if is_remote(path):
        fs, p = _resolve(path)
        return fs.isfile(p)
    return os.path.isfile(_local(path))


def listdir(path: str) -> list[str]:
    """Base names of the entries of a directory (empty when it does not exist)."""
    if is_remote(path):
        fs, p = _resolve(path)
        if not fs.exists(p):
            return []
        return sorted({str(e).rstrip("/").rsplit("/", 1)[-1] for e in fs.ls(p, detail=False)})
    p = _local(path)
    return sorted(os.listdir(p)) if os.path.isdir(p) else []


def rmtree(path: str, ignore_errors: bool = True) -> None:
    if is_remote(path):
        fs, p = _resolve(path)
        try:
            fs.rm(p, recursive=True)
        except Exception:
            if not ignore_errors:
                raise
        return
    shutil.rmtree(_local(path), ignore_errors=ignore_errors)


def join(base: str, *parts: str) -> str:
    if is_remote(base):
        return "/".join([str(base).rstrip("/"), *(str(p).strip("/") for p in parts)])
    return os.path.join(base, *parts)


def makedirs(path: str) -> None:
    if is_remote(path):
        fs, p = _resolve(path)
        fs.makedirs(p, exist_ok=True)
        return
    os.makedirs(_local(path), exist_ok=True)


def open_file(path: str, mode: str = "r"):
    if is_remote(path):
        fs, p = _resolve(path)
        return fs.open(p, mode)
    return open(_local(path), mode)
