"""File operations behind one set of functions, keyed by URL scheme.

Counterpart of axlearn/common/file_system.py:90-179 (``isdir``, ``listdir``, ``glob``, ``exists``,
``remove``, ``copy``, ``open``, ``readfile``, ``makedirs``, ``rmtree`` over local paths and object
stores).  Local paths and ``file://`` URLs are built in; another scheme (an object store, a
parallel file system client) is added with ``register_backend(scheme, backend)`` where the backend
provides the same functions.  Errors are ``OpError`` / ``NotFoundError`` whatever the backend.
"""

from __future__ import annotations

import builtins
import glob as _glob
import os
import shutil
from typing import IO, Any, Sequence, Union


class OpError(Exception):
    pass


class NotFoundError(OpError):
    pass


class _Local:
    @staticmethod
    def _p(path: str) -> str:
        return path[len("file://"):] if path.startswith("file://") else path

    def isdir(self, path):
        return os.path.isdir(self._p(path))

    def listdir(self, path):
        return sorted(os.listdir(self._p(path)))

    def glob(self, pattern):
        return sorted(_glob.glob(self._p(pattern)))

    def exists(self, path):
        return os.path.exists(self._p(path))

    def remove(self, path):
        os.remove(self._p(path))

    def copy(self, src, dst, overwrite=False):
        src, dst = self._p(src), self._p(dst)
        if os.path.exists(dst) and not overwrite:
            raise OpError(f"{dst} exists")
        tmp = f"{dst}.tmp{os.getpid()}"
        shutil.copyfile(src, tmp)
        os.replace(tmp, dst)                       # readers never see a partial file

    def open(self, path, mode="r"):
        return builtins.open(self._p(path), mode)

    def makedirs(self, path):
        os.makedirs(self._p(path), exist_ok=True)

    def rmtree(self, path):
        shutil.rmtree(self._p(path))


_BACKENDS: dict[str, Any] = {"": _Local(), "file": _Local()}


def register_backend(scheme: str, backend: Any) -> None:
    _BACKENDS[scheme] = backend


def _backend(path: str):
    scheme = path.split("://", 1)[0] if "://" in path else ""
    if scheme not in _BACKENDS:
        raise OpError(f"no file-system backend registered for scheme {scheme!r} ({path})")
    return _BACKENDS[scheme]


def _call(name: str, path: str, *args, **kwargs):
    try:
        return getattr(_backend(path), name)(path, *args, **kwargs)
    except FileNotFoundError as e:
        raise NotFoundError(str(e)) from e
    except OpError:
        raise
    except OSError as e:
        raise OpError(str(e)) from e


def isdir(path: str) -> bool:
    return _call("isdir", path)


def listdir(path: str) -> list[str]:
    return _call("listdir", path)


def glob(pattern: Union[str, Sequence[str]]) -> list[str]:
    patterns = [pattern] if isinstance(pattern, str) else list(pattern)
    out: list[str] = []
    for p in patterns:
        out.extend(_call("glob", p))
    return out


def exists(path: str) -> bool:
    return _call("exists", path)


def remove(path: str) -> None:
    _call("remove", path)


def copy(src: str, dst: str, overwrite: bool = False) -> None:
    if _backend(src) is _backend(dst):
        _call("copy", src, dst, overwrite)
        return
    if exists(dst) and not overwrite:
        raise OpError(f"{dst} exists")
    with open(src, "rb") as fi, open(dst, "wb") as fo:     # across backends: stream through
        shutil.copyfileobj(fi, fo)


def open(path: str, mode: str = "r") -> IO:  # pylint: disable=redefined-builtin
    return _call("open", path, mode)


def readfile(path: str) -> str:
    with open(path) as f:
        return f.read()


def makedirs(path: str) -> None:
    _call("makedirs", path)


def rmtree(path: str) -> None:
    _call("rmtree", path)
