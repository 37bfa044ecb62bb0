"""Module-aware error context (reference: axlearn/common/traceback_util.py:72-401).

A failure deep inside a model says little without the path of the module that was running: the
Python traceback shows ``layers.py`` lines, not *which* of 32 identical layers.  Every wrapped
module call therefore attaches one line -- module path, class and method -- to an exception that
passes through it (PEP 678 notes, so the line is printed with the normal traceback and the
exception's type and arguments are untouched).  ``annotate_stack`` does the same for plain
functions with arbitrary key / value context, ``no_stack_summary`` switches the mechanism off for
one function, and ``AXB200_STACK_SUMMARY=0`` for the process.
"""

from __future__ import annotations

import functools
import os
from typing import Any, Callable, Optional

_NOTE_PREFIX = "  in module "
_ANNOTATION_PREFIX = "  with "
_enabled: Optional[bool] = None


def is_stack_summary_enabled() -> bool:
    global _enabled
    if _enabled is None:
        _enabled = os.environ.get("AXB200_STACK_SUMMARY", "1") not in ("0", "false", "False")
    return _enabled


def set_stack_summary_enabled(flag: Optional[bool]) -> None:
    """``None`` re-reads the environment on the next query."""
    global _enabled
    _enabled = flag


def add_module_note(exc: BaseException, *, path: str, cls: str, method: str) -> None:
    """Records that ``exc`` passed through ``path`` (once per module call site)."""
    if not is_stack_summary_enabled() or getattr(exc, "__axb_no_summary__", False):
        return
    note = f"{_NOTE_PREFIX}{path} [{cls}.{method}]"
    notes = getattr(exc, "__notes__", None) or []
    if not notes or notes[-1] != note:
        exc.add_note(note)


def module_stack(exc: BaseException) -> list[str]:
    """Module paths recorded on ``exc``, innermost first."""
    out = []
    for note in getattr(exc, "__notes__", None) or []:
        if note.startswith(_NOTE_PREFIX):
            out.append(note[len(_NOTE_PREFIX):].split(" [", 1)[0])
    return out


def annotations(exc: BaseException) -> list[dict[str, str]]:
    """Key / value context recorded by ``annotate_stack`` frames, innermost first."""
    out = []
    for note in getattr(exc, "__notes__", None) or []:
        if note.startswith(_ANNOTATION_PREFIX):
            out.append(dict(item.split("=", 1) for item in note[len(_ANNOTATION_PREFIX):].split(", ")))
    return out


def annotate_stack(**aux: Any) -> Callable[[Callable], Callable]:
    """Decorator: exceptions leaving the function carry ``key=value`` context, e.g.
    ``@annotate_stack(stage="restore", step=step)``."""

    def decorator(fn: Callable) -> Callable:
        @functools.wraps(fn)
        def stack_annotation_wrapper(*args, **kwargs):
            try:
                return fn(*args, **kwargs)
            except BaseException as e:  # pylint: disable=broad-except
                if is_stack_summary_enabled() and not getattr(e, "__axb_no_summary__", False):
                    e.add_note(_ANNOTATION_PREFIX + ", ".join(f"{k}={v}" for k, v in aux.items()))
                raise

        return stack_annotation_wrapper

    return decorator


def no_stack_summary(fn: Callable) -> Callable:
    """Decorator: exceptions raised inside ``fn`` are never annotated (for control-flow
    exceptions such as an iterator's end, where the notes would only cost time)."""

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        try:
            return fn(*args, **kwargs)
        except BaseException as e:  # pylint: disable=broad-except
            try:
                e.__axb_no_summary__ = True
            except AttributeError:
                pass
            raise

    return wrapper


def wrap(fn: Callable, *, path: Callable[[], str], cls: str) -> Callable:
    """``fn`` with the module note attached to whatever it raises."""

    @functools.wraps(fn)
    def in_context_exception_wrapper(*args, **kwargs):
        try:
            return fn(*args, **kwargs)
        except BaseException as e:  # pylint: disable=broad-except
            add_module_note(e, path=path(), cls=cls, method=fn.__name__)
            raise

    return in_context_exception_wrapper
