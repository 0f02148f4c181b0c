"""Rank-aware logging.

`get_logger(__name__)` returns a `TurboLogger` whose `*_rank0` helpers only emit on the first
process and whose `*_rank0_once` helpers additionally de-duplicate by message.  A tqdm-safe
stream handler keeps progress bars intact.  Mirrors the behaviour of the reference logger
(logging.py:81-167 in the reference) with its own implementation.
"""
from __future__ import annotations

import logging
import os
import sys

_FORMAT = "[%(levelname)s|%(asctime)s] %(name)s:%(lineno)d >> %(message)s"
_configured = False


def _rank() -> int:
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return dist.get_rank()
    except Exception:
        pass
    return int(os.environ.get("RANK", "0"))


class TqdmStreamHandler(logging.StreamHandler):
    """Writes through `tqdm.write` when tqdm is importable so that bars are not broken."""

    def emit(self, record):
        try:
            msg = self.format(record)
            try:
                from tqdm import tqdm

                tqdm.write(msg, file=self.stream)
            except Exception:
                self.stream.write(msg + "\n")
            self.flush()
        except Exception:
            self.handleError(record)


class TurboLogger(logging.Logger):
    _seen: set[str] = set()

    def _r0(self, level, msg, *args, once=False, **kw):
        if _rank() != 0:
            return
        if once:
            key = f"{level}:{msg}"
            if key in TurboLogger._seen:
                return
            TurboLogger._seen.add(key)
        kw.setdefault("stacklevel", 3)
        self.log(level, msg, *args, **kw)

    def info_rank0(self, msg, *a, **k):
        self._r0(logging.INFO, msg, *a, **k)

    def warning_rank0(self, msg, *a, **k):
        self._r0(logging.WARNING, msg, *a, **k)

    def debug_rank0(self, msg, *a, **k):
        self._r0(logging.DEBUG, msg, *a, **k)

    def error_rank0(self, msg, *a, **k):
        self._r0(logging.ERROR, msg, *a, **k)

    def info_rank0_once(self, msg, *a, **k):
        self._r0(logging.INFO, msg, *a, once=True, **k)

    def warning_rank0_once(self, msg, *a, **k):
        self._r0(logging.WARNING, msg, *a, once=True, **k)


def logging_configure(level: str | int | None = None) -> None:
    """Install the package handler once; `level` may be a name (`info`) or a logging constant."""
    global _configured
    root = logging.getLogger("torchturbo_b200")
    if not _configured:
        h = TqdmStreamHandler(sys.stdout)
        h.setFormatter(logging.Formatter(_FORMAT, datefmt="%Y-%m-%d %H:%M:%S"))
        root.addHandler(h)
        root.propagate = False
        _configured = True
    if level is None:
        level = os.environ.get("TORCH_TURBO_LOG_LEVEL", "info")
    if isinstance(level, str):
        level = getattr(logging, level.upper(), logging.INFO)
    root.setLevel(level)


def get_logger(name: str = "torchturbo_b200") -> TurboLogger:
    prev = logging.getLoggerClass()
    logging.setLoggerClass(TurboLogger)
    try:
        if not name.startswith("torchturbo_b200"):
            name = "torchturbo_b200." + name
        logger = logging.getLogger(name)
    finally:
        logging.setLoggerClass(prev)
    if not _configured:
        logging_configure()
    return logger  # type: ignore[return-value]
