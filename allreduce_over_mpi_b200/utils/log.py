"""Tiny leveled logger gated by ``FT_LOG_LEVEL`` (error|warn|info|debug); stderr only.

Stands in for the reference's glog usage (LOG(INFO/WARNING/FATAL), benchmark.cpp:60-62):
glog is not a dependency here, and FATAL conditions raise exceptions instead of aborting.
"""
from __future__ import annotations

import os
import sys
import time

_LEVELS = {"error": 0, "warn": 1, "info": 2, "debug": 3}
_level = _LEVELS.get(os.environ.get("FT_LOG_LEVEL", "warn").lower(), 1)


def set_level(name: str) -> None:
    global _level
    _level = _LEVELS[name]


def log(level: str, msg: str, rank: int | None = None) -> None:
    if _LEVELS[level] <= _level:
        tag = f"[flextree {level}{'' if rank is None else f' r{rank}'} {time.strftime('%H:%M:%S')}] "
        print(tag + msg, file=sys.stderr, flush=True)


def info(msg, rank=None): log("info", msg, rank)
def warn(msg, rank=None): log("warn", msg, rank)
def debug(msg, rank=None): log("debug", msg, rank)
def error(msg, rank=None): log("error", msg, rank)
