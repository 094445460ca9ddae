"""`HH:MM:SS.mmm LEVEL msg key=value…` on stderr, level from KERN_LOG (default info).
Reference: crates/kern-serve/src/logline.rs:22-48."""
from __future__ import annotations

import logging
import os
import sys
import time


class LineFormatter(logging.Formatter):
    def format(self, record: logging.LogRecord) -> str:
        t = time.localtime(record.created)
        ms = int((record.created % 1) * 1000)
        return f"{t.tm_hour:02d}:{t.tm_min:02d}:{t.tm_sec:02d}.{ms:03d} {record.levelname:5s} {record.getMessage()}"


def setup_logging(level: str | None = None) -> None:
    h = logging.StreamHandler(sys.stderr)
    h.setFormatter(LineFormatter())
    root = logging.getLogger()
    root.handlers[:] = [h]
    root.setLevel((level or os.environ.get("KERN_LOG", "info")).upper())
