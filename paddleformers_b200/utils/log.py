"""Console logger with TRAIN / EVAL levels and a background JSON-lines metrics dumper.

Same roles as paddleformers/utils/log.py:42 (Logger) and :138 (MetricsDumper) in the reference.
"""
from __future__ import annotations

import json
import logging
import os
import queue
import sys
import threading
import time

TRAIN, EVAL = 21, 22
logging.addLevelName(TRAIN, "TRAIN")
logging.addLevelName(EVAL, "EVAL")

_COLORS = {"DEBUG": "\033[35m", "INFO": "\033[32m", "TRAIN": "\033[36m", "EVAL": "\033[34m", "WARNING": "\033[33m",
           "ERROR": "\033[31m", "CRITICAL": "\033[31;1m"}


class _Formatter(logging.Formatter):
    def format(self, record):
        msg = super().format(record)
        if sys.stderr.isatty():
            return f"{_COLORS.get(record.levelname, '')}{msg}\033[0m"
        return msg


class Logger(logging.Logger):
    def train(self, msg, *a, **k):
        self.log(TRAIN, msg, *a, **k)

    def eval(self, msg, *a, **k):
        self.log(EVAL, msg, *a, **k)

    def warning_once(self, msg):
        seen = self.__dict__.setdefault("_seen", set())
        if msg not in seen:
            seen.add(msg)
            self.warning(msg)


def _make_logger() -> Logger:
    logging.setLoggerClass(Logger)
    lg = logging.getLogger("paddleformers_b200")
    logging.setLoggerClass(logging.Logger)
    if not lg.handlers:
        h = logging.StreamHandler()
        h.setFormatter(_Formatter("[%(asctime)s] [%(levelname)8s] %(filename)s:%(lineno)d - %(message)s"))
        lg.addHandler(h)
        lg.setLevel(os.environ.get("PFB_LOG_LEVEL", "INFO"))
        lg.propagate = False
    return lg


logger = _make_logger()


class MetricsDumper:
    """Appends one JSON line per logging step to ``<path>`` from a background thread so that slow file systems never
    stall the training loop."""

    def __init__(self, path: str):
        self.path = path
        os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
        self._q: "queue.Queue" = queue.Queue()
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def _run(self):
        with open(self.path, "a") as f:
            while True:
                item = self._q.get()
                if item is None:
                    return
                f.write(json.dumps(item, default=str) + "\n")
                f.flush()

    def append(self, metrics: dict):
        self._q.put(dict(metrics, time=time.time()))

    def close(self):
        self._q.put(None)
        self._t.join(timeout=10)
