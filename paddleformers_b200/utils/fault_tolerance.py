"""Failure detection and restart-based recovery, all on the host.

* error strings / codes that an outer job platform can grep, like the reference's "recall error" codes
  (paddleformers/utils/fault_tolerance.py:16-28, paddleformers/trainer/trainer.py:2966-2972);
* a heartbeat watchdog over the rendezvous key-value store: every rank publishes a timestamp between steps, any rank
  can ask which peers have gone silent *before* it launches its next collective, so a dead rank is reported as a Python
  exception on the survivors instead of as a hang inside a kernel;
* ``run_with_restarts``: the launcher-side loop that restarts a failed job from the newest complete checkpoint.

Nothing here makes a GPU fault, trap or hang; device-side waits are bounded inside the kernels themselves and report
through the status word (``ops.functional.check_kernel_status``).
"""
from __future__ import annotations

import os
import subprocess
import sys
import threading
import time
from typing import Callable, Dict, List, Optional

PDC_DOWNLOAD_ERROR = "PaddleRecall error(105): checkpoint download failed"
LOSS_NAN_ERROR = "PaddleRecall error(106): LOSS_NAN_ERROR"
LOSS_INF_ERROR = "PaddleRecall error(107): LOSS_INF_ERROR"
RANK_LOST_ERROR = "PaddleRecall error(108): RANK_LOST_ERROR"


def is_ft_env() -> bool:
    return bool(os.environ.get("PFB_FT_ENV") or os.environ.get("PDC_LONGJOB_ID"))


class RankLostError(RuntimeError):
    pass


class HeartbeatMonitor:
    """Heartbeats through a ``torch.distributed`` store (TCPStore / FileStore / HashStore)."""

    def __init__(self, store, rank: int, world_size: int, timeout_s: float = 30.0, prefix: str = "hb"):
        self.store, self.rank, self.world, self.timeout, self.prefix = store, rank, world_size, timeout_s, prefix
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def beat(self, step: int = 0) -> None:
        self.store.set(f"{self.prefix}/{self.rank}", f"{time.time():.3f}:{step}")

    def start_background(self, interval_s: float = 1.0) -> None:
        def loop():
            while not self._stop.wait(interval_s):
                try:
                    self.beat()
                except Exception:  # noqa: BLE001 - the store may be gone during shutdown
                    return
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    def silent_ranks(self) -> List[int]:
        now = time.time()
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if hasattr(self.store, "check") and not self.store.check([f"{self.prefix}/{r}"]):
                    out.append(r)
                    continue
                ts = float(self.store.get(f"{self.prefix}/{r}").decode().split(":")[0])
            except Exception:  # noqa: BLE001
                out.append(r)
                continue
            if now - ts > self.timeout:
                out.append(r)
        return out

    def check(self) -> None:
        """Raise before the next collective if a peer stopped publishing heartbeats."""
        lost = self.silent_ranks()
        if lost:
            raise RankLostError(f"{RANK_LOST_ERROR}: no heartbeat from ranks {lost} for more than {self.timeout}s")


def run_with_restarts(cmd: List[str], output_dir: str, max_restarts: int = 3, env: Optional[Dict[str, str]] = None,
                      on_restart: Optional[Callable[[int, int], None]] = None) -> int:
    """Run ``cmd``; when it exits non-zero, kill its process group and run it again (the training script resumes from
    ``get_last_checkpoint(output_dir)``), up to ``max_restarts`` times. Returns the last exit code."""
    attempt = 0
    while True:
        proc = subprocess.Popen(cmd, env=dict(os.environ, **(env or {}), PFB_RESTART_COUNT=str(attempt)), start_new_session=True)
        rc = proc.wait()
        if rc == 0 or attempt >= max_restarts:
            return rc
        try:
            os.killpg(proc.pid, 15)
        except ProcessLookupError:
            pass
        attempt += 1
        if on_restart is not None:
            on_restart(attempt, rc)
