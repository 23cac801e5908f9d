"""Verified copies of checkpoints between a persistent store and a fast local device.

Long jobs keep their newest checkpoint on a fast device (local NVMe / a RAM disk) so that a restart after a failure does
not wait for the shared file system, and copy it to persistent storage in the background. The reference wires this to one
vendor's job platform (paddleformers/utils/pdc_sdk.py:64-600: upload / download through an agent binary, per-file hashes,
a checksum file per directory, ``pdc_backup_to_flash_device``, ``pdc_flash_do_check``; used at
paddleformers/trainer/trainer.py:1772-1776). This module provides the same operations on plain directories, so any mount
works:

* ``write_manifest(dir)`` / ``verify(dir)`` - per-file BLAKE2b digests and sizes in ``checksum.json``; ``verify`` names every
  missing, resized or corrupted file;
* ``mirror(src, dst)`` - copy a checkpoint directory file by file (several threads), verify the copy against the source
  manifest, and only then move it into place (``dst`` never holds a half-copied checkpoint);
* ``backup_to_fast_device`` / ``restore_latest`` - the two directions used around training: after a save, and before a
  resume (fast device first, persistent store as the fallback, the first candidate that verifies wins);
* ``MirrorCallback`` - runs the backup in a background thread after every checkpoint the trainer writes.
"""
from __future__ import annotations

import enum
import hashlib
import json
import os
import re
import shutil
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional, Tuple

from ..trainer.trainer_callback import TrainerCallback
from .log import logger

MANIFEST = "checksum.json"
_CKPT = re.compile(r"^checkpoint-(\d+)$")


class MirrorStatus(enum.Enum):
    """Outcome codes, in the spirit of the reference's ``PDCErrorCode``."""

    SUCCESS = 0
    SOURCE_MISSING = 1
    CHECKSUM_MISSING = 2
    CHECKSUM_MISMATCH = 3
    COPY_FAILED = 4
    NOTHING_TO_RESTORE = 5


def file_digest(path: str, chunk: int = 8 << 20) -> str:
    h = hashlib.blake2b(digest_size=32)
    with open(path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                break
            h.update(b)
    return h.hexdigest()


def _files(root: str) -> List[str]:
    out = []
    for d, _, names in os.walk(root):
        for n in names:
            rel = os.path.relpath(os.path.join(d, n), root)
            if rel != MANIFEST and not rel.endswith(".tmp"):
                out.append(rel)
    return sorted(out)


def write_manifest(root: str, workers: int = 8) -> Dict[str, Dict[str, object]]:
    files = _files(root)
    with ThreadPoolExecutor(max_workers=max(1, workers)) as ex:
        digests = list(ex.map(lambda r: file_digest(os.path.join(root, r)), files))
    manifest = {r: {"size": os.path.getsize(os.path.join(root, r)), "blake2b": dg} for r, dg in zip(files, digests)}
    tmp = os.path.join(root, MANIFEST + ".tmp")
    with open(tmp, "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    os.replace(tmp, os.path.join(root, MANIFEST))
    return manifest


def verify(root: str, manifest: Optional[Dict[str, Dict[str, object]]] = None, workers: int = 8) -> Tuple[MirrorStatus, List[str]]:
    """(status, problems): every file of the manifest must exist with its size and digest."""
    if not os.path.isdir(root):
        return MirrorStatus.SOURCE_MISSING, [root]
    if manifest is None:
        mf = os.path.join(root, MANIFEST)
        if not os.path.exists(mf):
            return MirrorStatus.CHECKSUM_MISSING, [mf]
        with open(mf) as f:
            manifest = json.load(f)

    def check(item):
        rel, meta = item
        p = os.path.join(root, rel)
        if not os.path.exists(p):
            return f"{rel}: missing"
        if os.path.getsize(p) != meta["size"]:
            return f"{rel}: size {os.path.getsize(p)} != {meta['size']}"
        if file_digest(p) != meta["blake2b"]:
            return f"{rel}: digest differs"
        return None

    with ThreadPoolExecutor(max_workers=max(1, workers)) as ex:
        problems = [p for p in ex.map(check, manifest.items()) if p]
    return (MirrorStatus.SUCCESS if not problems else MirrorStatus.CHECKSUM_MISMATCH), problems


def mirror(src: str, dst: str, workers: int = 8) -> MirrorStatus:
    """Copy ``src`` to ``dst`` and verify; ``dst`` appears only when the copy is complete and correct."""
    if not os.path.isdir(src):
        return MirrorStatus.SOURCE_MISSING
    mf = os.path.join(src, MANIFEST)
    if os.path.exists(mf):
        with open(mf) as f:
            manifest = json.load(f)
    else:
        manifest = write_manifest(src, workers)
    staging = dst.rstrip("/") + ".incoming"
    if os.path.exists(staging):
        shutil.rmtree(staging)
    os.makedirs(staging)

    def copy(rel):
        out = os.path.join(staging, rel)
        os.makedirs(os.path.dirname(out) or staging, exist_ok=True)
        shutil.copyfile(os.path.join(src, rel), out)

    try:
        with ThreadPoolExecutor(max_workers=max(1, workers)) as ex:
            list(ex.map(copy, list(manifest) + [MANIFEST]))
    except OSError as e:
        logger.warning(f"checkpoint mirror: copy {src} -> {dst} failed: {e}")
        shutil.rmtree(staging, ignore_errors=True)
        return MirrorStatus.COPY_FAILED
    status, problems = verify(staging, manifest, workers)
    if status is not MirrorStatus.SUCCESS:
        logger.warning(f"checkpoint mirror: {dst} failed verification: {problems[:3]}")
        failed = dst.rstrip("/") + ".failed"
        shutil.rmtree(failed, ignore_errors=True)
        os.replace(staging, failed)               # kept aside for inspection, like the reference's backup of failed dirs
        return status
    if os.path.exists(dst):
        shutil.rmtree(dst)
    os.replace(staging, dst)
    return MirrorStatus.SUCCESS


def list_checkpoints(root: str) -> List[Tuple[int, str]]:
    if not os.path.isdir(root):
        return []
    out = [(int(m.group(1)), os.path.join(root, n)) for n in os.listdir(root) for m in [_CKPT.match(n)] if m]
    return sorted(out)


def backup_to_fast_device(checkpoint_dir: str, fast_root: str, keep: int = 1, workers: int = 8) -> MirrorStatus:
    """Mirror one checkpoint onto the fast device and keep only the newest ``keep`` there."""
    name = os.path.basename(checkpoint_dir.rstrip("/"))
    os.makedirs(fast_root, exist_ok=True)
    status = mirror(checkpoint_dir, os.path.join(fast_root, name), workers)
    if status is MirrorStatus.SUCCESS and keep > 0:
        for _, old in list_checkpoints(fast_root)[:-keep]:
            shutil.rmtree(old, ignore_errors=True)
    return status


def restore_latest(roots: List[str], local_root: str, workers: int = 8) -> Tuple[MirrorStatus, Optional[str]]:
    """Newest checkpoint that verifies, searched over ``roots`` in the given order of preference at equal step (fast device
    first), copied under ``local_root`` unless it already lives there. Returns (status, local path)."""
    cands = []
    for prio, root in enumerate(roots):
        cands += [(-step, prio, path) for step, path in list_checkpoints(root)]
    for _, _, path in sorted(cands):
        status, problems = verify(path, workers=workers)
        if status is not MirrorStatus.SUCCESS:
            logger.warning(f"checkpoint mirror: skipping {path}: {status.name} {problems[:2]}")
            continue
        target = os.path.join(local_root, os.path.basename(path))
        if os.path.abspath(os.path.dirname(path)) == os.path.abspath(local_root):
            return MirrorStatus.SUCCESS, path
        st = mirror(path, target, workers)
        if st is MirrorStatus.SUCCESS:
            return st, target
    return MirrorStatus.NOTHING_TO_RESTORE, None


class MirrorCallback(TrainerCallback):
    """After every save, write the checkpoint's manifest and mirror it to ``fast_root`` in a background thread (rank 0 of
    the job; the per-rank files of the other ranks are on the shared output directory already)."""

    def __init__(self, fast_root: str, keep: int = 1):
        self.fast_root, self.keep = fast_root, keep
        self._thread: Optional[threading.Thread] = None
        self.last_status: Optional[MirrorStatus] = None

    def on_save(self, args, state, control, **kw):
        if not state.is_world_process_zero:
            return
        ckpt = os.path.join(args.output_dir, f"checkpoint-{state.global_step}")
        self.wait()

        def work():
            from ..trainer.checkpoint import wait_for_pending_saves

            wait_for_pending_saves()                       # asynchronous writers must have finished
            write_manifest(ckpt)
            self.last_status = backup_to_fast_device(ckpt, self.fast_root, self.keep)

        self._thread = threading.Thread(target=work, daemon=False)
        self._thread.start()

    def wait(self):
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    def on_train_end(self, args, state, control, **kw):
        self.wait()
