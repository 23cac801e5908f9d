"""Resolution of model files from a local directory or the local Hugging Face / ModelScope / AI Studio caches.

The reference resolves files across huggingface / aistudio / modelscope hubs (paddleformers/utils/download/,
selected by DOWNLOAD_SOURCE); this build works offline-first: a path, then the hub caches on disk, then (only if
``huggingface_hub`` is importable and the network allows) a hub download.
"""
from __future__ import annotations

import os
from typing import Optional


def _cache_roots():
    """Cache directories of the three hubs the reference can download from (DOWNLOAD_SOURCE = huggingface | modelscope |
    aistudio); the source named by DOWNLOAD_SOURCE is searched first."""
    hubs = {
        "huggingface": [os.path.join(os.environ[e], "hub") for e in ("PF_HOME", "HF_HOME") if os.environ.get(e)]
                       + [os.environ[e] for e in ("PF_HOME", "HF_HOME", "HF_HUB_CACHE") if os.environ.get(e)]
                       + [os.path.expanduser("~/.cache/huggingface/hub")],
        "modelscope": [os.path.join(os.environ.get("MODELSCOPE_CACHE", ""), "hub")] * bool(os.environ.get("MODELSCOPE_CACHE"))
                      + [os.path.expanduser("~/.cache/modelscope/hub"), os.path.expanduser("~/.cache/modelscope/hub/models")],
        "aistudio": [os.environ.get("AISTUDIO_CACHE_HOME", "")] * bool(os.environ.get("AISTUDIO_CACHE_HOME"))
                    + [os.path.expanduser("~/.cache/aistudio/hub"), os.path.expanduser("~/.cache/aistudio/models")],
    }
    first = os.environ.get("DOWNLOAD_SOURCE", "huggingface")
    order = [first] + [h for h in hubs if h != first]
    roots = []
    for h in order:
        roots.extend(hubs.get(h, []))
    return roots


def _download(repo: str, filename: str) -> Optional[str]:
    """One file from the hub named by DOWNLOAD_SOURCE, when its client library is importable and the network allows."""
    source = os.environ.get("DOWNLOAD_SOURCE", "huggingface")
    try:
        if source == "huggingface" and not os.environ.get("HF_HUB_OFFLINE"):
            from huggingface_hub import hf_hub_download

            return hf_hub_download(repo, filename)
        if source == "modelscope":
            from modelscope.hub.file_download import model_file_download

            return model_file_download(repo, filename)
        if source == "aistudio":
            from aistudio_sdk.hub import download as aistudio_download

            return aistudio_download(repo_id=repo, filename=filename)
    except Exception:  # noqa: BLE001  no client library, no network, or no such file: the caller reports it
        return None
    return None


def resolve_file_path(repo_or_dir: str, filename: str, required: bool = True) -> Optional[str]:
    if os.path.isdir(repo_or_dir):
        p = os.path.join(repo_or_dir, filename)
        if os.path.exists(p):
            return p
        if required:
            raise FileNotFoundError(f"{filename} not found in {repo_or_dir}")
        return None
    # hub cache layout: models--org--name/snapshots/<rev>/<file>
    key = "models--" + repo_or_dir.replace("/", "--")
    for root in _cache_roots():
        snap = os.path.join(root, key, "snapshots")
        if os.path.isdir(snap):
            for rev in sorted(os.listdir(snap), reverse=True):
                p = os.path.join(snap, rev, filename)
                if os.path.exists(p):
                    return p
        p = os.path.join(root, repo_or_dir, filename)
        if os.path.exists(p):
            return p
    got = _download(repo_or_dir, filename)
    if got is not None:
        return got
    if required:
        raise FileNotFoundError(f"cannot resolve {filename} for {repo_or_dir!r} (not a directory, not in a local cache)")
    return None


def resolve_dir(repo_or_dir: str) -> str:
    if os.path.isdir(repo_or_dir):
        return repo_or_dir
    p = resolve_file_path(repo_or_dir, "config.json")
    return os.path.dirname(p)
