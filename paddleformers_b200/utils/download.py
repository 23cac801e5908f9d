"""Resolution of model files from a local directory or the local Hugging Face / ModelScope caches.

The reference resolves files across huggingface / aistudio / modelscope hubs (paddleformers/utils/download/,
selected by DOWNLOAD_SOURCE); this build works offline-first: a path, then the hub caches on disk, then (only if
``huggingface_hub`` is importable and the network allows) a hub download.
"""
from __future__ import annotations

import os
from typing import Optional


def _cache_roots():
    roots = []
    for env in ("PF_HOME", "HF_HOME"):
        if os.environ.get(env):
            roots.append(os.path.join(os.environ[env], "hub"))
            roots.append(os.environ[env])
    roots.append(os.path.expanduser("~/.cache/huggingface/hub"))
    roots.append(os.path.expanduser("~/.cache/modelscope/hub"))
    return roots


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
    if os.environ.get("DOWNLOAD_SOURCE", "huggingface") == "huggingface" and not os.environ.get("HF_HUB_OFFLINE"):
        try:
            from huggingface_hub import hf_hub_download

            return hf_hub_download(repo_or_dir, filename)
        except Exception:
            pass
    if required:
        raise FileNotFoundError(f"cannot resolve {filename} for {repo_or_dir!r} (not a directory, not in a local cache)")
    return None


def resolve_dir(repo_or_dir: str) -> str:
    if os.path.isdir(repo_or_dir):
        return repo_or_dir
    p = resolve_file_path(repo_or_dir, "config.json")
    return os.path.dirname(p)
