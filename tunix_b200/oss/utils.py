"""Model download front-ends used by AutoModel (tunix/oss/utils.py:25-106).

This build runs without network access, so every front-end resolves to files that are already on disk: a local
directory, the Hugging Face cache, or a path given through the environment. They raise `FileNotFoundError`
with the searched locations instead of attempting a download.
"""
from __future__ import annotations

import os
from typing import Optional


def pathways_available() -> bool:
    return False


def _first_existing(cands) -> Optional[str]:
    for c in cands:
        if c and os.path.isdir(c):
            return c
    return None


def hf_pipeline(model_id: str, model_download_path: Optional[str] = None) -> str:
    """Directory holding the safetensors / config / tokenizer files of `model_id`."""
    hub = os.environ.get("HF_HOME", os.path.expanduser("~/.cache/huggingface"))
    snap_root = os.path.join(hub, "hub", "models--" + model_id.replace("/", "--"), "snapshots")
    snaps = sorted(os.listdir(snap_root)) if os.path.isdir(snap_root) else []
    cands = [model_id, os.path.join(model_download_path or "", model_id.split("/")[-1]), model_download_path,
             os.path.join(snap_root, snaps[-1]) if snaps else None]
    hit = _first_existing(cands)
    if hit is None:
        raise FileNotFoundError(f"{model_id}: no local copy found (looked in {[c for c in cands if c]}); "
                                "downloads are not available in this environment")
    return hit


def kaggle_pipeline(model_id: str, model_download_path: Optional[str] = None) -> str:
    root = os.environ.get("KAGGLEHUB_CACHE", os.path.expanduser("~/.cache/kagglehub"))
    cands = [os.path.join(model_download_path or "", model_id.replace("/", "_")), os.path.join(root, "models", model_id)]
    hit = _first_existing(cands)
    if hit is None:
        raise FileNotFoundError(f"{model_id}: no local Kaggle copy found (looked in {cands})")
    return hit


def load_file_from_gcs(file_dir: str, target_dir: Optional[str] = None) -> str:
    if file_dir.startswith("gs://"):
        raise FileNotFoundError(f"{file_dir}: object storage is not reachable from this environment; copy the files locally")
    return file_dir
