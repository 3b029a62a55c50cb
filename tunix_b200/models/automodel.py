"""AutoModel: resolve a model id to a family / preset and build it (tunix/models/automodel.py:384-654).

Sources: a local directory with safetensors (`model_path`), or random initialisation (`ModelSource.RANDOM`,
what benchmarks and tests use). Remote hubs (HF, Kaggle, GCS) need network access; they resolve to
`snapshot_download` style helpers only when the corresponding package and connectivity exist."""
from __future__ import annotations

import enum
import os
from typing import Optional

import torch

from . import naming
from .config import ModelConfig, get_config
from .safetensors_loader import load_safetensors_into
from .transformer import Transformer, create_model


class ModelSource(enum.Enum):
    HUGGINGFACE = "huggingface"
    KAGGLE = "kaggle"
    GCS = "gcs"
    INTERNAL = "internal"
    LOCAL = "local"
    RANDOM = "random"


def download_model(model_id: str, source: ModelSource, download_path: Optional[str] = None) -> str:
    if source == ModelSource.HUGGINGFACE:
        from huggingface_hub import snapshot_download
        return snapshot_download(repo_id=model_id, local_dir=download_path)
    if source == ModelSource.KAGGLE:
        import kagglehub
        return kagglehub.model_download(model_id)
    raise ValueError(f"model source {source} cannot be downloaded; pass model_path=")


class AutoModel:
    @staticmethod
    def from_pretrained(model_id: str, mesh=None, *, model_source: ModelSource = ModelSource.LOCAL,
                        model_path: Optional[str] = None, model_download_path: Optional[str] = None,
                        device=None, dtype: Optional[torch.dtype] = None, load_dtype: Optional[torch.dtype] = None,
                        remat_config: Optional[str] = None, use_flash_attention: Optional[bool] = None,
                        seed: int = 0, **config_overrides):
        """Returns (model, model_path)."""
        try:
            cfg: ModelConfig = naming.config_for(model_id)
        except (KeyError, ValueError):
            # no preset of that name: a checkpoint directory describes itself through its config.json
            path = model_path or (model_id if os.path.isdir(model_id) else None)
            if path is None or not os.path.exists(os.path.join(path, "config.json")):
                raise
            from .hf_config import config_from_hf
            cfg = config_from_hf(path)
            model_path = path
        over = dict(config_overrides)
        if dtype is not None:
            over["dtype"] = dtype
        if remat_config is not None:
            over["remat_config"] = remat_config
        if use_flash_attention is not None:
            over["use_flash_attention"] = use_flash_attention
        if over:
            cfg = cfg.replace(**over)
        if isinstance(model_source, str):
            model_source = ModelSource(model_source)
        if model_source == ModelSource.RANDOM:
            return create_model(cfg, device=device, seed=seed), None
        if model_path is None:
            model_path = download_model(model_id, model_source, model_download_path)
        if not os.path.exists(model_path):
            raise FileNotFoundError(model_path)
        model = Transformer(cfg, device=device)
        load_safetensors_into(model, model_path, dtype=load_dtype)
        return model, model_path
