"""Host-side image preprocessing for vision-language models (tunix/processors/image_processor.py:23-157).

Per image: bilinear resize to (image_height, image_width) with PIL, `(x - mean) / std`, clip to [-1, 1]. A batch
entry may hold any number of images; entries are padded with all-zero images to the batch maximum so the
vision tower sees a rectangular `[batch, images, H, W, C]` array. `to_pinned()` lands the result in pinned
host memory for an asynchronous copy to the device.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Sequence

import numpy as np


@dataclasses.dataclass
class ImageConfig:
    image_height: int = 896
    image_width: int = 896
    image_channels: int = 3
    image_mean: Sequence[float] = (127.5, 127.5, 127.5)
    image_std: Sequence[float] = (127.5, 127.5, 127.5)


class ImageProcessor:
    def __init__(self, config: Any = None):
        self.config = config or ImageConfig()
        c = self.config
        self._h, self._w, self._c = c.image_height, c.image_width, c.image_channels
        self._mean = np.asarray(c.image_mean, np.float32)
        self._std = np.asarray(c.image_std, np.float32)

    def _blank(self) -> np.ndarray:
        return np.zeros((self._h, self._w, self._c), np.float32)

    def preprocess_image(self, image) -> np.ndarray:
        if image is None:
            return self._blank()
        from PIL import Image
        if isinstance(image, str):
            image = Image.open(image)
        elif isinstance(image, np.ndarray):
            image = Image.fromarray(image)
        if self._c == 3 and image.mode != "RGB":
            image = image.convert("RGB")
        image = image.resize((self._w, self._h), resample=Image.Resampling.BILINEAR)   # PIL takes width first
        arr = np.asarray(image, np.float32)
        if arr.ndim == 2:
            arr = arr[..., None]
        return np.clip((arr - self._mean) / self._std, -1.0, 1.0).astype(np.float32)

    def __call__(self, images) -> list:
        if not isinstance(images, list):
            images = [[images]]
        most = max([len(b) if isinstance(b, list) else (0 if b is None else 1) for b in images] + [0])
        out = []
        for entry in images:
            items = [] if entry is None else (entry if isinstance(entry, list) else [entry])
            row = [self.preprocess_image(im) for im in items]
            row += [self._blank() for _ in range(most - len(items))]
            out.append(row)
        return out

    def to_pinned(self, images):
        """[batch, images, H, W, C] float32 tensor in pinned host memory (plain memory without CUDA)."""
        import torch
        arr = np.asarray(self(images), np.float32)
        t = torch.from_numpy(arr)
        return t.pin_memory() if torch.cuda.is_available() else t
