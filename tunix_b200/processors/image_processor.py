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


# ------------------------------------------------------------------------------------------ Gemma 4
# Gemma 4 takes images at their own aspect ratio: an image is resized so that it holds at most a budget of
# patches (a multiple of the pooling cell in both directions), cut into patches with their (x, y) grid positions,
# and padded to the budget with position (-1, -1); the number of soft tokens an image yields therefore varies, and
# the prompt's image placeholder is expanded to that many soft-token slots between begin / end-of-image markers
# (tunix/processors/image_processor.py:181-576).
POSITIONS_PAD_VALUE = -1


def get_target_dimensions(height: int, width: int, patch_size: int = 16, max_patches: int = 10080,
                          pooling_kernel_size: int = 3) -> tuple:
    """Largest (height, width), multiples of `pooling_kernel_size * patch_size`, with the image's aspect ratio and at
    most `max_patches` patches; a side that would round to zero becomes one pooling cell."""
    import math
    cell = pooling_kernel_size * patch_size
    if height * width == 0:
        return cell, cell
    f = math.sqrt(max_patches * patch_size ** 2 / (height * width))
    th, tw = int(f * height // cell) * cell, int(f * width // cell) * cell
    longest = (max_patches // pooling_kernel_size ** 2) * cell
    if th == 0 and tw == 0:
        return cell, cell
    if th == 0:
        return cell, min(max(1, width // height) * cell, longest)
    if tw == 0:
        return min(max(1, height // width) * cell, longest), cell
    return th, tw


def _rgb_uint8(image) -> np.ndarray:
    from PIL import Image
    if isinstance(image, Image.Image):
        return np.asarray(image.convert("RGB"))
    image = np.asarray(image)
    if image.ndim == 2:
        return np.stack([image] * 3, -1)
    if image.shape[-1] == 4:
        return image[..., :3]
    if image.shape[-1] == 1:
        return np.concatenate([image] * 3, -1)
    return image


def preprocess_gemma4_image(image, patch_size: int = 16, max_soft_tokens: int = 1120, pooling_kernel_size: int = 3) -> np.ndarray:
    """RGB float32 in [0, 1] at the target size (bicubic resize; the model rescales to [-1, 1] itself)."""
    from PIL import Image
    img = _rgb_uint8(image)
    th, tw = get_target_dimensions(img.shape[0], img.shape[1], patch_size, max_soft_tokens * pooling_kernel_size ** 2,
                                   pooling_kernel_size)
    if (th, tw) != img.shape[:2]:
        img = np.asarray(Image.fromarray(img).resize((tw, th), resample=Image.Resampling.BICUBIC))
    return img.astype(np.float32) / 255.0


def num_soft_tokens_for_image(image: np.ndarray, patch_size: int = 16, pooling_kernel_size: int = 3) -> int:
    return (image.shape[0] // patch_size) * (image.shape[1] // patch_size) // pooling_kernel_size ** 2


def patchify(image: np.ndarray, patch_size: int) -> tuple:
    """[H, W, C] -> (patches [h*w, patch*patch*C] in row-major grid order, positions [h*w, 2] as (x, y))."""
    H, W, C = image.shape
    h, w = H // patch_size, W // patch_size
    p = image[:h * patch_size, :w * patch_size].reshape(h, patch_size, w, patch_size, C).transpose(0, 2, 1, 3, 4)
    gx, gy = np.meshgrid(np.arange(w), np.arange(h))
    return p.reshape(h * w, patch_size * patch_size * C), np.stack([gx, gy], -1).reshape(h * w, 2).astype(np.int32)


def patchify_and_pad(images: Sequence[np.ndarray], patch_size: int = 16, max_soft_tokens: int = 1120,
                     pooling_kernel_size: int = 3) -> tuple:
    """Stack variable-size images as [n, max_patches, dim] / [n, max_patches, 2]; padding patches are zero with
    position (-1, -1). Returns (patches, positions, real patches per image)."""
    budget = max_soft_tokens * pooling_kernel_size ** 2
    dim = 3 * patch_size ** 2
    patches = np.zeros((len(images), budget, dim), np.float32)
    positions = np.full((len(images), budget, 2), POSITIONS_PAD_VALUE, np.int32)
    real = []
    for i, im in enumerate(images):
        p, xy = patchify(im, patch_size)
        if len(p) > budget:
            raise ValueError(f"image {i} has {len(p)} patches, the budget is {budget}")
        patches[i, :len(p)], positions[i, :len(p)] = p, xy
        real.append(len(p))
    return patches, positions, real


def add_variable_extra_tokens_for_images(tokens: np.ndarray, *, soft_token_counts, placeholder_token: int = 258880,
                                         start_token: int = 255999, end_token: int = 258882, soft_token: int = -2,
                                         double_new_line_token: int = 108, pad_id: int = 0) -> np.ndarray:
    """Each image placeholder of a row becomes `\\n\\n <start> soft x count <end> \\n\\n`; rows are right-padded to
    the longest. `soft_token_counts` is one tuple per row (or one flat list used for every row); `soft_token` is
    the id written at the soft-token slots (the reference writes -2; pass the model's image token id to feed
    `Gemma4Multimodal` directly)."""
    rows = []
    for b in range(tokens.shape[0]):
        counts = soft_token_counts if (len(soft_token_counts) and isinstance(soft_token_counts[0], int)) else (
            soft_token_counts[b] if b < len(soft_token_counts) else ())
        out, k = [], 0
        for t in tokens[b].tolist():
            if t == placeholder_token and k < len(counts):
                out += [double_new_line_token, start_token] + [soft_token] * counts[k] + [end_token, double_new_line_token]
                k += 1
            else:
                out.append(t)
        rows.append(out)
    width = max(len(r) for r in rows)
    res = np.full((len(rows), width), pad_id, np.int32)
    for b, r in enumerate(rows):
        res[b, :len(r)] = r
    return res


@dataclasses.dataclass
class PreprocessedVisionInput:
    patches: np.ndarray            # [batch * images, max_patches, 3 * patch^2]
    positions_xy: np.ndarray       # [batch * images, max_patches, 2], (-1, -1) = padding
    soft_token_counts: tuple       # per batch row, per image
    images_per_row: int


def process_gemma4_inputs(images, tokens: list, *, patch_size: int = 16, max_soft_tokens: int = 280,
                          pooling_kernel_size: int = 3, pad_id: int = 0, placeholder_token: int = 258880,
                          soft_token: int | None = None, **marker_tokens) -> tuple:
    """images: one image, a list with one image per row, or a list of lists; tokens: one id array per row with one
    placeholder per image. Rows with fewer images than the batch maximum get all-padding images. Returns
    (PreprocessedVisionInput, token arrays with the placeholders expanded)."""
    if not isinstance(images, list):
        images = [[images]]
    elif images and not isinstance(images[0], list):
        images = [[im] for im in images]
    most = max((len(r) for r in images), default=0)
    budget = max_soft_tokens * pooling_kernel_size ** 2
    all_p, all_xy, counts = [], [], []
    for row in images:
        proc = [preprocess_gemma4_image(im, patch_size, max_soft_tokens, pooling_kernel_size) for im in row]
        counts.append(tuple(num_soft_tokens_for_image(p, patch_size, pooling_kernel_size) for p in proc))
        p, xy, _ = patchify_and_pad(proc, patch_size, max_soft_tokens, pooling_kernel_size)
        pad = most - len(row)
        if pad:
            p = np.concatenate([p, np.zeros((pad, budget, p.shape[-1]), np.float32)])
            xy = np.concatenate([xy, np.full((pad, budget, 2), POSITIONS_PAD_VALUE, np.int32)])
        all_p.append(p)
        all_xy.append(xy)
    vis = PreprocessedVisionInput(np.concatenate(all_p) if all_p else np.zeros((0, budget, 3 * patch_size ** 2), np.float32),
                                  np.concatenate(all_xy) if all_xy else np.zeros((0, budget, 2), np.int32), tuple(counts), most)
    width = max(len(t) for t in tokens)
    padded = np.stack([np.pad(np.asarray(t), (0, width - len(t)), constant_values=pad_id) for t in tokens])
    expanded = add_variable_extra_tokens_for_images(padded, soft_token_counts=tuple(counts), placeholder_token=placeholder_token,
                                                    soft_token=placeholder_token if soft_token is None else soft_token,
                                                    pad_id=pad_id, **marker_tokens)
    return vis, [np.asarray([t for t in row if t != pad_id], np.int32) for row in expanded.tolist()]
