"""Image + text samples for vision-language training.

Every sample and every batch has a fixed shape (text padded to ``max_text_len``, images resized to one
square size), so data-parallel ranks always agree on tensor shapes.  Prompt tokens and padding carry the
label -100 and do not contribute to the loss.
Parity: kempnerforge/data/vlm_dataset.py:41-253 (``HuggingFaceVLMDataset``, ``VLMCollator``; prompt and
text are tokenised separately so the loss mask ends exactly at the prompt boundary).
"""

from __future__ import annotations

import os
from typing import Any

import numpy as np
import torch
from torch.utils.data import Dataset

from kempnerforge_b200.metrics.logger import get_logger

log = get_logger(__name__)

DEFAULT_IMAGE_MEAN = (0.5, 0.5, 0.5)
DEFAULT_IMAGE_STD = (0.5, 0.5, 0.5)
IGNORE_INDEX = -100


def image_to_tensor(img: Any, size: int, mean=DEFAULT_IMAGE_MEAN, std=DEFAULT_IMAGE_STD) -> torch.Tensor:
    """PIL image -> normalised float32 (3, size, size); grey / RGBA inputs are converted to RGB first."""
    from PIL import Image

    if not isinstance(img, Image.Image):
        raise TypeError(f"expected a PIL.Image, got {type(img).__name__} (decode raw bytes with PIL first)")
    rgb = img.convert("RGB").resize((size, size), Image.Resampling.BILINEAR)
    x = torch.from_numpy(np.asarray(rgb, dtype=np.float32) / 255.0).permute(2, 0, 1)
    m = torch.tensor(mean, dtype=torch.float32).view(3, 1, 1)
    s = torch.tensor(std, dtype=torch.float32).view(3, 1, 1)
    return ((x - m) / s).contiguous()


def pad_token_id(tokenizer: Any) -> int:
    for attr in ("pad_token_id", "eos_token_id"):
        v = getattr(tokenizer, attr, None)
        if v is not None:
            return int(v)
    return 0


def encode_text(tokenizer: Any, text: str, max_text_len: int, prompt: str | None = None):
    """(input_ids, labels), both (max_text_len,) int64, right padded.  ``prompt`` (if any) goes first and is
    excluded from the loss.  Prompt and text are tokenised on their own and concatenated as id lists:
    sub-word tokenisers may merge across the boundary otherwise and the mask would be off by a token."""
    ids: list[int] = []
    n_prompt = 0
    if prompt:
        ids = list(tokenizer(prompt, add_special_tokens=False)["input_ids"])
        n_prompt = min(len(ids), max_text_len)
    ids = (ids + list(tokenizer(text, add_special_tokens=False)["input_ids"]))[:max_text_len]
    input_ids = torch.full((max_text_len,), pad_token_id(tokenizer), dtype=torch.long)
    labels = torch.full((max_text_len,), IGNORE_INDEX, dtype=torch.long)
    if ids:
        t = torch.tensor(ids, dtype=torch.long)
        input_ids[: len(ids)] = t
        labels[n_prompt : len(ids)] = t[n_prompt:]
    return input_ids, labels


def _pad_text(samples: list[dict], pad_id: int, max_text_len: int):
    b = len(samples)
    input_ids = torch.full((b, max_text_len), pad_id, dtype=torch.long)
    labels = torch.full((b, max_text_len), IGNORE_INDEX, dtype=torch.long)
    for i, s in enumerate(samples):
        n = min(s["input_ids"].shape[0], max_text_len)
        input_ids[i, :n] = s["input_ids"][:n]
        labels[i, :n] = s["labels"][:n]
    return input_ids, labels


class HuggingFaceVLMDataset(Dataset):
    """Map-style image-caption dataset from the Hugging Face hub or from a ``save_to_disk`` directory."""

    def __init__(self, dataset_name: str, split: str, image_field: str, text_field: str, tokenizer_path: str,
                 max_text_len: int, prompt_field: str | None = None, image_size: int = 224,
                 image_mean=DEFAULT_IMAGE_MEAN, image_std=DEFAULT_IMAGE_STD, dataset_config: str | None = None,
                 *, rows: Any = None, tokenizer: Any = None) -> None:
        if rows is None:
            import datasets as hf

            if os.path.isdir(dataset_name):
                loaded = hf.load_from_disk(dataset_name)
                rows = loaded if isinstance(loaded, hf.Dataset) else loaded[split]
            else:
                rows = hf.load_dataset(dataset_name, dataset_config, split=split)
            if not isinstance(rows, hf.Dataset):
                raise TypeError(f"need a map-style datasets.Dataset, got {type(rows).__name__} (pass one split)")
        if tokenizer is None:
            from transformers import AutoTokenizer

            tokenizer = AutoTokenizer.from_pretrained(tokenizer_path)
        self.rows, self.tokenizer = rows, tokenizer
        self.image_field, self.text_field, self.prompt_field = image_field, text_field, prompt_field
        self.image_size, self.image_mean, self.image_std = image_size, tuple(image_mean), tuple(image_std)
        self.max_text_len = max_text_len
        log.info("HuggingFaceVLMDataset %s[%s]: %d samples, image %dpx, text %d tokens", dataset_name, split,
                 len(rows), image_size, max_text_len)

    def __len__(self) -> int:
        return len(self.rows)

    def __getitem__(self, idx: int) -> dict[str, torch.Tensor]:
        row = self.rows[idx]
        text = row[self.text_field]
        if not isinstance(text, str):
            raise TypeError(f"field {self.text_field!r} must hold str, got {type(text).__name__}")
        prompt = row[self.prompt_field] if self.prompt_field else None
        ids, labels = encode_text(self.tokenizer, text, self.max_text_len, prompt if isinstance(prompt, str) else None)
        pixels = image_to_tensor(row[self.image_field], self.image_size, self.image_mean, self.image_std)
        return {"pixel_values": pixels, "input_ids": ids, "labels": labels}


class VLMCollator:
    """Batch of fixed shape: pixel_values (B, 3, H, W), input_ids / labels (B, max_text_len) and
    image_positions (B,) (zeros: one image per sample, placed before the text)."""

    def __init__(self, pad_id: int, max_text_len: int) -> None:
        if max_text_len <= 0:
            raise ValueError("max_text_len must be positive")
        self.pad_id, self.max_text_len = pad_id, max_text_len

    def __call__(self, samples: list[dict[str, torch.Tensor]]) -> dict[str, torch.Tensor]:
        if not samples:
            raise ValueError("VLMCollator received an empty batch")
        input_ids, labels = _pad_text(samples, self.pad_id, self.max_text_len)
        return {"pixel_values": torch.stack([s["pixel_values"] for s in samples]), "input_ids": input_ids,
                "labels": labels, "image_positions": torch.zeros(len(samples), dtype=torch.long)}


_pil_to_tensor = image_to_tensor   # underscore spellings used by code written against the reference
_tokenize_and_mask = encode_text
