"""Video + caption samples: a clip becomes up to ``max_frames`` still frames plus a mask of real frames.

Shapes are fixed (frames zero-padded to ``max_frames``, text padded to ``max_text_len``).  A clip that cannot
be decoded keeps its shape, has an all-False ``frame_mask`` and all labels ignored, so it costs a step but
never breaks one.  ``decode_video_frames`` is looked up on this module at call time, so tests replace it.
Parity: kempnerforge/data/video_dataset.py:58-295 (``WebVidVideoDataset`` over CSV manifests and mp4 files,
``VideoCollator``, ``build_video_dataset`` through the ``video_dataset`` registry).
"""

from __future__ import annotations

import csv
import glob
import os
from typing import Any

import torch
from torch.utils.data import Dataset

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.data.video_io import decode_video_frames  # noqa: F401  (patched by tests)
from kempnerforge_b200.data.vlm_dataset import (DEFAULT_IMAGE_MEAN, DEFAULT_IMAGE_STD, IGNORE_INDEX, _pad_text,
                                                 encode_text, image_to_tensor, pad_token_id)
from kempnerforge_b200.metrics.logger import get_logger

log = get_logger(__name__)

# metadata lives under "val" while the clips live under "validation"
_MANIFEST_DIR = {"train": "train", "validation": "val"}
_CLIP_DIR = {"train": "train", "validation": "validation"}


class VideoDataset(Dataset):
    """Base class: samples are dicts with pixel_values (F, 3, H, W), frame_mask (F,), input_ids, labels."""


def read_manifest(csv_dir: str, max_samples: int = 0) -> tuple[list[str], list[str]]:
    """(video ids, captions) from the partition CSVs (columns ``videoid`` and ``name``), in sorted file order,
    stopping as soon as ``max_samples`` rows are collected.  Ids stay strings: their digits form the path."""
    files = sorted(glob.glob(os.path.join(csv_dir, "*.csv")))
    if not files:
        raise FileNotFoundError(f"no partition CSVs under {csv_dir!r}")
    ids: list[str] = []
    captions: list[str] = []
    for path in files:
        with open(path, newline="", encoding="utf-8") as f:
            for row in csv.DictReader(f):
                ids.append(str(row["videoid"]))
                captions.append(str(row["name"]))
                if max_samples and len(ids) >= max_samples:
                    return ids, captions
    return ids, captions


class WebVidVideoDataset(VideoDataset):
    """``<root>/raw/<dataset_name>/data/<split>/partitions/*.csv`` + ``<root>/raw/videos/<split>/...mp4``.
    Training clips are nested by id prefix (``12/1234/123456/1234567.mp4``); validation clips are flat."""

    def __init__(self, data_root: str, split: str, tokenizer_path: str, max_text_len: int, *, max_frames: int,
                 min_frames: int, fps: float, frame_size: int = 224, max_samples: int = 0, prompt: str = "",
                 dataset_name: str = "webvid-10M", sampling_policy: str = "uniform",
                 image_mean=DEFAULT_IMAGE_MEAN, image_std=DEFAULT_IMAGE_STD, tokenizer: Any = None) -> None:
        if split not in _CLIP_DIR:
            raise ValueError(f"split must be one of {tuple(_CLIP_DIR)} (got {split!r})")
        self._split = split
        self._video_dir = os.path.join(data_root, "raw", "videos", _CLIP_DIR[split])
        self._ids, self._caps = read_manifest(
            os.path.join(data_root, "raw", dataset_name, "data", _MANIFEST_DIR[split], "partitions"), max_samples)
        if tokenizer is None:
            from transformers import AutoTokenizer

            tokenizer = AutoTokenizer.from_pretrained(tokenizer_path)
        self._tokenizer = tokenizer
        self._pad_id = pad_token_id(tokenizer)
        self._max_text_len, self._prompt = max_text_len, prompt
        self._max_frames, self._min_frames, self._fps, self._frame_size = max_frames, min_frames, fps, frame_size
        self._sampling_policy = sampling_policy
        self._image_mean, self._image_std = tuple(image_mean), tuple(image_std)
        log.info("WebVidVideoDataset %s/%s[%s]: %d clips, <=%d frames at %s fps, %dpx", data_root, dataset_name, split,
                 len(self._ids), max_frames, fps, frame_size)

    # read-only public views of the fields (subclasses that skip __init__ set the underscored names directly)
    split = property(lambda self: self._split)
    clip_dir = property(lambda self: self._video_dir)
    ids = property(lambda self: self._ids)
    captions = property(lambda self: self._caps)
    tokenizer = property(lambda self: self._tokenizer)
    pad_id = property(lambda self: self._pad_id)
    max_text_len = property(lambda self: self._max_text_len)
    max_frames = property(lambda self: self._max_frames)

    def _video_path(self, videoid: str) -> str:
        return self.clip_path(videoid)

    def clip_path(self, videoid: str) -> str:
        s = str(videoid)
        if self._split == "train":
            return os.path.join(self._video_dir, s[:2], s[:4], s[:6], s + ".mp4")
        return os.path.join(self._video_dir, s + ".mp4")

    def __len__(self) -> int:
        return len(self._ids)

    def __getitem__(self, idx: int) -> dict[str, torch.Tensor]:
        import kempnerforge_b200.data.video_dataset as this_module

        path = self.clip_path(self._ids[idx])
        try:
            frames = this_module.decode_video_frames(path, fps=self._fps, min_frames=self._min_frames,
                                                     max_frames=self._max_frames, sampling_policy=self._sampling_policy)
        except Exception as e:  # noqa: BLE001  any decoding problem turns into a masked sample
            log.debug("could not decode %s: %s", path, e)
            frames = []
        pixels = torch.zeros(self._max_frames, 3, self._frame_size, self._frame_size)
        mask = torch.zeros(self._max_frames, dtype=torch.bool)
        for i, frame in enumerate(frames[: self._max_frames]):
            pixels[i] = image_to_tensor(frame, self._frame_size, self._image_mean, self._image_std)
            mask[i] = True
        ids, labels = encode_text(self._tokenizer, self._caps[idx], self._max_text_len, self._prompt or None)
        if not mask.any():
            labels = torch.full_like(labels, IGNORE_INDEX)
        return {"pixel_values": pixels, "frame_mask": mask, "input_ids": ids, "labels": labels}


class VideoCollator:
    """pixel_values (B, F, 3, H, W), frame_mask (B, F) bool, input_ids / labels (B, max_text_len)."""

    def __init__(self, pad_id: int, max_text_len: int) -> None:
        if max_text_len <= 0:
            raise ValueError("max_text_len must be positive")
        self.pad_id, self.max_text_len = pad_id, max_text_len

    def __call__(self, samples: list[dict[str, torch.Tensor]]) -> dict[str, torch.Tensor]:
        if not samples:
            raise ValueError("VideoCollator received an empty batch")
        input_ids, labels = _pad_text(samples, self.pad_id, self.max_text_len)
        return {"pixel_values": torch.stack([s["pixel_values"] for s in samples]),
                "frame_mask": torch.stack([s["frame_mask"] for s in samples]), "input_ids": input_ids, "labels": labels}


def _webvid_from_config(video_config: Any, tokenizer_path: str, max_text_len: int, **kw) -> WebVidVideoDataset:
    c = video_config
    return WebVidVideoDataset(c.data_root, c.split, tokenizer_path, max_text_len, max_frames=c.max_frames,
                              min_frames=c.min_frames, fps=c.fps, frame_size=c.frame_size, max_samples=c.max_samples,
                              prompt=c.prompt, dataset_name=c.dataset_name, sampling_policy=c.sampling_policy, **kw)


registry.register("video_dataset", "webvid", _webvid_from_config)


def build_video_dataset(video_config: Any, tokenizer_path: str, max_text_len: int, **kw) -> VideoDataset:
    """The dataset named by ``video_config.dataset_type`` (a ``video_dataset`` registry entry)."""
    return registry.get("video_dataset", video_config.dataset_type)(video_config, tokenizer_path, max_text_len, **kw)
