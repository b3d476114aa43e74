"""Data pipeline: datasets, samplers, stateful loader and the factory the trainer uses."""

from __future__ import annotations

import os

from kempnerforge_b200.data.dataloader import StatefulDataLoader
from kempnerforge_b200.data.dataset import (
    HuggingFaceDataset,
    MemoryMappedDataset,
    MixtureDataset,
    StreamingHuggingFaceDataset,
    compute_packed_output,
)
from kempnerforge_b200.data.sampler import DistributedSampler, MixtureSampler


def _eos_id(config) -> int | None:
    if not config.data.tokenizer_path:
        return None
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(config.data.tokenizer_path).eos_token_id


def _one_dataset(config, path: str = "", hf_name: str = "", hf_config: str = "", rank: int = 0, world: int = 1):
    dc, tc = config.data, config.train
    window = tc.seq_len + 1
    if path:
        eos = _eos_id(config) if dc.pack_sequences else None
        return MemoryMappedDataset(path, window, dc.file_pattern, dc.pack_sequences, eos)
    if dc.hf_streaming:
        return StreamingHuggingFaceDataset(hf_name, tc.seq_len, dc.tokenizer_path, hf_config or None,
                                           dc.hf_dataset_split, dc.hf_dataset_text_field, rank, world,
                                           dc.pack_sequences, seed=tc.effective_data_seed)
    return HuggingFaceDataset(hf_name, tc.seq_len, dc.tokenizer_path, hf_config or None, dc.hf_dataset_split,
                              dc.hf_dataset_text_field, dc.pack_sequences)


def build_train_dataloader(config, dp_rank: int = 0, dp_size: int = 1):
    """The training data source named by the config; synthetic uniform tokens when none is configured."""
    dc, tc = config.data, config.train
    seed = tc.effective_data_seed
    if dc.datasets:
        parts, names, weights = [], [], []
        for i, src in enumerate(dc.datasets):
            parts.append(_one_dataset(config, src.path, src.hf_name, src.hf_config, dp_rank, dp_size))
            names.append(src.name or os.path.basename(os.path.normpath(src.path)) or src.hf_name or f"dataset_{i}")
            weights.append(src.weight)
        ds = MixtureDataset(parts, names)
        sampler = MixtureSampler(ds.cumulative_sizes, weights, dp_size, dp_rank, True, seed, True, dc.mix_temperature)
    elif dc.dataset_path or dc.hf_dataset_name:
        ds = _one_dataset(config, dc.dataset_path, dc.hf_dataset_name or "", dc.hf_dataset_config or "", dp_rank, dp_size)
        sampler = None if dc.hf_streaming and not dc.dataset_path else DistributedSampler(len(ds), dp_size, dp_rank, True, seed, True)
    else:
        from kempnerforge_b200.training.trainer import SyntheticTokens

        return SyntheticTokens(config.model.vocab_size, tc.batch_size, tc.seq_len, seed, dp_rank, dc.pin_memory)
    return StatefulDataLoader(ds, tc.batch_size, sampler, dc.num_workers, dc.pin_memory, dc.prefetch_factor, True)


def build_vlm_dataloader(config, dp_rank: int = 0, dp_size: int = 1, *, dataset=None, tokenizer=None):
    """Image-text or video-caption batches of fixed shape for a vision-language run.

    ``[video]`` present -> the registered video dataset (clips -> frames + frame_mask); otherwise the
    Hugging Face image-text dataset named by ``data.hf_dataset_name``.  Synthetic data is not offered for
    VLM runs.  Parity: scripts/train.py:290-344 of the reference.
    """
    from kempnerforge_b200.data.vlm_dataset import HuggingFaceVLMDataset, VLMCollator, pad_token_id

    dc, tc, vlm = config.data, config.train, config.vlm
    if dataset is None:
        if config.is_video:
            from kempnerforge_b200.data.video_dataset import build_video_dataset

            extra = {"tokenizer": tokenizer} if tokenizer is not None else {}
            dataset = build_video_dataset(config.video, dc.tokenizer_path, vlm.max_text_len, **extra)
        else:
            if not (dc.hf_dataset_name and (dc.tokenizer_path or tokenizer is not None)):
                raise ValueError("VLM training requires data.hf_dataset_name and data.tokenizer_path")
            enc = config.vision_encoder
            dataset = HuggingFaceVLMDataset(
                dc.hf_dataset_name, dc.hf_dataset_split, dc.hf_dataset_image_field, dc.hf_dataset_text_field,
                dc.tokenizer_path, vlm.max_text_len, prompt_field=dc.hf_dataset_prompt_field or None,
                image_size=getattr(enc, "image_size", 224) or 224, dataset_config=dc.hf_dataset_config,
                tokenizer=tokenizer)
    tok = getattr(dataset, "tokenizer", tokenizer)
    pad = getattr(dataset, "pad_id", None)
    if pad is None:
        pad = pad_token_id(tok) if tok is not None else 0
    if config.is_video:
        from kempnerforge_b200.data.video_dataset import VideoCollator

        collate = VideoCollator(pad, vlm.max_text_len)
    else:
        collate = VLMCollator(pad, vlm.max_text_len)
    sampler = DistributedSampler(len(dataset), dp_size, dp_rank, True, tc.effective_data_seed, True)
    return StatefulDataLoader(dataset, tc.batch_size, sampler, dc.num_workers, dc.pin_memory, dc.prefetch_factor, True,
                              collate_fn=collate)


__all__ = [n for n in dir() if not n.startswith("_")]
