"""Image / video datasets, collators, frame sampling (CPU, no network, no video decoder)."""

import os

import pytest
import torch

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.config.vlm import VideoConfig
from kempnerforge_b200.data import video_dataset as vd
from kempnerforge_b200.data.video_io import clip_duration_seconds, pick_frames, sample_timestamps
from kempnerforge_b200.data.vlm_dataset import (HuggingFaceVLMDataset, VLMCollator, encode_text, image_to_tensor)


class ToyTokenizer:
    """Whitespace tokenizer: each distinct word gets the next id; id 0 pads."""

    pad_token_id = 0
    eos_token_id = 1

    def __init__(self):
        self.vocab: dict[str, int] = {}

    def __call__(self, text, add_special_tokens=False):
        return {"input_ids": [self.vocab.setdefault(w, len(self.vocab) + 2) for w in text.split()]}


def test_sample_timestamps_policy():
    assert sample_timestamps(0.0, 2.0, 4, 16) == [0.0]
    ts = sample_timestamps(10.0, 2.0, 4, 16)       # 20 wanted, capped at 16
    assert len(ts) == 16 and ts[0] == 0.0 and ts[-1] == pytest.approx(10.0)
    assert all(b > a for a, b in zip(ts, ts[1:]))
    assert len(sample_timestamps(0.5, 2.0, 4, 16)) == 4   # 1 wanted, raised to min_frames
    assert sample_timestamps(3.0, 0.1, 1, 8) == [0.0]
    assert registry.get("sampling_policy", "uniform") is sample_timestamps
    for bad in [(1.0, 0.0, 1, 2), (1.0, 1.0, 0, 2), (1.0, 1.0, 3, 2)]:
        with pytest.raises(ValueError):
            sample_timestamps(*bad)


def test_pick_frames_first_at_or_after_and_tail():
    frames = [(0.0, "a"), (0.4, "b"), (0.8, "c"), (1.2, "d")]
    assert pick_frames(frames, [0.0, 0.5, 1.0]) == ["a", "c", "d"]
    assert pick_frames(frames, [0.0, 5.0, 6.0]) == ["a", "d", "d"]   # past the end -> last frame
    assert pick_frames([], [0.0, 1.0]) == []
    seen = []

    def gen():
        for item in frames:
            seen.append(item[1])
            yield item

    pick_frames(gen(), [0.0, 0.3])
    assert seen == ["a", "b"]  # stops reading once every target is served


def test_clip_duration_fallbacks():
    class S:
        duration, time_base, frames, average_rate = None, None, 50, 25

    class C:
        duration = None

    assert clip_duration_seconds(S(), C()) == 2.0
    C.duration = 3_000_000
    assert clip_duration_seconds(S(), C()) == 3.0
    S.duration, S.time_base = 100, 0.05
    assert clip_duration_seconds(S(), C()) == 5.0


def test_encode_text_masks_prompt_and_padding():
    tok = ToyTokenizer()
    ids, labels = encode_text(tok, "a cat sits", 8, prompt="describe this")
    assert ids.tolist()[:5] == [2, 3, 4, 5, 6] and ids.tolist()[5:] == [0, 0, 0]
    assert labels.tolist() == [-100, -100, 4, 5, 6, -100, -100, -100]
    ids, labels = encode_text(tok, "a cat sits on the mat today again", 4)
    assert ids.shape == (4,) and (labels == ids).all()
    ids, labels = encode_text(tok, "x", 2, prompt="one two three")
    assert (labels == -100).all()


def test_image_to_tensor_and_vlm_dataset_and_collator():
    from PIL import Image

    img = Image.new("L", (10, 20), color=255)
    t = image_to_tensor(img, 8)
    assert t.shape == (3, 8, 8) and torch.allclose(t, torch.ones_like(t))
    with pytest.raises(TypeError):
        image_to_tensor(b"raw", 8)
    rows = [{"image": Image.new("RGB", (12, 12), color=(0, 0, 0)), "caption": "a b c", "q": "what"},
            {"image": img, "caption": "d e", "q": "which one"}]
    ds = HuggingFaceVLMDataset("toy", "train", "image", "caption", "", 6, prompt_field="q", image_size=8, rows=rows,
                               tokenizer=ToyTokenizer())
    assert len(ds) == 2
    s0 = ds[0]
    assert s0["pixel_values"].shape == (3, 8, 8) and s0["pixel_values"].max() == -1.0
    assert s0["labels"].tolist()[0] == -100 and (s0["labels"][1:4] >= 0).all()
    batch = VLMCollator(pad_id=0, max_text_len=6)([ds[0], ds[1]])
    assert batch["pixel_values"].shape == (2, 3, 8, 8) and batch["input_ids"].shape == (2, 6)
    assert batch["image_positions"].tolist() == [0, 0]
    with pytest.raises(ValueError):
        VLMCollator(0, 6)([])


def _write_webvid(root, n=3):
    part = os.path.join(root, "raw", "webvid-10M", "data", "train", "partitions")
    os.makedirs(part)
    with open(os.path.join(part, "0000.csv"), "w") as f:
        f.write("videoid,name,page_dir\n")
        for i in range(n):
            f.write(f"12345{i},clip number {i},x\n")
    return part


def test_webvid_dataset_with_stub_decoder(tmp_path, monkeypatch):
    from PIL import Image

    _write_webvid(str(tmp_path))
    calls = []

    def fake_decode(path, *, fps, min_frames, max_frames, sampling_policy="uniform"):
        calls.append(path)
        if path.endswith("123451.mp4"):
            raise OSError("corrupt file")
        return [Image.new("RGB", (16, 16), color=(255, 255, 255))] * 3

    monkeypatch.setattr(vd, "decode_video_frames", fake_decode)
    cfg = VideoConfig(data_root=str(tmp_path), max_frames=4, min_frames=1, frame_size=8, max_samples=2, prompt="say")
    ds = vd.build_video_dataset(cfg, "", 6, tokenizer=ToyTokenizer())
    assert len(ds) == 2
    good, bad = ds[0], ds[1]
    assert calls[0].endswith(os.path.join("raw", "videos", "train", "12", "1234", "123450", "123450.mp4"))
    assert good["pixel_values"].shape == (4, 3, 8, 8) and good["frame_mask"].tolist() == [True, True, True, False]
    assert good["pixel_values"][3].abs().sum() == 0 and good["labels"][0] == -100 and (good["labels"][1:4] >= 0).all()
    assert not bad["frame_mask"].any() and (bad["labels"] == -100).all()   # undecodable clip: no loss
    batch = vd.VideoCollator(ds.pad_id, 6)([good, bad])
    assert batch["pixel_values"].shape == (2, 4, 3, 8, 8) and batch["frame_mask"].shape == (2, 4)
    with pytest.raises(FileNotFoundError):
        vd.read_manifest(str(tmp_path / "nothing"))
