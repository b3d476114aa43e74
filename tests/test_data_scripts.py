"""The data-preparation scripts: shard validation and the COCO-captions converter (host only)."""

from __future__ import annotations

import importlib.util
import json
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def _load(name):
    spec = importlib.util.spec_from_file_location(f"kf_script_{name}", ROOT / "scripts" / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_prepare_data_reports_shards_and_writes_metadata(tmp_path, capsys):
    pd = _load("prepare_data")
    np.save(tmp_path / "a.npy", np.arange(1000, dtype=np.uint16) % 200)
    np.save(tmp_path / "b.npy", np.arange(500, dtype=np.uint16) % 200)
    assert pd.main([str(tmp_path), "--seq-len", "99", "--vocab-size", "256", "--write-metadata"]) == 0
    out = capsys.readouterr().out
    assert "2 valid shard(s), 0 invalid; 1,500 tokens, 15 samples" in out
    import yaml

    meta = yaml.safe_load((tmp_path / "metadata.yaml").read_text())
    assert meta["num_shards"] == 2 and meta["total_tokens"] == 1500 and meta["shards"][0]["samples"] == 10


def test_prepare_data_flags_bad_shards(tmp_path, capsys):
    pd = _load("prepare_data")
    np.save(tmp_path / "ok.npy", np.arange(100, dtype=np.uint16))
    np.save(tmp_path / "float.npy", np.zeros(100, dtype=np.float32))
    np.save(tmp_path / "matrix.npy", np.zeros((10, 10), dtype=np.uint16))
    assert pd.main([str(tmp_path), "--seq-len", "9"]) == 2
    err = capsys.readouterr().err
    assert "INVALID float.npy" in err and "INVALID matrix.npy" in err
    assert pd.main([str(tmp_path), "--pattern", "ok.npy", "--seq-len", "9", "--vocab-size", "50"]) == 2   # id 99 >= 50
    assert pd.main([str(tmp_path), "--pattern", "*.bin"]) == 1                                           # nothing matches
    (np.arange(64, dtype=np.uint16)).tofile(tmp_path / "t.bin")
    info = pd.inspect_shard(tmp_path / "t.bin", 7, None)
    assert info["dtype"] == "uint32" and info["tokens"] == 32 and info["samples"] == 4


def test_coco_annotation_readers():
    coco = _load("prep_vlm_coco")
    karpathy = {"images": [
        {"split": "train", "filepath": "train2014", "filename": "a.jpg", "sentences": [{"raw": " a cat "}, {"raw": "cat again"}]},
        {"split": "restval", "filepath": "val2014", "filename": "b.jpg", "sentences": [{"raw": "a dog"}]},
        {"split": "test", "filepath": "val2014", "filename": "c.jpg", "sentences": [{"raw": "a bird"}]}]}
    train = list(coco.iter_karpathy(karpathy, "train"))
    assert train == [("train2014/a.jpg", "a cat"), ("train2014/a.jpg", "cat again"), ("val2014/b.jpg", "a dog")]
    assert list(coco.iter_karpathy(karpathy, "test")) == [("val2014/c.jpg", "a bird")]
    official = {"images": [{"id": 7, "file_name": "x.jpg"}], "annotations": [{"image_id": 7, "caption": "a tree \n"}]}
    assert list(coco.iter_official(official)) == [("x.jpg", "a tree")]


def test_coco_converter_writes_a_dataset_of_existing_images(tmp_path):
    pytest.importorskip("datasets")
    from PIL import Image

    coco = _load("prep_vlm_coco")
    img_dir = tmp_path / "images"
    img_dir.mkdir()
    Image.new("RGB", (8, 8), color=(10, 20, 30)).save(img_dir / "x.jpg")
    ann = {"images": [{"id": 1, "file_name": "x.jpg"}, {"id": 2, "file_name": "missing.jpg"}],
           "annotations": [{"image_id": 1, "caption": "a square"}, {"image_id": 2, "caption": "nothing"}]}
    (tmp_path / "ann.json").write_text(json.dumps(ann))
    rc = coco.main(["--annotations", str(tmp_path / "ann.json"), "--images", str(img_dir), "--out", str(tmp_path / "hf"),
                    "--prompt", "Describe:"])
    assert rc == 0 and (tmp_path / "hf").exists()
    import datasets

    ds = datasets.load_from_disk(str(tmp_path / "hf"))
    assert len(ds) == 1 and ds[0]["text"] == "a square" and ds[0]["prompt"] == "Describe:"


def test_coco_converter_reference_spellings_and_all_splits(tmp_path):
    pytest.importorskip("datasets")
    from PIL import Image

    coco = _load("prep_vlm_coco")
    img_dir = tmp_path / "images"
    img_dir.mkdir()
    Image.new("RGB", (8, 8)).save(img_dir / "x.jpg")
    for split in ("train", "val"):
        ann = {"images": [{"split": split, "filepath": "", "filename": "x.jpg", "sentences": [{"raw": f"{split} caption"}]}]}
        (tmp_path / f"coco_karpathy_{split}.json").write_text(json.dumps(ann))
    rc = coco.main(["--caption-json", str(tmp_path / "coco_karpathy_train.json"), "--image-root", str(img_dir),
                    "--out", str(tmp_path / "hf"), "--num-samples", "5", "--all-splits"])
    assert rc == 0
    import datasets

    dd = datasets.load_from_disk(str(tmp_path / "hf"))
    assert sorted(dd) == ["train", "val"] and dd["val"][0]["text"] == "val caption"


def test_script_command_lines_accept_the_reference_spellings(capsys):
    gen = _load("generate")
    with pytest.raises(SystemExit):
        gen.main(["--help"])
    text = capsys.readouterr().out
    for flag in ("--max_tokens", "--top_k", "--top_p", "--device", "--dtype"):
        assert flag in text, flag
    harness = _load("eval_harness")
    with pytest.raises(SystemExit):
        harness.main(["--help"])
    text = capsys.readouterr().out
    for flag in ("--config", "--hf-model", "--checkpoint", "--tasks", "--num-fewshot"):
        assert flag in text, flag
