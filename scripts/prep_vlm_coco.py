#!/usr/bin/env python
"""Turn a COCO-captions style annotation file (Karpathy split JSON or the official captions JSON) plus an image
directory into a HuggingFace ``Dataset`` on disk with ``image`` / ``text`` (/ ``prompt``) columns, the format the
image-text dataset of this framework reads.

    python scripts/prep_vlm_coco.py --annotations dataset_coco.json --images /data/coco --out /data/coco_hf --split train

Same role as the reference's scripts/prep_vlm_coco.py.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def iter_karpathy(ann: dict, split: str):
    for img in ann["images"]:
        if img.get("split") != split and not (split == "train" and img.get("split") == "restval"):
            continue
        rel = Path(img.get("filepath", "")) / img["filename"]
        for sent in img["sentences"]:
            yield str(rel), sent["raw"].strip()


def iter_official(ann: dict):
    names = {i["id"]: i["file_name"] for i in ann["images"]}
    for a in ann["annotations"]:
        yield names[a["image_id"]], a["caption"].strip()


def _build_split(datasets, ann_path: Path, root: Path, split: str, prompt: str, limit: int):
    ann = json.loads(ann_path.read_text())
    first = ann["images"][0] if ann.get("images") else {}
    pairs = iter_karpathy(ann, split) if "sentences" in first else iter_official(ann)
    rows = {"image": [], "text": [], "prompt": []}
    missing = 0
    for rel, text in pairs:
        path = root / rel
        if not path.exists():
            missing += 1
            continue
        rows["image"].append(str(path))
        rows["text"].append(text)
        rows["prompt"].append(prompt)
        if limit and len(rows["text"]) >= limit:
            break
    if not rows["text"]:
        return None, missing
    return datasets.Dataset.from_dict(rows).cast_column("image", datasets.Image()), missing


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    # --caption-json / --image-root / --num-samples / --all-splits are the reference's spellings
    ap.add_argument("--annotations", "--caption-json", dest="annotations", required=True)
    ap.add_argument("--images", "--image-root", dest="images", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--split", default="train")
    ap.add_argument("--prompt", default="")
    ap.add_argument("--max-samples", "--num-samples", dest="max_samples", type=int, default=0, help="per-split cap, 0 = all")
    ap.add_argument("--all-splits", action="store_true",
                    help="read coco_karpathy_{train,val,test}.json beside --annotations and save a DatasetDict")
    args = ap.parse_args(argv)
    try:
        import datasets
    except ImportError:
        print("the `datasets` package is required", file=sys.stderr)
        return 2
    root = Path(args.images)
    if args.all_splits:
        base = Path(args.annotations)
        folder = base if base.is_dir() else base.parent
        parts = {}
        for split in ("train", "val", "test"):
            path = folder / f"coco_karpathy_{split}.json"
            if not path.exists():
                continue
            ds, missing = _build_split(datasets, path, root, split, args.prompt, args.max_samples)
            if ds is not None:
                parts[split] = ds
                print(f"{split}: {len(ds)} samples ({missing} images missing)")
        if not parts:
            print("no coco_karpathy_{train,val,test}.json with usable pairs found", file=sys.stderr)
            return 1
        datasets.DatasetDict(parts).save_to_disk(args.out)
        print(f"wrote splits {sorted(parts)} to {args.out}")
        return 0
    ds, missing = _build_split(datasets, Path(args.annotations), root, args.split, args.prompt, args.max_samples)
    if ds is None:
        print("no (image, caption) pairs found", file=sys.stderr)
        return 1
    ds.save_to_disk(args.out)
    print(f"wrote {len(ds)} samples to {args.out} ({missing} images missing)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
