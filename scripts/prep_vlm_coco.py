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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--annotations", required=True)
    ap.add_argument("--images", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--split", default="train")
    ap.add_argument("--prompt", default="")
    ap.add_argument("--max-samples", type=int, default=0)
    args = ap.parse_args(argv)
    try:
        import datasets
    except ImportError:
        print("the `datasets` package is required", file=sys.stderr)
        return 2
    ann = json.loads(Path(args.annotations).read_text())
    pairs = iter_karpathy(ann, args.split) if "sentences" in (ann["images"][0] if ann.get("images") else {}) else iter_official(ann)
    root = Path(args.images)
    rows = {"image": [], "text": [], "prompt": []}
    missing = 0
    for rel, text in pairs:
        path = root / rel
        if not path.exists():
            missing += 1
            continue
        rows["image"].append(str(path))
        rows["text"].append(text)
        rows["prompt"].append(args.prompt)
        if args.max_samples and len(rows["text"]) >= args.max_samples:
            break
    if not rows["text"]:
        print("no (image, caption) pairs found", file=sys.stderr)
        return 1
    ds = datasets.Dataset.from_dict(rows).cast_column("image", datasets.Image())
    ds.save_to_disk(args.out)
    print(f"wrote {len(ds)} samples to {args.out} ({missing} images missing)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
