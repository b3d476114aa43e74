#!/usr/bin/env python
"""Validate (and describe) a directory of pre-tokenised shards.

    python scripts/prepare_data.py /data/tokens --pattern "*.npy" --seq-len 4096 [--vocab-size 128256] [--write-metadata]

Checks that every shard opens as a memory map, reports dtype / token counts / samples per shard at the given
sequence length, optionally checks token ids against the vocabulary size, and can write a ``metadata.yaml``
summary next to the shards.  Same purpose as the reference's scripts/prepare_data.py:28-122.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np


def inspect_shard(path: Path, seq_len: int, vocab_size: int | None, sample: int = 1_000_000) -> dict:
    if path.suffix == ".bin":
        size = path.stat().st_size
        dtype = np.uint32 if size % 4 == 0 else np.uint16
        arr = np.memmap(str(path), dtype=dtype, mode="r")
    else:
        arr = np.load(str(path), mmap_mode="r")
    if arr.ndim != 1:
        raise ValueError(f"{path.name}: expected a 1-D token array, got shape {arr.shape}")
    if not np.issubdtype(arr.dtype, np.integer):
        raise ValueError(f"{path.name}: tokens must be integers, got {arr.dtype}")
    info = {"file": path.name, "dtype": str(arr.dtype), "tokens": int(arr.shape[0]),
            "samples": int(arr.shape[0] // (seq_len + 1))}
    if vocab_size is not None:
        head = np.asarray(arr[:sample])
        top = int(head.max()) if head.size else 0
        if top >= vocab_size:
            raise ValueError(f"{path.name}: token id {top} >= vocab_size {vocab_size}")
        info["max_token_id_sampled"] = top
    return info


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("data_dir")
    ap.add_argument("--pattern", default="*.npy")
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--vocab-size", type=int, default=None)
    ap.add_argument("--write-metadata", action="store_true")
    args = ap.parse_args(argv)
    files = sorted(Path(args.data_dir).glob(args.pattern))
    if not files:
        print(f"no files match {args.pattern!r} in {args.data_dir}", file=sys.stderr)
        return 1
    rows, bad = [], 0
    for f in files:
        try:
            rows.append(inspect_shard(f, args.seq_len, args.vocab_size))
        except Exception as exc:
            bad += 1
            print(f"INVALID {f.name}: {exc}", file=sys.stderr)
    total_tokens = sum(r["tokens"] for r in rows)
    total_samples = sum(r["samples"] for r in rows)
    for r in rows:
        print(f"{r['file']:40s} {r['dtype']:8s} tokens={r['tokens']:>14,} samples={r['samples']:>10,}")
    print(f"{len(rows)} valid shard(s), {bad} invalid; {total_tokens:,} tokens, {total_samples:,} samples "
          f"of {args.seq_len} (+1) tokens")
    if args.write_metadata and rows:
        import yaml

        meta = {"tokenized": True, "file_pattern": args.pattern, "dtype": rows[0]["dtype"],
                "num_shards": len(rows), "total_tokens": total_tokens, "shards": rows}
        (Path(args.data_dir) / "metadata.yaml").write_text(yaml.safe_dump(meta, sort_keys=False))
    return 0 if bad == 0 else 2


if __name__ == "__main__":
    sys.exit(main())
