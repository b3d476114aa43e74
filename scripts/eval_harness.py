#!/usr/bin/env python
"""Run lm-evaluation-harness tasks on a checkpoint.

    python scripts/eval_harness.py cfg.toml --checkpoint checkpoints/latest --tasks hellaswag,arc_easy [--limit 100]

The checkpoint is converted to HuggingFace format in a temporary directory (see convert_checkpoint.py) and handed to
``lm_eval.simple_evaluate(model="hf")``.  Same flow as the reference's scripts/eval_harness.py:98-133.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("config", nargs="?", default=None)
    ap.add_argument("--config", dest="config_opt", default=None, help="TOML config (the reference's spelling of the positional)")
    ap.add_argument("--checkpoint", default=None, help="DCP checkpoint directory (converted to HuggingFace format first)")
    ap.add_argument("--hf-model", default=None, help="already converted HuggingFace directory (skips the conversion)")
    ap.add_argument("--tasks", default="hellaswag,arc_easy,arc_challenge,winogrande,piqa,boolq")
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--batch-size", default="auto")
    ap.add_argument("--limit", type=float, default=None)
    ap.add_argument("--num-fewshot", type=int, default=None)
    ap.add_argument("--output", default=None)
    args, overrides = ap.parse_known_args(argv)
    args.config = args.config or args.config_opt
    if not args.hf_model and not (args.checkpoint and args.config):
        ap.error("give --hf-model, or --checkpoint together with a config")
    try:
        import lm_eval
    except ImportError:
        print("lm-evaluation-harness (lm_eval) is not installed", file=sys.stderr)
        return 2
    from convert_checkpoint import dcp_to_hf

    from kempnerforge_b200.config import load_config

    cfg = load_config(args.config, overrides) if args.config else None
    tokenizer = args.tokenizer or (cfg.data.tokenizer_path if cfg else None) or args.hf_model
    if not tokenizer:
        print("a tokenizer is required (--tokenizer or data.tokenizer_path)", file=sys.stderr)
        return 2
    export_dtype = cfg.checkpoint.export_dtype if cfg else "bfloat16"
    with tempfile.TemporaryDirectory(prefix="kf_hf_") as tmp:
        if args.hf_model:
            tmp = args.hf_model
        else:
            dcp_to_hf(os.path.realpath(args.checkpoint), tmp, cfg.model, export_dtype)
        results = lm_eval.simple_evaluate(
            model="hf", model_args=f"pretrained={tmp},tokenizer={tokenizer},dtype={export_dtype}",
            tasks=[t.strip() for t in args.tasks.split(",") if t.strip()], batch_size=args.batch_size,
            limit=args.limit, num_fewshot=args.num_fewshot)
    summary = results.get("results", {})
    print(json.dumps(summary, indent=2, default=str))
    if args.output:
        with open(args.output, "w") as fh:
            json.dump(summary, fh, indent=2, default=str)
    return 0


if __name__ == "__main__":
    sys.exit(main())
