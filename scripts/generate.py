#!/usr/bin/env python
"""Text generation from a checkpoint on one device (no process group needed).

    python scripts/generate.py cfg.toml --checkpoint checkpoints/latest --prompt "Once upon" --max-new-tokens 64
    python scripts/generate.py cfg.toml --checkpoint ... --interactive

Same contract as the reference's scripts/generate.py:42-151 (DCP ``{"model": ...}`` load, prompt or REPL,
temperature / top-k / top-p sampling).  Without a tokenizer path the prompt is read as space-separated token ids.
"""

from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed.checkpoint as dcp  # noqa: E402

from kempnerforge_b200.config import load_config  # noqa: E402
from kempnerforge_b200.models import Transformer  # noqa: E402
from kempnerforge_b200.models.generate import generate  # noqa: E402


def load_model(cfg, checkpoint: str | None, device: torch.device) -> Transformer:
    with torch.device(device):
        model = Transformer(cfg.model)
    model = model.to(dtype=cfg.train.param_dtype if device.type == "cuda" else torch.float32)
    if checkpoint:
        path = os.path.realpath(checkpoint)
        state = {"model": model.state_dict()}
        dcp.load(state, checkpoint_id=path)
        model.load_state_dict(state["model"])
    return model.eval()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("config")
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--prompt", default=None)
    # spellings with underscores are the reference's command line (scripts/generate.py:88-147)
    ap.add_argument("--max-new-tokens", "--max_tokens", dest="max_new_tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", "--top_k", dest="top_k", type=int, default=0)
    ap.add_argument("--top-p", "--top_p", dest="top_p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--interactive", action="store_true")
    ap.add_argument("--device", default=None, help="default: cuda when available")
    ap.add_argument("--dtype", default=None, choices=["float32", "bfloat16", "float16"])
    args, overrides = ap.parse_known_args(argv)
    cfg = load_config(args.config, overrides)
    device = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    model = load_model(cfg, args.checkpoint, device)
    if args.dtype:
        model = model.to(getattr(torch, args.dtype))
    tok = None
    if cfg.data.tokenizer_path:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(cfg.data.tokenizer_path)
    gen = torch.Generator(device="cpu").manual_seed(args.seed)

    def run(prompt: str) -> str:
        ids = tok.encode(prompt) if tok else [int(t) for t in prompt.split()]
        x = torch.tensor([ids], device=device)
        room = cfg.model.max_seq_len - len(ids)
        if room <= 0:
            raise SystemExit(f"the prompt has {len(ids)} tokens; the model's context is {cfg.model.max_seq_len}")
        out = generate(model, x, min(args.max_new_tokens, room), args.temperature, args.top_k, args.top_p,
                       eos_token_id=tok.eos_token_id if tok else None,
                       generator=None if device.type == "cuda" else gen)
        new = out[0].tolist()
        return tok.decode(new) if tok else " ".join(map(str, new))

    if args.interactive:
        while True:
            try:
                line = input("prompt> ")
            except EOFError:
                break
            if line.strip() in ("", "quit", "exit"):
                break
            print(run(line))
    else:
        print(run(args.prompt or "1 2 3"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
