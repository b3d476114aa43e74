#!/usr/bin/env python
"""Convert between this framework's DCP checkpoints and HuggingFace (Llama / Mixtral-style) weights.

    python scripts/convert_checkpoint.py to-hf   <dcp_step_dir> <hf_dir> --config cfg.toml [--dtype bfloat16]
    python scripts/convert_checkpoint.py from-hf <hf_dir> <dcp_step_dir> --config cfg.toml
    python scripts/convert_checkpoint.py dcp-to-hf --dcp-dir <dcp_step_dir> --hf-dir <hf_dir> --config cfg.toml [--dtype bfloat16]
    python scripts/convert_checkpoint.py hf-to-dcp --hf-dir <hf_dir> --dcp-dir <dcp_step_dir> --config cfg.toml

``to-hf`` merges per-stage ``pp*/`` sub-directories of a pipeline-parallel checkpoint, renames the keys,
casts to the export dtype and writes ``model.safetensors`` (or ``pytorch_model.bin``) plus ``config.json``.
The sub-command forms are the reference's command line (scripts/convert_checkpoint.py:48-310); the key maps are the same.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import sys
from pathlib import Path

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed.checkpoint as dcp  # noqa: E402

from kempnerforge_b200.config import load_config  # noqa: E402
from kempnerforge_b200.models import Transformer  # noqa: E402

_TO_HF = [
    (r"^token_embedding\.embedding\.weight$", "model.embed_tokens.weight"),
    (r"^output_head\.proj\.weight$", "lm_head.weight"),
    (r"^norm\.weight$", "model.norm.weight"),
    (r"^layers\.(\d+)\.attention_norm\.", r"model.layers.\1.input_layernorm."),
    (r"^layers\.(\d+)\.mlp_norm\.", r"model.layers.\1.post_attention_layernorm."),
    (r"^layers\.(\d+)\.attention\.", r"model.layers.\1.self_attn."),
    (r"^layers\.(\d+)\.mlp\.router\.gate\.", r"model.layers.\1.mlp.gate."),
    (r"^layers\.(\d+)\.mlp\.router\.expert_bias$", r"model.layers.\1.mlp.expert_bias"),
    (r"^layers\.(\d+)\.mlp\.router\.expert_ema$", r"model.layers.\1.mlp.expert_ema"),
    (r"^layers\.(\d+)\.mlp\.shared_expert\.", r"model.layers.\1.mlp.shared_experts."),
    (r"^layers\.(\d+)\.", r"model.layers.\1."),
]
_FROM_HF = [
    (r"^model\.embed_tokens\.weight$", "token_embedding.embedding.weight"),
    (r"^lm_head\.weight$", "output_head.proj.weight"),
    (r"^model\.norm\.weight$", "norm.weight"),
    (r"^model\.layers\.(\d+)\.input_layernorm\.", r"layers.\1.attention_norm."),
    (r"^model\.layers\.(\d+)\.post_attention_layernorm\.", r"layers.\1.mlp_norm."),
    (r"^model\.layers\.(\d+)\.self_attn\.", r"layers.\1.attention."),
    (r"^model\.layers\.(\d+)\.mlp\.gate\.weight$", r"layers.\1.mlp.router.gate.weight"),
    (r"^model\.layers\.(\d+)\.mlp\.expert_bias$", r"layers.\1.mlp.router.expert_bias"),
    (r"^model\.layers\.(\d+)\.mlp\.expert_ema$", r"layers.\1.mlp.router.expert_ema"),
    (r"^model\.layers\.(\d+)\.mlp\.shared_experts\.", r"layers.\1.mlp.shared_expert."),
    (r"^model\.layers\.(\d+)\.", r"layers.\1."),
]


def _rename(key: str, table) -> str:
    for pat, rep in table:
        new, n = re.subn(pat, rep, key)
        if n:
            return new
    return key


def kf_to_hf_key(key: str) -> str:
    return _rename(key, _TO_HF)


def hf_to_kf_key(key: str) -> str:
    return _rename(key, _FROM_HF)


def build_hf_config(mc, dtype: str = "bfloat16") -> dict:
    cfg = {
        "architectures": ["MixtralForCausalLM" if mc.is_moe else "LlamaForCausalLM"],
        "model_type": "mixtral" if mc.is_moe else "llama",
        "hidden_size": mc.dim,
        "intermediate_size": mc.computed_expert_ffn_hidden_dim if mc.is_moe else mc.computed_ffn_hidden_dim,
        "num_hidden_layers": mc.n_layers,
        "num_attention_heads": mc.n_heads,
        "num_key_value_heads": mc.n_kv_heads,
        "vocab_size": mc.vocab_size,
        "max_position_embeddings": mc.max_seq_len,
        "rms_norm_eps": mc.norm_eps,
        "rope_theta": mc.rope_theta,
        "tie_word_embeddings": mc.tie_embeddings,
        "hidden_act": str(mc.activation),
        "torch_dtype": dtype,
    }
    if mc.is_moe:
        cfg.update(num_local_experts=mc.num_experts, num_experts_per_tok=mc.moe_top_k,
                   router_aux_loss_coef=mc.moe_aux_loss_weight)
    return cfg


def load_dcp_model_state(step_dir: Path, model: torch.nn.Module) -> dict[str, torch.Tensor]:
    """Model tensors of a checkpoint; ``pp*/`` stage directories are merged."""
    template = {k: torch.empty_like(v) for k, v in model.state_dict().items()}
    stage_dirs = sorted(p for p in step_dir.glob("pp*") if p.is_dir())
    if not stage_dirs:
        state = {"model": template}
        dcp.load(state, checkpoint_id=str(step_dir))
        return state["model"]
    merged: dict[str, torch.Tensor] = {}
    for d in stage_dirs:
        keys = {k[len("model."):] for k in dcp.FileSystemReader(str(d)).read_metadata().state_dict_metadata
                if k.startswith("model.")}
        part = {"model": {k: template[k] for k in keys if k in template}}
        dcp.load(part, checkpoint_id=str(d))
        merged.update(part["model"])
    missing = set(template) - set(merged)
    if missing:
        raise KeyError(f"pipeline stages do not cover: {sorted(missing)[:5]} ...")
    return merged


def dcp_to_hf(dcp_dir: str, hf_dir: str, model_config, dtype: str = "bfloat16") -> None:
    model = Transformer(model_config)
    state = load_dcp_model_state(Path(dcp_dir), model)
    tdtype = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[dtype]
    hf_state = {kf_to_hf_key(k): v.to(tdtype).contiguous() for k, v in state.items()}
    if model_config.tie_embeddings:
        hf_state.pop("lm_head.weight", None)
    out = Path(hf_dir)
    out.mkdir(parents=True, exist_ok=True)
    try:
        from safetensors.torch import save_file

        save_file(hf_state, str(out / "model.safetensors"))
    except ImportError:
        torch.save(hf_state, out / "pytorch_model.bin")
    (out / "config.json").write_text(json.dumps(build_hf_config(model_config, dtype), indent=2))
    print(f"wrote {len(hf_state)} tensors to {out}")


def hf_to_dcp(hf_dir: str, dcp_dir: str, model_config) -> None:
    src = Path(hf_dir)
    if (src / "model.safetensors").exists():
        from safetensors.torch import load_file

        hf_state = load_file(str(src / "model.safetensors"))
    else:
        hf_state = torch.load(src / "pytorch_model.bin", map_location="cpu", weights_only=True)
    model = Transformer(model_config)
    want = model.state_dict()
    new = {}
    for k, v in hf_state.items():
        kk = hf_to_kf_key(k)
        if kk in want:
            new[kk] = v.to(want[kk].dtype)
    if model_config.tie_embeddings and "output_head.proj.weight" not in new:
        new["output_head.proj.weight"] = new["token_embedding.embedding.weight"]
    missing = set(want) - set(new)
    if missing:
        raise KeyError(f"HF checkpoint lacks: {sorted(missing)[:5]} ...")
    Path(dcp_dir).mkdir(parents=True, exist_ok=True)
    dcp.save({"model": new}, checkpoint_id=str(dcp_dir))
    (Path(dcp_dir) / "metadata.json").write_text(json.dumps({"step": 0, "tokens_seen": 0}))
    print(f"wrote DCP checkpoint with {len(new)} tensors to {dcp_dir}")


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[1])
    if argv and argv[0] in ("dcp-to-hf", "hf-to-dcp"):
        # the reference's command line: sub-commands with named directories
        ap.add_argument("direction", choices=["dcp-to-hf", "hf-to-dcp"])
        ap.add_argument("--dcp-dir", required=True, help="DCP checkpoint directory")
        ap.add_argument("--hf-dir", required=True, help="HuggingFace directory")
        ap.add_argument("--config", required=True, help="TOML config file")
        ap.add_argument("--dtype", default=None, choices=["float32", "bfloat16", "float16"])
        args, overrides = ap.parse_known_args(argv)
        to_hf = args.direction == "dcp-to-hf"
        src, dst = (args.dcp_dir, args.hf_dir) if to_hf else (args.hf_dir, args.dcp_dir)
    else:
        ap.add_argument("direction", choices=["to-hf", "from-hf"])
        ap.add_argument("src")
        ap.add_argument("dst")
        ap.add_argument("--config", required=True)
        ap.add_argument("--dtype", default=None)
        args, overrides = ap.parse_known_args(argv)
        to_hf = args.direction == "to-hf"
        src, dst = args.src, args.dst
    cfg = load_config(args.config, overrides)
    if to_hf:
        dcp_to_hf(src, dst, cfg.model, args.dtype or cfg.checkpoint.export_dtype)
    else:
        hf_to_dcp(src, dst, cfg.model)
    return 0


if __name__ == "__main__":
    sys.exit(main())
