"""Weights to and from the Hugging Face layout of the same architectures (Qwen3, Llama 3).

The module tree here keeps the reference's names (``token_emb``, ``blocks.N.gqa.q_proj``, ``blocks.N.ffn.gate_proj``,
``norm``, ``lm_head``; reference ``torchure/models/qwen3/qwen3.py:266-353``); the Hugging Face classes call the same
tensors ``model.embed_tokens``, ``model.layers.N.self_attn.q_proj``, ``model.layers.N.mlp.gate_proj``, ``model.norm``.
Both use the half-split RoPE convention and apply the per-head QK-norm before the rotation, so the mapping is a pure
renaming: no tensor is permuted.

    python -m torchure_b200.models.hf import <hf_dir> <out_model.pt>     # also prints the `model` section of a config
    python -m torchure_b200.models.hf export <model.pt> <config.json> <out_hf_dir>

``import`` writes an unsharded state dict that a run on any mesh can start from (config key ``init_from``).
"""

from __future__ import annotations

import argparse
import json

import torch

_TOP = {"token_emb.weight": "model.embed_tokens.weight", "norm.weight": "model.norm.weight",
        "lm_head.weight": "lm_head.weight"}
_BLOCK = {"gqa.q_proj.weight": "self_attn.q_proj.weight", "gqa.k_proj.weight": "self_attn.k_proj.weight",
          "gqa.v_proj.weight": "self_attn.v_proj.weight", "gqa.o_proj.weight": "self_attn.o_proj.weight",
          "gqa.q_norm.weight": "self_attn.q_norm.weight", "gqa.k_norm.weight": "self_attn.k_norm.weight",
          "ffn.gate_proj.weight": "mlp.gate_proj.weight", "ffn.up_proj.weight": "mlp.up_proj.weight",
          "ffn.down_proj.weight": "mlp.down_proj.weight", "norm1.weight": "input_layernorm.weight",
          "norm2.weight": "post_attention_layernorm.weight"}
_BLOCK_BACK = {v: k for k, v in _BLOCK.items()}
_TOP_BACK = {v: k for k, v in _TOP.items()}


def to_hf_state_dict(state: dict) -> dict:
    out = {}
    for key, value in state.items():
        if key in _TOP:
            out[_TOP[key]] = value
        elif key.startswith("blocks."):
            _, idx, rest = key.split(".", 2)
            if rest not in _BLOCK:
                raise KeyError(f"no Hugging Face name for {key!r} (dense decoder blocks only)")
            out[f"model.layers.{idx}.{_BLOCK[rest]}"] = value
        else:
            raise KeyError(f"no Hugging Face name for {key!r}")
    return out


def from_hf_state_dict(hf_state: dict, tie_embeddings: bool = True) -> dict:
    out = {}
    for key, value in hf_state.items():
        if "rotary_emb" in key:        # buffers recomputed from the config
            continue
        if key in _TOP_BACK:
            out[_TOP_BACK[key]] = value
        elif key.startswith("model.layers."):
            _, _, idx, rest = key.split(".", 3)
            if rest not in _BLOCK_BACK:
                raise KeyError(f"{key!r} has no counterpart here (biases, sliding-window or MoE variants are not covered)")
            out[f"blocks.{idx}.{_BLOCK_BACK[rest]}"] = value
        else:
            raise KeyError(f"{key!r} has no counterpart here")
    if tie_embeddings and "lm_head.weight" not in out:
        out["lm_head.weight"] = out["token_emb.weight"]
    return out


def model_section_from_hf(hf_config) -> dict:
    """The ``model`` section of a run config for a Hugging Face Qwen3 / Llama config object."""
    kind = getattr(hf_config, "model_type", "")
    if kind not in ("qwen3", "llama"):
        raise ValueError(f"model_type {kind!r} is not covered (qwen3 and llama are)")
    if getattr(hf_config, "attention_bias", False) or getattr(hf_config, "mlp_bias", False):
        raise ValueError("projection biases are not covered")
    heads = hf_config.num_attention_heads
    cfg = dict(num_layers=hf_config.num_hidden_layers, num_heads=heads,
               num_kv_heads=getattr(hf_config, "num_key_value_heads", None) or heads, emb_dim=hf_config.hidden_size,
               head_dim=getattr(hf_config, "head_dim", None) or hf_config.hidden_size // heads,
               vocab_size=hf_config.vocab_size, ffn_dim=hf_config.intermediate_size, norm_eps=hf_config.rms_norm_eps,
               rope_theta=float(getattr(hf_config, "rope_theta", None) or hf_config.rope_parameters["rope_theta"]),
               tie_embeddings=bool(getattr(hf_config, "tie_word_embeddings", False)))
    return {"name": "qwen3_dense" if kind == "qwen3" else "llama3_2", "config": cfg}


def hf_config_from_model_section(section: dict):
    import transformers

    c = section["config"]
    common = dict(vocab_size=c["vocab_size"], hidden_size=c["emb_dim"], intermediate_size=c["ffn_dim"],
                  num_hidden_layers=c["num_layers"], num_attention_heads=c["num_heads"],
                  num_key_value_heads=c["num_kv_heads"], tie_word_embeddings=c.get("tie_embeddings", True),
                  attention_bias=False)
    if section["name"] == "qwen3_dense":
        return transformers.Qwen3Config(head_dim=c.get("head_dim") or c["emb_dim"] // c["num_heads"],
                                        rms_norm_eps=c.get("norm_eps", 1e-6), rope_theta=c.get("rope_theta", 1e6),
                                        use_sliding_window=False, **common)
    if section["name"] == "llama3_2":
        return transformers.LlamaConfig(head_dim=c.get("head_dim") or c["emb_dim"] // c["num_heads"],
                                        rms_norm_eps=c.get("norm_eps", 1e-5), rope_theta=c.get("rope_theta", 5e5),
                                        mlp_bias=False, **common)
    raise ValueError(f"model {section['name']!r} has no Hugging Face counterpart here")


def import_hf(hf_dir: str, out_path: str) -> dict:
    """Read a local Hugging Face model directory; write our unsharded state dict; return the config's model section."""
    import transformers

    hf = transformers.AutoModelForCausalLM.from_pretrained(hf_dir, torch_dtype=torch.float32)
    section = model_section_from_hf(hf.config)
    state = from_hf_state_dict(hf.state_dict(), section["config"]["tie_embeddings"])
    torch.save({k: v.detach().clone().contiguous() for k, v in state.items()}, out_path)
    return section


def export_hf(model_path: str, section: dict, out_dir: str) -> None:
    """Write a Hugging Face model directory from our unsharded state dict and the config's model section."""
    import transformers

    hf = transformers.AutoModelForCausalLM.from_config(hf_config_from_model_section(section))
    state = to_hf_state_dict(torch.load(model_path, map_location="cpu", weights_only=True))
    missing, unexpected = hf.load_state_dict(state, strict=False)
    bad = [m for m in missing if "rotary" not in m and "inv_freq" not in m]
    if bad or unexpected:
        raise RuntimeError(f"state dict does not fit the architecture: missing {bad}, unexpected {unexpected}")
    hf.save_pretrained(out_dir)


def main() -> None:
    ap = argparse.ArgumentParser(description="Convert weights between this repository's layout and Hugging Face's")
    sub = ap.add_subparsers(dest="cmd", required=True)
    imp = sub.add_parser("import")
    imp.add_argument("hf_dir")
    imp.add_argument("out")
    exp = sub.add_parser("export")
    exp.add_argument("model")
    exp.add_argument("config", help="run config (JSON) whose `model` section describes the architecture")
    exp.add_argument("out_dir")
    args = ap.parse_args()
    if args.cmd == "import":
        print(json.dumps({"model": import_hf(args.hf_dir, args.out)}, indent=2))
    else:
        with open(args.config) as f:
            export_hf(args.model, json.load(f)["model"], args.out_dir)


if __name__ == "__main__":
    main()
