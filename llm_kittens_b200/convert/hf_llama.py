"""Hugging Face Llama-3 checkpoints <-> flat parameter buffer / model file.

The reference converts HF and Meta checkpoints in its PyTorch script (train_llama3.py:366-430, 841-930: the
``unpermute`` of the q / k projection rows undoes the half-split rotary layout that the HF exporter applies) and
has a small driver around it (dev/download_llama3.py). This module does the same conversion in both directions on
state dicts, without touching the network:

    python -m llm_kittens_b200.convert.hf_llama --hf-dir /path/to/Llama-3.2-1B --out llama3.2_1B_bf16.bin

Rotary convention: the framework rotates interleaved pairs (2i, 2i+1) (Meta's layout); HF rotates (i, i + HS/2)
and stores q / k rows permuted accordingly, so those rows are permuted back here.
"""
from __future__ import annotations

import argparse

import torch

from ..models.config import ModelConfig


def config_from_hf(hf, padded_vocab_size: int | None = None) -> ModelConfig:
    """``hf``: a ``transformers.LlamaConfig`` (or anything with the same attribute names)."""
    rope_scaling = getattr(hf, "rope_scaling", None) or {}
    if not rope_scaling:
        rope_scaling = (getattr(hf, "rope_parameters", None) or {})
    scaled = str(rope_scaling.get("rope_type", rope_scaling.get("type", "default"))) == "llama3"
    theta = getattr(hf, "rope_theta", None)
    if theta is None:
        theta = (getattr(hf, "rope_parameters", None) or {}).get("rope_theta", 500000.0)
    V = hf.vocab_size
    return ModelConfig(family="llama3", max_seq_len=hf.max_position_embeddings, vocab_size=V,
                       padded_vocab_size=padded_vocab_size or V, num_layers=hf.num_hidden_layers, num_heads=hf.num_attention_heads,
                       num_kv_heads=getattr(hf, "num_key_value_heads", hf.num_attention_heads), channels=hf.hidden_size,
                       hidden_dim=hf.intermediate_size, norm_eps=hf.rms_norm_eps, rope_theta=float(theta), use_scaled_rope=scaled,
                       tied_embeddings=bool(getattr(hf, "tie_word_embeddings", False)), descriptor="hf-llama")


def _hf_to_interleaved(w: torch.Tensor, heads: int) -> torch.Tensor:
    """[heads*HS, C] rows in HF order (first half / second half of every head) -> interleaved pairs."""
    rows, cols = w.shape
    hs = rows // heads
    return w.view(heads, 2, hs // 2, cols).transpose(1, 2).reshape(rows, cols)


def _interleaved_to_hf(w: torch.Tensor, heads: int) -> torch.Tensor:
    rows, cols = w.shape
    hs = rows // heads
    return w.view(heads, hs // 2, 2, cols).transpose(1, 2).reshape(rows, cols)


def params_from_hf(state_dict: dict, config: ModelConfig, dtype=torch.bfloat16) -> torch.Tensor:
    """Flat parameter vector (checkpoint order of ``config.layout()``) from an HF ``LlamaForCausalLM`` state dict."""
    lay = config.layout()
    flat = torch.zeros(lay.total, dtype=dtype)
    v = lay.views(flat)
    sd = {k.removeprefix("model."): t for k, t in state_dict.items()}
    V = config.vocab_size
    v["wte"][:V].copy_(sd["embed_tokens.weight"])
    v["lnfw"].copy_(sd["norm.weight"])
    if not config.tied_embeddings:
        v["lm_head"][:V].copy_(state_dict.get("lm_head.weight", sd["embed_tokens.weight"]))
    for l in range(config.num_layers):
        p = f"layers.{l}."
        q = _hf_to_interleaved(sd[p + "self_attn.q_proj.weight"].float(), config.num_heads)
        k = _hf_to_interleaved(sd[p + "self_attn.k_proj.weight"].float(), config.num_kv_heads)
        v["qkvw"][l].copy_(torch.cat([q, k, sd[p + "self_attn.v_proj.weight"].float()], dim=0))
        v["attprojw"][l].copy_(sd[p + "self_attn.o_proj.weight"])
        v["ln1w"][l].copy_(sd[p + "input_layernorm.weight"])
        v["ln2w"][l].copy_(sd[p + "post_attention_layernorm.weight"])
        v["fcw_up"][l].copy_(sd[p + "mlp.up_proj.weight"])
        v["fcw_gate"][l].copy_(sd[p + "mlp.gate_proj.weight"])
        v["fcprojw"][l].copy_(sd[p + "mlp.down_proj.weight"])
    return flat


def params_to_hf(flat: torch.Tensor, config: ModelConfig) -> dict:
    """The inverse: an HF-style state dict (float32 tensors) from the flat parameter vector."""
    v = config.layout().views(flat.float())
    V, NH, NKV, HS = config.vocab_size, config.num_heads, config.num_kv_heads, config.head_size
    sd = {"model.embed_tokens.weight": v["wte"][:V].clone(), "model.norm.weight": v["lnfw"].clone()}
    sd["lm_head.weight"] = (v["wte"] if config.tied_embeddings else v["lm_head"])[:V].clone()
    for l in range(config.num_layers):
        p = f"model.layers.{l}."
        qkv = v["qkvw"][l]
        q, k, vv = qkv[:NH * HS], qkv[NH * HS:(NH + NKV) * HS], qkv[(NH + NKV) * HS:]
        sd[p + "self_attn.q_proj.weight"] = _interleaved_to_hf(q.contiguous(), NH)
        sd[p + "self_attn.k_proj.weight"] = _interleaved_to_hf(k.contiguous(), NKV)
        sd[p + "self_attn.v_proj.weight"] = vv.clone()
        sd[p + "self_attn.o_proj.weight"] = v["attprojw"][l].clone()
        sd[p + "input_layernorm.weight"] = v["ln1w"][l].clone()
        sd[p + "post_attention_layernorm.weight"] = v["ln2w"][l].clone()
        sd[p + "mlp.up_proj.weight"] = v["fcw_up"][l].clone()
        sd[p + "mlp.gate_proj.weight"] = v["fcw_gate"][l].clone()
        sd[p + "mlp.down_proj.weight"] = v["fcprojw"][l].clone()
    return sd


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Convert a local Hugging Face Llama checkpoint to a model file")
    ap.add_argument("--hf-dir", required=True, help="directory with config.json and the weight files (no download is attempted)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--fp32", action="store_true")
    args = ap.parse_args(argv)
    from transformers import AutoConfig, AutoModelForCausalLM

    from ..utils import formats

    hf_cfg = AutoConfig.from_pretrained(args.hf_dir, local_files_only=True)
    model = AutoModelForCausalLM.from_pretrained(args.hf_dir, local_files_only=True, torch_dtype=torch.float32)
    cfg = config_from_hf(hf_cfg)
    flat = params_from_hf(model.state_dict(), cfg, dtype=torch.float32 if args.fp32 else torch.bfloat16)
    formats.write_model(args.out, cfg, flat)
    print(f"wrote {args.out}: {cfg.num_layers} layers, {flat.numel():,} parameters")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
