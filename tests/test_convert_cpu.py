"""HF Llama conversion: logits of a random tiny HF model equal the oracle's on the converted parameters."""
import pytest
import torch


def test_hf_llama_roundtrip_and_logits():
    transformers = pytest.importorskip("transformers")
    from llm_kittens_b200.convert import hf_llama
    from llm_kittens_b200.oracle.torch_model import forward_logits

    hf_cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                      rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False, attention_bias=False)
    torch.manual_seed(0)
    model = transformers.LlamaForCausalLM(hf_cfg).eval()
    cfg = hf_llama.config_from_hf(hf_cfg)
    assert (cfg.num_heads, cfg.num_kv_heads, cfg.channels, cfg.hidden_dim) == (4, 2, 64, 128)
    flat = hf_llama.params_from_hf(model.state_dict(), cfg, dtype=torch.float32)
    tokens = torch.randint(0, 128, (2, 16))
    with torch.no_grad():
        ref = model(tokens).logits
        ours = forward_logits(cfg, cfg.layout().views(flat), tokens, rope_interleaved=True)
    assert torch.allclose(ours, ref, atol=2e-4), (ours - ref).abs().max()
    back = hf_llama.params_to_hf(flat, cfg)
    for k, t in model.state_dict().items():
        assert torch.allclose(back[k], t.float(), atol=0), k
