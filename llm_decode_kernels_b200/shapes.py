"""Model shapes of the benchmark configurations and seeded random weights for them.

The configurations name real checkpoints (TinyLlama-1.1B, Llama-3-70B) whose weights are not available offline;
random N(0, 0.02) weights of the same shapes stand in (HF LlamaConfig's initializer_range; norm weights are 1).
"""
import types

import torch

TINYLLAMA = dict(hidden_size=2048, num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4,
                 intermediate_size=5632, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0)
LLAMA3_70B = dict(hidden_size=8192, num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8,
                  intermediate_size=28672, vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0)


def config(shape: dict, **override):
    return types.SimpleNamespace(**{**shape, **override})


def random_layer_state(c, i, device, gen, dtype=torch.float16):
    """HF-named tensors of decoder layer i."""
    rn = lambda *s: (torch.randn(*s, generator=gen, device=device) * 0.02).to(dtype)
    H, I = c.hidden_size, c.intermediate_size
    D = getattr(c, "head_dim", None) or H // c.num_attention_heads
    p = f"model.layers.{i}."
    return {p + "input_layernorm.weight": torch.ones(H, dtype=dtype, device=device),
            p + "post_attention_layernorm.weight": torch.ones(H, dtype=dtype, device=device),
            p + "self_attn.q_proj.weight": rn(c.num_attention_heads * D, H),
            p + "self_attn.k_proj.weight": rn(c.num_key_value_heads * D, H),
            p + "self_attn.v_proj.weight": rn(c.num_key_value_heads * D, H),
            p + "self_attn.o_proj.weight": rn(H, c.num_attention_heads * D),
            p + "mlp.gate_proj.weight": rn(I, H),
            p + "mlp.up_proj.weight": rn(I, H),
            p + "mlp.down_proj.weight": rn(H, I)}


def random_llama_state(c, device, seed, dtype=torch.float16, layers=None):
    """Whole HF-Llama-named state dict; `layers` builds only the first that many decoder layers."""
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *s: (torch.randn(*s, generator=g, device=device) * 0.02).to(dtype)
    H, V = c.hidden_size, c.vocab_size
    sd = {"model.embed_tokens.weight": rn(V, H), "model.norm.weight": torch.ones(H, dtype=dtype, device=device),
          "lm_head.weight": rn(V, H)}
    for i in range(c.num_hidden_layers if layers is None else layers):
        sd.update(random_layer_state(c, i, device, g, dtype))
    return sd
