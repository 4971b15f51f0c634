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


class LazyRandomState:
    """A state-dict look-alike that makes each tensor when it is asked for, from a seed derived from the key.

    A 70B-shape model in fp16 is 140 GB; its quantized form is 38 GB. `Model` reads every key exactly once, layer by
    layer, so handing it this object instead of a dict keeps only one fp16 matrix alive at a time. Every rank of a
    tensor-parallel group builds the same full matrix from the same seed and keeps its own slice."""

    def __init__(self, c, device, seed=0, dtype=torch.float16):
        self.c, self.device, self.seed, self.dtype = c, device, seed, dtype
        H, I, V = c.hidden_size, c.intermediate_size, c.vocab_size
        D = getattr(c, "head_dim", None) or H // c.num_attention_heads
        self.shapes = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,), "lm_head.weight": (V, H)}
        for i in range(c.num_hidden_layers):
            p = f"model.layers.{i}."
            self.shapes.update({
                p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,),
                p + "self_attn.q_proj.weight": (c.num_attention_heads * D, H),
                p + "self_attn.k_proj.weight": (c.num_key_value_heads * D, H),
                p + "self_attn.v_proj.weight": (c.num_key_value_heads * D, H),
                p + "self_attn.o_proj.weight": (H, c.num_attention_heads * D),
                p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H),
                p + "mlp.down_proj.weight": (H, I)})
        self.order = {k: n for n, k in enumerate(self.shapes)}

    def __contains__(self, key):
        return key in self.shapes

    def keys(self):
        return self.shapes.keys()

    def __getitem__(self, key):
        shape = self.shapes[key]
        if len(shape) == 1:
            return torch.ones(shape, dtype=self.dtype, device=self.device)
        g = torch.Generator(device=self.device).manual_seed(self.seed * 100003 + self.order[key])
        return (torch.randn(*shape, generator=g, device=self.device) * 0.02).to(self.dtype)
