"""Sequential GPTQ calibration of a HF Llama model into the decode runtime's INT4 format.

Same entry point and output as the reference's runtime/gptq.py:31-107: `calibrate(hf, tok, group, clip, n, L, lm_head,
log)` returns {"layers.{i}.qkv|o|gu|down", "lm_head"} -> (q uint8 [N, K], scale fp16 [N, K/G], zero fp16 [N, K/G]), the
dict that `DecodeConfig(quant="pre", qparams=...)` consumes.

Method (as there): decoder layers are handled in order. The inputs of layer i are the outputs of the already
quantized layers 0..i-1; forward hooks on the layer's four distinct linear inputs accumulate H = sum x^T x; q/k/v share
one input and are quantized as one stacked matrix (rows are independent in GPTQ), likewise gate/up; the dequantized
weights are written into the HF layer before its outputs are recomputed for the next layer; the LM head is calibrated
last on the final-norm outputs; the HF weights are restored at the end.

Calibration text: the reference samples WikiText-2 (train). That dataset is not available offline, so
`calibration_windows` here draws uniform random token ids (seeded) - the substitution the reference's own unit test
makes (tests/test_quant_local.py:76). Replace the function to calibrate on real text.
"""
import time

import torch

from .quant import dequantize, quantize_gptq


def calibration_windows(tok, n=128, L=512, seed=0, vocab_size=None):
    """n windows of L token ids: BOS followed by L-1 uniform random ids in [0, vocab)."""
    vocab = vocab_size or getattr(tok, "vocab_size", None) or 32000
    g = torch.Generator().manual_seed(seed)
    bos = torch.tensor([getattr(tok, "bos_token_id", 1) or 1])
    return [torch.cat([bos, torch.randint(0, vocab, (L - 1,), generator=g)]) for _ in range(n)]


class _StopForward(Exception):
    pass


class _InputTap(torch.nn.Module):
    """Stands in for decoder layer 0 during the first pass: records what the model feeds it, then aborts the forward."""

    def __init__(self, sink, kwargs_sink):
        super().__init__()
        self.sink, self.kwargs_sink = sink, kwargs_sink

    def forward(self, hidden_states, *args, **kwargs):
        self.sink.append(hidden_states)
        self.kwargs_sink.update(kwargs)
        raise _StopForward


@torch.no_grad()
def calibrate(hf, tok, group=128, clip=False, n=128, L=512, lm_head=True, log=print):
    dev = next(hf.parameters()).device
    layers = hf.model.layers
    windows = calibration_windows(tok, n, L)

    # inputs of layer 0 and the keyword arguments (rotary embeddings, mask, positions) every layer receives
    acts, layer_kwargs = [], {}
    first = layers[0]
    layers[0] = _InputTap(acts, layer_kwargs)
    try:
        for w in windows:
            try:
                hf.model(w[None].to(dev), use_cache=False)
            except _StopForward:
                pass
    finally:
        layers[0] = first
    for k in ("past_key_values", "past_key_value", "use_cache"):
        layer_kwargs.pop(k, None)

    def run(layer, x):
        out = layer(x, **layer_kwargs)
        return out[0] if isinstance(out, tuple) else out

    result, originals = {}, []
    t0 = time.time()
    for i, layer in enumerate(layers):
        att, mlp = layer.self_attn, layer.mlp
        plan = (("qkv", att.q_proj, (att.q_proj, att.k_proj, att.v_proj)),
                ("o", att.o_proj, (att.o_proj,)),
                ("gu", mlp.gate_proj, (mlp.gate_proj, mlp.up_proj)),
                ("down", mlp.down_proj, (mlp.down_proj,)))
        hess = {key: [None, 0] for key, _, _ in plan}

        def tap(key):
            def hook(_mod, args, _out):
                x = args[0].reshape(-1, args[0].shape[-1]).float()
                h = hess[key]
                h[0] = x.t() @ x if h[0] is None else h[0] + x.t() @ x
                h[1] += x.shape[0]
            return hook

        handles = [probe.register_forward_hook(tap(key)) for key, probe, _ in plan]
        for x in acts:
            run(layer, x)
        for h in handles:
            h.remove()
        for key, _, mods in plan:
            W = torch.cat([m.weight.data for m in mods], 0)
            H, cnt = hess[key]
            q, s, z = quantize_gptq(W, 2 * H / cnt, group, clip=clip)
            result[f"layers.{i}.{key}"] = (q.cpu(), s.cpu(), z.cpu())
            deq = dequantize(q, s, z, group)
            row = 0
            for m in mods:
                originals.append((m, m.weight.data.detach().cpu().clone()))
                m.weight.data.copy_(deq[row:row + m.weight.shape[0]])
                row += m.weight.shape[0]
        del hess
        acts = [run(layer, x) for x in acts]   # the next layer sees this layer's quantized outputs
        log(f"gptq layer {i}: {time.time() - t0:.0f}s")

    if lm_head:
        H, cnt = None, 0
        for x in acts:
            y = hf.model.norm(x).reshape(-1, x.shape[-1]).float()
            H = y.t() @ y if H is None else H + y.t() @ y
            cnt += y.shape[0]
        q, s, z = quantize_gptq(hf.lm_head.weight.data, 2 * H / cnt, group, clip=clip)
        result["lm_head"] = (q.cpu(), s.cpu(), z.cpu())

    for m, w in originals:
        m.weight.data.copy_(w.to(dev))
    log(f"gptq done: {time.time() - t0:.0f}s, {len(result)} matrices")
    return result


def calibrate_cached(hf, tok, cache_dir, group=128, clip=False, n=128, L=512, lm_head=True, seed=0, log=print):
    """calibrate() behind the on-disk cache of checkpoint.cached_qparams: the key names the model's shapes, the group
    size, the clipping switch and the calibration set (windows, length, seed), so a second run with the same settings
    loads the parameters instead of calibrating for minutes. The calibration windows are this module's
    `calibration_windows` with the given seed."""
    from . import checkpoint
    c = hf.config
    key = checkpoint.qparams_key(hidden=c.hidden_size, layers=c.num_hidden_layers, heads=c.num_attention_heads,
                                 kv_heads=c.num_key_value_heads, inter=c.intermediate_size, vocab=c.vocab_size,
                                 group=group, clip=clip, n=n, L=L, lm_head=lm_head, seed=seed,
                                 weights=_fingerprint(hf))
    return checkpoint.cached_qparams(cache_dir, key,
                                     lambda: calibrate(hf, tok, group=group, clip=clip, n=n, L=L, lm_head=lm_head, log=log))


def _fingerprint(hf):
    """A cheap identity of the weights being calibrated: sums of a few tensors (the cache must not hand the
    parameters of one checkpoint to another of the same shape)."""
    sd = hf.state_dict()
    keys = sorted(sd)[:: max(1, len(sd) // 8)]
    return [round(float(sd[k].float().sum()), 4) for k in keys]
