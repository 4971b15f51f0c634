"""Weights on disk, on either side of the decode path.

The reference builds its runtime from a Hugging Face state dict in memory and quantizes every matrix at start-up
(runtime/model.py:56-72, 75-116); GPTQ parameters are calibrated once per process and kept in a dict
(README.md:43-44, bench/e2e.py:56-66). For checkpoints of real size that is minutes of work per run, so this module adds
the two formats that stand on either side of the path:

  * IN  - `HFCheckpoint(dir)`: a Hugging Face Llama checkpoint directory (config.json plus *.safetensors, sharded or
    not, with or without model.safetensors.index.json), read lazily: a state-dict look-alike that fetches a tensor
    from its shard when `Model` asks for it, so only one fp16 matrix is alive at a time.
  * OUT - `save_quantized(model, dir)` / `load_quantized(dir)`: the model in kernel format - per matrix the packed
    INT4 words and the (scale, zero) pairs exactly as runtime/quant.py lays them out, the norm vectors, the embedding -
    in one safetensors file plus meta.json. `Model.from_quantized(dir, cfg)` starts from it without touching a
    quantizer (DecodeConfig.quant = "packed").
  * `cached_qparams(dir, key, make)`: GPTQ results ({name: (q, scale, zero)}) stored under a key that names what
    they depend on (shapes, group, clipping, calibration seed and size); `make()` runs only on a miss.

Everything here is host-side file handling on CPU tensors; nothing is launched.
"""
import hashlib
import json
import types
from pathlib import Path

import torch
from safetensors import safe_open
from safetensors.torch import load_file, save_file

FORMAT = "b200-w4a16-packed"
FORMAT_VERSION = 1
CONFIG_KEYS = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "intermediate_size",
               "vocab_size", "rms_norm_eps", "rope_theta", "head_dim")
MATRICES = ("qkv", "o", "gu", "down")


# ------------------------------------------------------------------------------------------------ Hugging Face side
class HFCheckpoint:
    """Lazy view of a Hugging Face checkpoint directory: `ck[name]` reads one tensor, `name in ck`, `ck.keys()`.
    `ck.config` is a namespace with the fields `Model` reads."""

    def __init__(self, path):
        self.path = Path(path)
        cfg = json.loads((self.path / "config.json").read_text())
        rope = cfg.get("rope_theta")
        if rope is None and isinstance(cfg.get("rope_parameters"), dict):   # newer transformers keep it there
            rope = cfg["rope_parameters"].get("rope_theta")
        cfg["rope_theta"] = 10000.0 if rope is None else rope
        self.config = types.SimpleNamespace(**{k: cfg[k] for k in CONFIG_KEYS if cfg.get(k) is not None})
        index = self.path / "model.safetensors.index.json"
        if index.is_file():
            self.where = dict(json.loads(index.read_text())["weight_map"])
        else:
            self.where = {}
            for f in sorted(self.path.glob("*.safetensors")):
                with safe_open(str(f), framework="pt") as sf:
                    for k in sf.keys():
                        self.where[k] = f.name
        if not self.where:
            raise FileNotFoundError(f"no safetensors weights under {self.path}")
        self._open = {}

    def keys(self):
        return self.where.keys()

    def __contains__(self, key):
        return key in self.where

    def __getitem__(self, key):
        fname = self.where[key]
        if fname not in self._open:
            self._open[fname] = safe_open(str(self.path / fname), framework="pt")
        return self._open[fname].get_tensor(key)


def write_hf_checkpoint(state, config, path, shards=1):
    """Write a state dict as a Hugging Face style directory (config.json, safetensors shard(s), index). The inverse of
    HFCheckpoint, used to export random-weight stand-ins and by the tests."""
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    cfg = {k: getattr(config, k) for k in CONFIG_KEYS if getattr(config, k, None) is not None}
    (path / "config.json").write_text(json.dumps(dict(cfg, model_type="llama", architectures=["LlamaForCausalLM"])))
    names = list(state.keys())
    per = -(-len(names) // shards)
    weight_map = {}
    for s in range(shards):
        part = names[s * per:(s + 1) * per]
        fname = "model.safetensors" if shards == 1 else f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        save_file({k: state[k].detach().cpu().contiguous() for k in part}, str(path / fname))
        weight_map.update({k: fname for k in part})
    if shards > 1:
        (path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    return path


# ------------------------------------------------------------------------------------------------ kernel-format side
def save_quantized(model, path):
    """Store a built `Model` in kernel format: <path>/weights.safetensors and <path>/meta.json. Needs the row-major
    packed tensors (DecodeConfig.keep_packed=True, the default) and a model that is not tensor-parallel (shards are
    cut again when the file is loaded with a tensor-parallel configuration)."""
    if model.tp != 1:
        raise ValueError("save the unsharded model; tensor-parallel ranks cut their shards when they load it")
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    t = {"embed": model.emb, "norm_f": model.norm_f}
    for i, lw in enumerate(model.layers):
        t[f"layers.{i}.ln1"], t[f"layers.{i}.ln2"] = lw["ln1"], lw["ln2"]
        for name in MATRICES:
            if lw[name].packed is None:
                raise ValueError("the row-major packed tensors were dropped (keep_packed=False); nothing to save")
            t[f"layers.{i}.{name}.packed"], t[f"layers.{i}.{name}.sz"] = lw[name].packed, lw[name].sz
    t["lm_head.packed"], t["lm_head.sz"] = model.lm_head.packed, model.lm_head.sz
    save_file({k: v.detach().cpu().contiguous() for k, v in t.items()}, str(path / "weights.safetensors"))
    meta = {"format": FORMAT, "version": FORMAT_VERSION, "group": model.cfg.group, "quant": model.cfg.quant,
            "config": {"hidden_size": model.H, "num_hidden_layers": model.L, "num_attention_heads": model.n_q,
                       "num_key_value_heads": model.n_kv, "intermediate_size": model.I, "vocab_size": model.V_full,
                       "rms_norm_eps": model.eps, "rope_theta": model.rope_theta, "head_dim": model.D},
            "layout": "packed int32 [N, K/8]: element 8j+2i in bits [4i, 4i+4), 8j+2i+1 in bits [16+4i, 16+4i+4) of "
                      "word j; sz fp16 [N, K/group, 2] = (scale, zero); qkv rows [q; k; v], gu rows [gate; up]"}
    (path / "meta.json").write_text(json.dumps(meta, indent=1))
    return path


def load_quantized(path):
    """-> (config namespace, group, state, qparams): `state` holds embedding and norm vectors under their Hugging Face
    names, `qparams` maps "layers.{i}.{qkv,o,gu,down}" / "lm_head" to (packed, sz) - what
    DecodeConfig(quant="packed", qparams=...) consumes. CPU tensors."""
    path = Path(path)
    meta = json.loads((path / "meta.json").read_text())
    if meta.get("format") != FORMAT or meta.get("version") != FORMAT_VERSION:
        raise ValueError(f"{path}: not a {FORMAT} v{FORMAT_VERSION} directory")
    t = load_file(str(path / "weights.safetensors"))
    c = types.SimpleNamespace(**meta["config"])
    state = {"model.embed_tokens.weight": t["embed"], "model.norm.weight": t["norm_f"]}
    qparams = {"lm_head": (t["lm_head.packed"], t["lm_head.sz"])}
    for i in range(c.num_hidden_layers):
        state[f"model.layers.{i}.input_layernorm.weight"] = t[f"layers.{i}.ln1"]
        state[f"model.layers.{i}.post_attention_layernorm.weight"] = t[f"layers.{i}.ln2"]
        for name in MATRICES:
            qparams[f"layers.{i}.{name}"] = (t[f"layers.{i}.{name}.packed"], t[f"layers.{i}.{name}.sz"])
    return c, meta["group"], state, qparams


# ------------------------------------------------------------------------------------------------ cached GPTQ results
def qparams_key(**what):
    """A short stable name for everything a set of GPTQ parameters depends on (pass shapes, group, clip, calibration
    seed / windows / length, ...)."""
    blob = json.dumps(what, sort_keys=True, default=str).encode()
    return hashlib.sha256(blob).hexdigest()[:16]


def cached_qparams(cache_dir, key, make):
    """{name: (q uint8 [N, K], scale fp16 [N, K/G], zero fp16 [N, K/G])} from <cache_dir>/qparams-<key>.safetensors,
    or from make() - whose result is then stored there."""
    f = Path(cache_dir) / f"qparams-{key}.safetensors"
    if f.is_file():
        t = load_file(str(f))
        names = sorted({k.rsplit(".", 1)[0] for k in t})
        return {n: (t[n + ".q"], t[n + ".scale"], t[n + ".zero"]) for n in names}
    qp = make()
    f.parent.mkdir(parents=True, exist_ok=True)
    flat = {}
    for n, (q, s, z) in qp.items():
        # clone: safetensors refuses two names over one storage (tied or reused tensors)
        flat[n + ".q"], flat[n + ".scale"], flat[n + ".zero"] = (x.detach().cpu().contiguous().clone() for x in (q, s, z))
    save_file(flat, str(f))
    return qp
