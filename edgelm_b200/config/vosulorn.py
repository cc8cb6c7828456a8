"""The Vosulorn decoder's configuration, from its own config.json keys.

config.json: `architecture` "Vosulorn", `vocab`, `width`, `norm.eps`, `embedding.scale` (the embedding's rows are
multiplied by it) and `layers`, a list with one entry per layer: `type` ("delta", "attention" or "latent_attention"),
`mixer` (the mixer's sizes and constants) and `mlp` ({"kind": "moe", "expert": {"ff": n}, "router": {"experts": n,
"top": k}} or null for a layer without a feed-forward).  Optional: `max_positions`.  Tensors: `embed`, `l<i>.norm1`,
`l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.e<j>.{gate,up,down}`, `l<i>.mlp.router`, `l<i>.mlp.router.b`, `final.norm`, `head`.

Every layer is pre-norm: x += mixer(norm1(x)); x += ff(norm2(x)).  The mixers:
  delta              the gated delta rule (`parts/gated_delta.py`): `heads`, `kv_heads`, `dim`, `vdim`, `conv`
  attention          grouped heads with biases, neighbouring-pair rotation of the first `rot.dims` dimensions (`rot.base`,
                     optional `rot.scaling` {factor, low, high, original}), `scale`, a chunked mask `mask.size` (absent:
                     causal) and a sink per head (`parts/masked_attention.py`)
  latent_attention   keys and values from a shared latent (`parts/latent_attention.py`): `heads`, `dim`, `rot_dim`,
                     `vdim`, `kv_rank`, `scale`, `rot.base`; with `kv_from`: j it keeps nothing and reads what layer j kept
"""
from dataclasses import dataclass
from typing import Any, Mapping, Tuple

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, ScheduleEntry, optional, require
from .registry import register_architecture

DEFAULT_MAX_POSITIONS = 1 << 20


def _sub(d, key, where):
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where}: key '{key}' should be an object, found {v!r}")
    return v


def _rotation(m, where, dims_key=None):
    """(dims, base, scaling) of a mixer's `rot` object; (0, None, None) without one."""
    rot = m.get("rot")
    if rot is None:
        return 0, None, None
    if not isinstance(rot, Mapping):
        raise ConfigError(f"{where}: key 'rot' should be an object")
    scaling = rot.get("scaling")
    if scaling is not None:
        if not isinstance(scaling, Mapping):
            raise ConfigError(f"{where} rot: key 'scaling' should be an object")
        scaling = {k: require(scaling, k, float, where + " rot scaling") for k in ("factor", "low", "high", "original")}
    return require(rot, "dims", int, where + " rot"), require(rot, "base", float, where + " rot"), scaling


@register_architecture("Vosulorn", model_type="vosulorn")
@dataclass(frozen=True)
class VosulornConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[Mapping[str, Any], ...]
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Vosulorn"

    @classmethod
    def from_dict(cls, d):
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' should be a non-empty list")
        emb = d.get("embedding")
        cfg = cls(vocab=require(d, "vocab", int), width=require(d, "width", int),
                  eps=require(_sub(d, "norm", "config.json"), "eps", float, "config.json norm"),
                  embedding_scale=optional(emb, "scale", float, 1.0, "config.json embedding") if isinstance(emb, Mapping) else 1.0,
                  layers=tuple(layers), max_positions=optional(d, "max_positions", int, DEFAULT_MAX_POSITIONS))
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.max_positions <= 0 or not cfg.eps > 0:
            raise ConfigError("config.json: vocab, width, max_positions and norm.eps must be positive")
        cfg.plan()     # every layer's keys are read and checked here
        return cfg

    def to_dict(self):
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "embedding": {"scale": self.embedding_scale}, "layers": [dict(l) for l in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ------------------------------------------------------------------ mixers
    def _delta(self, m, where):
        return PartSpec("gated_delta", {
            "hidden_size": self.width, "heads": require(m, "heads", int, where), "kv_heads": optional(m, "kv_heads", int, None, where) or require(m, "heads", int, where),
            "head_dim": require(m, "dim", int, where), "v_head_dim": optional(m, "vdim", int, None, where) or require(m, "dim", int, where),
            "conv": require(m, "conv", int, where), "eps": self.eps,
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "conv": ".conv", "b": "mix.b", "a": "mix.a", "A_log": "mix.A_log",
                      "dt_bias": "mix.dt_bias", "g": "mix.g", "norm": "mix.norm", "o": "mix.o"}})

    def _attention(self, m, where):
        dims, base, scaling = _rotation(m, where)
        mask = m.get("mask")
        if mask is not None and not isinstance(mask, Mapping):
            raise ConfigError(f"{where}: key 'mask' should be an object")
        heads, dim = require(m, "heads", int, where), require(m, "dim", int, where)
        return PartSpec("masked_attention", {
            "hidden_size": self.width, "num_heads": heads, "num_kv_heads": optional(m, "kv_heads", int, None, where) or heads,
            "head_dim": dim, "v_head_dim": optional(m, "vdim", int, None, where) or dim, "scale": require(m, "scale", float, where),
            "rot_dims": dims, "rot_base": base, "rot_scaling": scaling, "rot_pairs": "interleaved", "bias": True,
            "mask": {"kind": "chunk", "size": require(mask, "size", int, where + " mask")} if mask is not None else None,
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "bias": ".b", "sink": "mix.sink"}})

    def _latent(self, i, m, where):
        dims, base, scaling = _rotation(m, where)
        rot_dim = require(m, "rot_dim", int, where)
        if dims != rot_dim:
            raise ConfigError(f"{where}: rot.dims {dims} differs from rot_dim {rot_dim}: the rotated part of a head is rotated whole")
        kv_from = optional(m, "kv_from", int, None, where)
        spec = {"hidden_size": self.width, "num_heads": require(m, "heads", int, where), "head_dim": require(m, "dim", int, where),
                "rot_dim": rot_dim, "v_head_dim": require(m, "vdim", int, where), "kv_rank": require(m, "kv_rank", int, where),
                "scale": require(m, "scale", float, where), "eps": self.eps, "rot_base": base, "rot_scaling": scaling,
                "reads_cache": kv_from is not None,
                "names": {"q": "mix.q", "dkv": "mix.dkv", "dkv_norm": "mix.dkv.norm", "uk": "mix.uk", "uv": "mix.uv", "o": "mix.o"}}
        if kv_from is not None:
            src = self.layers[kv_from] if 0 <= kv_from < i and isinstance(self.layers[kv_from], Mapping) else None
            sm = src.get("mixer") if src is not None and src.get("type") == "latent_attention" else None
            if not isinstance(sm, Mapping) or sm.get("kv_from") is not None:
                raise ConfigError(f"{where}: kv_from {kv_from} should name an earlier latent_attention layer that keeps its own latent")
            if (sm.get("kv_rank"), sm.get("rot_dim"), sm.get("rot")) != (m.get("kv_rank"), m.get("rot_dim"), m.get("rot")):
                raise ConfigError(f"{where}: layer {kv_from}'s kv_rank, rot_dim and rotation differ from this layer's")
        return PartSpec("latent_attention", spec), kv_from

    def _layer(self, i, layer):
        where = f"config.json layers[{i}]"
        if not isinstance(layer, Mapping):
            raise ConfigError(f"{where} should be an object")
        kind = require(layer, "type", str, where)
        m = _sub(layer, "mixer", where)
        reads = None
        if kind == "delta":
            mixer = self._delta(m, where + " mixer")
        elif kind == "attention":
            mixer = self._attention(m, where + " mixer")
        elif kind == "latent_attention":
            mixer, reads = self._latent(i, m, where + " mixer")
        else:
            raise ConfigError(f"{where}: a layer of type '{kind}' is not part of this architecture (delta, attention, latent_attention)")
        norm = {"dim": self.width, "eps": self.eps}
        mlp, ffn, ffn_norm = layer.get("mlp"), None, None
        if mlp is not None:
            if not isinstance(mlp, Mapping):
                raise ConfigError(f"{where}: key 'mlp' should be an object or null")
            mk = require(mlp, "kind", str, where + " mlp")
            if mk != "moe":
                raise ConfigError(f"{where} mlp: kind '{mk}' is not part of this architecture (moe)")
            router = _sub(mlp, "router", where + " mlp")
            ffn = PartSpec("moe", {"hidden_size": self.width, "intermediate_size": require(_sub(mlp, "expert", where + " mlp"), "ff", int, where + " mlp expert"),
                                   "experts": require(router, "experts", int, where + " mlp router"), "top": require(router, "top", int, where + " mlp router"),
                                   "names": {"expert": "mlp.e", "gate": "gate", "up": "up", "down": "down", "router": "mlp.router",
                                             "router_bias": "mlp.router.b"}})
            ffn_norm = PartSpec("rmsnorm", {**norm, "name": "norm2"})
        spec = LayerSpec(prefix=f"l{i}.", block="prenorm", mixer=mixer, mixer_norm=PartSpec("rmsnorm", {**norm, "name": "norm1"}),
                         ffn=ffn, ffn_norm=ffn_norm)
        return spec, reads

    def plan(self) -> ModelPlan:
        built = [self._layer(i, l) for i, l in enumerate(self.layers)]
        norm = {"dim": self.width, "eps": self.eps}
        return ModelPlan(
            hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "dim": self.width, "name": "embed", "scale": self.embedding_scale}),
            layers=tuple(spec for spec, _ in built),
            schedule=tuple(ScheduleEntry(i, reads) for i, (_, reads) in enumerate(built)),     # (a layer runs once: entry i is layer i)
            final_norm=PartSpec("rmsnorm", {**norm, "name": "final.norm"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "dim": self.width, "tied_to": None, "name": "head"}),
            stop_token_ids=(), bos_token_id=None,
        ).validate()
