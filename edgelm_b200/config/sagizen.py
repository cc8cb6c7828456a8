"""The Sagizen decoder's configuration, from its own config.json keys.

config.json: `architecture` "Sagizen", `vocab`, `width`, `norm.eps`, and `layers`, a list with one entry per layer:
`type` ("mamba2" or "parallel"), `mixer` (the mixer's sizes and constants) and `mlp` ({"kind": "dense", "ff": n} or
null for a layer without a feed-forward).  Optional: `max_positions` (the longest sequence; the design itself has no
bound, since its rotation needs no table).  Tensors: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.shift`,
`l<i>.mix.*`, `l<i>.mlp.{gate,up,down}`, `final.norm`, `head`.

Every layer norms its sublayers' OUTPUTS (x += norm1(mixer(h)); x += norm2(ff(x))) and blends the mixer's input with
the previous token's (token shift).  A "mamba2" layer has the selective state-space mixer; a "parallel" layer has two
mixers side by side on the same input, whose results are summed with the two scales of the configuration: `left`, a
grouped-query attention with biases, partly rotated heads with linearly scaled positions, unit-norm queries and keys,
a sliding window and pooled blocks behind it; `right`, a time mix with a matrix-valued state and a per-token decay.
"""
from dataclasses import dataclass
from typing import Any, Mapping, Tuple

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, ScheduleEntry, coerce, optional, require
from .registry import register_architecture

DEFAULT_MAX_POSITIONS = 1 << 20


def _sub(d, key, where):
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where}: key '{key}' should be an object, found {v!r}")
    return v


@register_architecture("Sagizen", model_type="sagizen")
@dataclass(frozen=True)
class SagizenConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[Mapping[str, Any], ...]
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Sagizen"

    @classmethod
    def from_dict(cls, d):
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' should be a non-empty list")
        cfg = cls(vocab=require(d, "vocab", int), width=require(d, "width", int), eps=require(_sub(d, "norm", "config.json"), "eps", float, "config.json norm"),
                  layers=tuple(layers), max_positions=optional(d, "max_positions", int, DEFAULT_MAX_POSITIONS))
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.max_positions <= 0 or not cfg.eps > 0:
            raise ConfigError("config.json: vocab, width, max_positions and norm.eps must be positive")
        cfg.plan()     # every layer's keys are read and checked here
        return cfg

    def to_dict(self):
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "layers": [dict(l) for l in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ------------------------------------------------------------------ mixers
    def _mamba2(self, m, where):
        return PartSpec("mamba2", {
            "hidden_size": self.width, "heads": require(m, "heads", int, where), "head_dim": require(m, "vdim", int, where),
            "state": require(m, "state", int, where), "groups": require(m, "groups", int, where), "conv": require(m, "conv", int, where),
            "norm_groups": require(m, "norm_groups", int, where), "eps": self.eps,
            "names": {"in": "mix.in", "conv": "mix.conv", "conv_bias": "mix.conv.b", "dt_bias": "mix.dt_bias", "A_log": "mix.A_log",
                      "D": "mix.D", "norm": "mix.norm", "out": "mix.o"}})

    def _left(self, m, where):
        mask, rot = _sub(m, "mask", where), m.get("rot")
        spec = {"hidden_size": self.width, "num_heads": require(m, "heads", int, where), "num_kv_heads": require(m, "kv_heads", int, where),
                "head_dim": require(m, "dim", int, where), "v_head_dim": require(m, "vdim", int, where),
                "window": require(mask, "size", int, where + " mask"), "pool": optional(mask, "pool", int, None, where + " mask"),
                "scale": require(m, "scale", float, where), "unit_norm": True, "eps": self.eps, "bias": True,
                "names": {"q": "mix.left.q", "k": "mix.left.k", "v": "mix.left.v", "o": "mix.left.o", "bias": ".b"}}
        if rot is not None:
            if not isinstance(rot, Mapping):
                raise ConfigError(f"{where}: key 'rot' should be an object")
            scaling = rot.get("scaling")
            spec.update({"rot_dims": require(rot, "dims", int, where + " rot"), "rot_base": require(rot, "base", float, where + " rot"),
                         "rot_scaling": require(scaling, "factor", float, where + " rot scaling") if isinstance(scaling, Mapping) else 1.0})
        return PartSpec("pooled_window_attention", spec)

    def _right(self, m, where, rank):
        return PartSpec("decay_timemix", {
            "hidden_size": self.width, "heads": require(m, "heads", int, where), "head_dim": require(m, "dim", int, where),
            "decay_rank": rank, "eps": self.eps,
            "names": {"mu": "mix.right.mu.", "r": "mix.right.r", "k": "mix.right.k", "v": "mix.right.v", "g": "mix.right.g",
                      "w1": "mix.right.w1", "w2": "mix.right.w2", "w0": "mix.right.w0", "bonus": "mix.right.u",
                      "norm": "mix.right.norm", "out": "mix.right.o"}})

    def _layer(self, i, layer, decay_rank):
        where = f"config.json layers[{i}]"
        if not isinstance(layer, Mapping):
            raise ConfigError(f"{where} should be an object")
        kind = require(layer, "type", str, where)
        m = _sub(layer, "mixer", where)
        if kind == "mamba2":
            mixer = self._mamba2(m, where + " mixer")
        elif kind == "parallel":
            mixer = PartSpec("parallel", {
                "hidden_size": self.width, "left": self._left(_sub(m, "left", where + " mixer"), where + " mixer left"),
                "right": self._right(_sub(m, "right", where + " mixer"), where + " mixer right", decay_rank),
                "left_scale": require(m, "left_scale", float, where + " mixer"), "right_scale": require(m, "right_scale", float, where + " mixer")})
        else:
            raise ConfigError(f"{where}: a layer of type '{kind}' is not part of this architecture (mamba2, parallel)")
        norm = {"dim": self.width, "eps": self.eps}
        mlp, ffn, ffn_norm = layer.get("mlp"), None, None
        if mlp is not None:
            if not isinstance(mlp, Mapping):
                raise ConfigError(f"{where}: key 'mlp' should be an object or null")
            mk = require(mlp, "kind", str, where + " mlp")
            if mk != "dense":
                raise ConfigError(f"{where} mlp: kind '{mk}' is not part of this architecture (dense)")
            ffn = PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": require(mlp, "ff", int, where + " mlp"),
                                      "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
            ffn_norm = PartSpec("rmsnorm", {**norm, "name": "norm2"})
        return LayerSpec(prefix=f"l{i}.", block="sublayer_norm", mixer=mixer, mixer_norm=PartSpec("rmsnorm", {**norm, "name": "norm1"}),
                         ffn=ffn, ffn_norm=ffn_norm, options={"shift": "shift"})

    def with_decay_ranks(self, ranks):
        """The same configuration with the rank of each time mix's decay projection (a size that only the tensors'
        shapes give): `ranks` maps a layer's index to it."""
        layers = []
        for i, l in enumerate(self.layers):
            if i in ranks:
                l = dict(l)
                l["decay_rank"] = int(ranks[i])
            layers.append(l)
        import dataclasses
        return dataclasses.replace(self, layers=tuple(layers))

    def shape_given_sizes(self, shapes):
        """Sizes that config.json does not hold and the stored tensors' shapes give: the rank of a time mix's decay
        projection, from `l<i>.mix.right.w1` [rank, width].  Returns the completed configuration."""
        ranks = {}
        for i, l in enumerate(self.layers):
            name = f"l{i}.mix.right.w1"
            if isinstance(l, Mapping) and l.get("type") == "parallel" and name in shapes and len(shapes[name]) == 2:
                ranks[i] = int(shapes[name][0])
        return self.with_decay_ranks(ranks) if ranks else self

    DEFAULT_DECAY_RANK = 32     # (used only where neither the configuration nor a stored tensor gives it: a plan without weights)

    def plan(self) -> ModelPlan:
        layers = tuple(self._layer(i, l, coerce(l.get("decay_rank", self.DEFAULT_DECAY_RANK), "decay_rank", int) if isinstance(l, Mapping) else 0)
                       for i, l in enumerate(self.layers))
        norm = {"dim": self.width, "eps": self.eps}
        return ModelPlan(
            hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "dim": self.width, "name": "embed"}),
            layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
            final_norm=PartSpec("rmsnorm", {**norm, "name": "final.norm"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "dim": self.width, "tied_to": None, "name": "head"}),
            stop_token_ids=(), bos_token_id=None,
        ).validate()
