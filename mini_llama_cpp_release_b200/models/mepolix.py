"""Mepolix: a decoder whose layers mix tokens in one of two ways, listed layer by layer in
config.json, with the norm on each branch's output.

    x = E[token]
    per layer:  x ← x + LN(mixer(x));  x ← x + LN(ff(x))         (LN: layer norm with a gain, no bias; ff may be absent)
    logits = c · tanh(W_head LN(x) / c)

Layer types: "delta", the gated delta rule (`parts/recurrent.py: GatedDeltaMixer`), and "parallel", softmax
attention with a sink, per-head q/k norm and a partial, stretched rotation (`parts/attention.py: SinkAttention`)
beside a gated diagonal linear recurrence (`GatedLinearRecurrence`), the two summed with fixed factors
(`ParallelMixer`).  The feed-forward is SwiGLU.  A layer may name another layer whose tensors it uses
(`weights_of`): it then runs those weights again with a cache and state of its own, which in this library is a
second schedule entry of the same layer.

config.json (every size and constant comes from it):
    architecture, vocab, width, logit_softcap, norm.eps,
    layers[i]: type, mixer {...}, mlp {kind: "dense", ff} or null, optionally weights_of
      delta mixer:     heads, kv_heads, dim, vdim, conv
      parallel mixer:  left {heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor, original, fast, slow}}},
                       right {width, blocks, conv}, left_scale, right_scale
Tensors: embed, head, final.norm, l<i>.norm1, l<i>.norm2, l<i>.mix.<...>, l<i>.mlp.{gate,up,down}.
The model names no largest position; sequences are bounded by the cache alone.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import ConfigError, ModelConfig, as_int
from ..config.registry import register_architecture
from ..config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

NO_POSITION_LIMIT = 2 ** 31 - 1


def _need(d: Dict[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"missing config key: {where}.{key}")
    return d[key]


def _number(d: Dict[str, Any], key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise ConfigError(f"config key {where}.{key} must be a finite number, got {v!r}")
    return float(v)


def _count(d: Dict[str, Any], key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or v < 1:
        raise ConfigError(f"config key {where}.{key} must be a positive integer, got {v!r}")
    return int(v)


@dataclass(frozen=True, kw_only=True)
class MepolixConfig(ModelConfig):
    hidden_size: int
    norm_eps: float
    logit_softcap: Optional[float]
    layers: Tuple[Dict[str, Any], ...]

    KEYS = ("vocab", "width", "norm", "logit_softcap", "layers")

    @classmethod
    def parse(cls, raw: Dict[str, Any]) -> "MepolixConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ConfigError(f"missing config key: {key}")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config key layers must be a list with at least one layer")
        shared = dict(cls.shared_fields({**raw, "vocab_size": raw["vocab"],
                                         "max_position_embeddings": raw.get("max_position_embeddings", NO_POSITION_LIMIT)}))
        cap = raw.get("logit_softcap")
        cfg = cls(**shared, hidden_size=as_int(raw, "width"), norm_eps=_number(raw["norm"], "eps", "norm"),
                  logit_softcap=float(cap) if cap else None, layers=tuple(raw["layers"]),
                  extra={k: v for k, v in raw.items() if k not in cls.SHARED_KEYS and k not in cls.KEYS})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        super().validate()
        if self.hidden_size <= 0:
            raise ConfigError(f"width must be positive, got {self.hidden_size}")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError(f"logit_softcap must be positive, got {self.logit_softcap}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in ("delta", "parallel"):
                raise ConfigError(f"{where}.type must be \"delta\" or \"parallel\", got {kind!r}")
            _need(layer, "mixer", where)
            src = layer.get("weights_of")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(self.layers) or src == i:
                    raise ConfigError(f"{where}.weights_of must name another layer, got {src!r}")
                if self.layers[src].get("weights_of") is not None:
                    raise ConfigError(f"{where}.weights_of names layer {src}, which has no tensors of its own")
                if self.layers[src].get("type") != kind:
                    raise ConfigError(f"{where} uses the weights of layer {src}, which is of another type")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not supported: dense only")

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps}, "logit_softcap": self.logit_softcap, "layers": [dict(l) for l in self.layers]}
        if self.max_position_embeddings != NO_POSITION_LIMIT:
            d["max_position_embeddings"] = self.max_position_embeddings
        d["torch_dtype"] = self.torch_dtype
        for key in ("bos_token_id", "eos_token_id"):
            v = getattr(self, key)
            if v is not None:
                d[key] = list(v) if isinstance(v, tuple) and len(v) > 1 else (v[0] if isinstance(v, tuple) else v)
        d.update(self.extra)
        return d


def _delta_mixer(c: MepolixConfig, m: Dict[str, Any], where: str) -> PartSpec:
    return PartSpec("mixer", "gated_delta", dict(
        hidden_size=c.hidden_size, num_heads=_count(m, "heads", where), num_kv_heads=_count(m, "kv_heads", where),
        head_dim=_count(m, "dim", where), v_head_dim=_count(m, "vdim", where), conv=_count(m, "conv", where),
        norm_eps=c.norm_eps))


def _parallel_mixer(c: MepolixConfig, m: Dict[str, Any], where: str) -> PartSpec:
    left, right = _need(m, "left", where), _need(m, "right", where)
    rot = _need(left, "rot", where + ".left")
    rope = PartSpec("position", "rope_partial", dict(dims=int(_need(rot, "dims", where + ".left.rot")),
                                                     base=_number(rot, "base", where + ".left.rot"),
                                                     scaling=rot.get("scaling")))
    attn = PartSpec("mixer", "sink_attention", dict(
        hidden_size=c.hidden_size, num_heads=_count(left, "heads", where + ".left"),
        num_kv_heads=_count(left, "kv_heads", where + ".left"), head_dim=_count(left, "dim", where + ".left"),
        v_head_dim=_count(left, "vdim", where + ".left"), scale=_number(left, "scale", where + ".left"),
        norm_eps=c.norm_eps, position=rope, value_scale=_number(m, "left_scale", where)))
    rec = PartSpec("mixer", "gated_linear_recurrence", dict(
        hidden_size=c.hidden_size, width=_count(right, "width", where + ".right"),
        blocks=_count(right, "blocks", where + ".right"), conv=_count(right, "conv", where + ".right"),
        out_scale=_number(m, "right_scale", where)))
    return PartSpec("mixer", "parallel", dict(left=attn, right=rec))


@register_architecture("Mepolix", config_class=MepolixConfig)
def mepolix(config: MepolixConfig) -> ModelSpec:
    c = config
    norm = lambda tensor: PartSpec("norm", "layernorm", dict(size=c.hidden_size, eps=c.norm_eps, tensor=tensor))
    layers: List[LayerSpec] = []
    index_of: Dict[int, int] = {}                        # the config's layer number → its place among the layers with tensors
    schedule: List[ScheduleEntry] = []
    for i, layer in enumerate(c.layers):
        if layer.get("weights_of") is not None:
            continue
        where = f"layers[{i}].mixer"
        mixer = _delta_mixer(c, layer["mixer"], where) if layer["type"] == "delta" else _parallel_mixer(c, layer["mixer"], where)
        params: Dict[str, Any] = dict(mixer=mixer, mixer_norm=norm("norm1"), names={"mixer": "mix.", "mixer_norm": "",
                                                                                 "feed_forward": "mlp.", "feed_forward_norm": ""})
        if layer.get("mlp") is not None:
            params["feed_forward"] = PartSpec("feed_forward", "swiglu", dict(
                hidden_size=c.hidden_size, intermediate_size=_count(layer["mlp"], "ff", f"layers[{i}].mlp"),
                names={"gate": "gate", "up": "up", "down": "down"}))
            params["feed_forward_norm"] = norm("norm2")
        index_of[i] = len(layers)
        layers.append(LayerSpec(f"l{i}.", PartSpec("block", "branch_norm", params)))
    for i, layer in enumerate(c.layers):
        src = layer.get("weights_of")
        schedule.append(ScheduleEntry(layer=index_of[i if src is None else src]))
    return ModelSpec(
        config=c,
        embedding=PartSpec("embedding", "token_embedding", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size, tensor="embed")),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("norm"),
        head=PartSpec("head", "linear_head", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size, tensor="head",
                                                  softcap=c.logit_softcap)),
        names={"embedding": "", "final_norm": "final.", "head": ""},
    )
