"""Kebesun: a decoder whose config.json lists its layers, each one norm feeding a mixer and a feed-forward side by side,
with a run of layers that is walked several times.

    e = E[token];  x = e
    layers [start, stop) are walked `times` times in a row with the same weights (each walk with a cache and state of its
    own); before every walk  x <- W_in [x ; e]
    per layer:  h = N(x);  x <- x + s1 * mixer(h) + s2 * ff(h)         N: RMS norm with gain 1 + w; s1, s2 per channel
    logits = W_head N_f(x)

Mixers: "attention" (grouped-query attention over a sliding window that also keeps the sequence's first tokens,
rotate-half rotation with linearly stretched positions: `parts/attention.py: SinkAttention` without its norm and sink),
"gla" (gated linear attention, `parts/recurrent.py: GatedLinearAttention`) and "latent_attention" (keys and values
expanded from a cached low-rank latent, YaRN-stretched rotation: `parts/attention.py: LatentAttention`).
Feed-forwards: dense SwiGLU, or a mixture of SwiGLU experts (`parts/feed_forward.py: MixtureOfExperts`), or none.

config.json (every size and constant comes from it):
    architecture, vocab, width, norm.eps, loop {start, stop, times} (optional),
    layers[i]: type, mixer {...}, mlp {kind: "dense", ff} | {kind: "moe", expert {ff}, router {experts, top}} | null
      attention:         heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor}}, mask {size, keep_first}
      gla:               heads, dim, vdim, tau
      latent_attention:  heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims, scaling {factor, original, fast, slow}}
Tensors: embed, head, final.norm, loop.in, l<i>.norm1, l<i>.ls1, l<i>.ls2, l<i>.mix.<...>, l<i>.mlp.<...>.
The model names no largest position; sequences are bounded by the cache alone.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import ConfigError, ModelConfig, as_int
from ..config.registry import register_architecture
from ..config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .mepolix import NO_POSITION_LIMIT, _count, _need, _number

MIXERS = ("attention", "gla", "latent_attention")


@dataclass(frozen=True, kw_only=True)
class KebesunConfig(ModelConfig):
    hidden_size: int
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]
    loop: Optional[Tuple[int, int, int]]            # (start, stop, times)

    KEYS = ("vocab", "width", "norm", "layers", "loop")

    @classmethod
    def parse(cls, raw: Dict[str, Any]) -> "KebesunConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ConfigError(f"missing config key: {key}")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config key layers must be a list with at least one layer")
        shared = dict(cls.shared_fields({**raw, "vocab_size": raw["vocab"],
                                         "max_position_embeddings": raw.get("max_position_embeddings", NO_POSITION_LIMIT)}))
        loop = raw.get("loop")
        if loop is not None:
            loop = (as_int(loop, "start"), as_int(loop, "stop"), as_int(loop, "times"))
        cfg = cls(**shared, hidden_size=as_int(raw, "width"), norm_eps=_number(raw["norm"], "eps", "norm"),
                  layers=tuple(raw["layers"]), loop=loop,
                  extra={k: v for k, v in raw.items() if k not in cls.SHARED_KEYS and k not in cls.KEYS})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        super().validate()
        if self.hidden_size <= 0:
            raise ConfigError(f"width must be positive, got {self.hidden_size}")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        n = len(self.layers)
        if self.loop is not None:
            start, stop, times = self.loop
            if not 0 <= start <= stop <= n or times < 1:
                raise ConfigError(f"loop must name layers start <= stop within 0..{n} and times >= 1, got {self.loop}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"{where}.type must be one of {', '.join(MIXERS)}; got {kind!r}")
            _need(layer, "mixer", where)
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") not in ("dense", "moe"):
                raise ConfigError(f"{where}.mlp.kind must be \"dense\" or \"moe\", got {mlp.get('kind')!r}")

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps}, "layers": [dict(l) for l in self.layers]}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.max_position_embeddings != NO_POSITION_LIMIT:
            d["max_position_embeddings"] = self.max_position_embeddings
        d["torch_dtype"] = self.torch_dtype
        for key in ("bos_token_id", "eos_token_id"):
            v = getattr(self, key)
            if v is not None:
                d[key] = list(v) if isinstance(v, tuple) and len(v) > 1 else (v[0] if isinstance(v, tuple) else v)
        d.update(self.extra)
        return d


def _rotation(rot: Optional[Dict[str, Any]], where: str) -> PartSpec:
    if not rot:
        return PartSpec("position", "rope_partial", dict(dims=0, base=1.0, scaling=None))
    return PartSpec("position", "rope_partial", dict(dims=int(_need(rot, "dims", where)), base=_number(rot, "base", where),
                                                     scaling=rot.get("scaling")))


def _attention(c: KebesunConfig, m: Dict[str, Any], where: str) -> PartSpec:
    mask = m.get("mask") or {}
    window = int(mask["size"]) if mask.get("size") else None
    return PartSpec("mixer", "sink_attention", dict(
        hidden_size=c.hidden_size, num_heads=_count(m, "heads", where), num_kv_heads=_count(m, "kv_heads", where),
        head_dim=_count(m, "dim", where), v_head_dim=_count(m, "vdim", where), scale=_number(m, "scale", where),
        norm_eps=c.norm_eps, position=_rotation(m.get("rot"), where + ".rot"), qk_norm=False, sink=False, window=window,
        keep_first=int(mask.get("keep_first") or 0) if window else 0))


def _gla(c: KebesunConfig, m: Dict[str, Any], where: str) -> PartSpec:
    return PartSpec("mixer", "gated_linear_attention", dict(
        hidden_size=c.hidden_size, num_heads=_count(m, "heads", where), head_dim=_count(m, "dim", where),
        v_head_dim=_count(m, "vdim", where), tau=_number(m, "tau", where), norm_eps=c.norm_eps,
        decay_rank=m.get("decay_rank")))


def _latent(c: KebesunConfig, m: Dict[str, Any], where: str) -> PartSpec:
    rot_dim = int(_need(m, "rot_dim", where))
    rot = dict(m.get("rot") or {})
    if rot and int(rot.get("dims", rot_dim)) != rot_dim:
        raise ConfigError(f"{where}.rot.dims must equal rot_dim ({rot_dim}), got {rot.get('dims')}")
    return PartSpec("mixer", "latent_attention", dict(
        hidden_size=c.hidden_size, num_heads=_count(m, "heads", where), head_dim=int(_need(m, "dim", where)), rot_dim=rot_dim,
        v_head_dim=_count(m, "vdim", where), kv_rank=_count(m, "kv_rank", where), scale=_number(m, "scale", where),
        norm_eps=c.norm_eps, position=_rotation(rot if rot_dim else None, where + ".rot")))


def _feed_forward(c: KebesunConfig, mlp: Dict[str, Any], where: str) -> PartSpec:
    if mlp.get("kind", "dense") == "dense":
        return PartSpec("feed_forward", "swiglu", dict(hidden_size=c.hidden_size, intermediate_size=_count(mlp, "ff", where),
                                                       names={"gate": "gate", "up": "up", "down": "down"}))
    router, expert = _need(mlp, "router", where), _need(mlp, "expert", where)
    return PartSpec("feed_forward", "mixture", dict(
        hidden_size=c.hidden_size, intermediate_size=_count(expert, "ff", where + ".expert"),
        num_experts=_count(router, "experts", where + ".router"), top=_count(router, "top", where + ".router")))


@register_architecture("Kebesun", config_class=KebesunConfig)
def kebesun(config: KebesunConfig) -> ModelSpec:
    c = config
    norm = lambda tensor: PartSpec("norm", "rmsnorm", dict(size=c.hidden_size, eps=c.norm_eps, tensor=tensor, offset=1.0))
    builders = {"attention": _attention, "gla": _gla, "latent_attention": _latent}
    layers: List[LayerSpec] = []
    for i, layer in enumerate(c.layers):
        params: Dict[str, Any] = dict(
            mixer=builders[layer["type"]](c, layer["mixer"], f"layers[{i}].mixer"), norm=norm("norm1"), layer_scale=True,
            names={"norm": "", "mixer": "mix.", "feed_forward": "mlp.", "mixer_scale": "ls1", "feed_forward_scale": "ls2"})
        if layer.get("mlp") is not None:
            params["feed_forward"] = _feed_forward(c, layer["mlp"], f"layers[{i}].mlp")
        layers.append(LayerSpec(f"l{i}.", PartSpec("block", "parallel", params)))
    n = len(layers)
    order: List[int] = list(range(n))
    if c.loop is not None:
        start, stop, times = c.loop
        mix = n                                          # the step before each walk, as one more "layer" without a mixer
        layers.append(LayerSpec("loop.", PartSpec("block", "stream_mix", dict(size=c.hidden_size, tensor="in"))))
        if stop > start:                                 # (an empty run has no walk and no step before one; its tensor is still the file's)
            order = list(range(start)) + ([mix] + list(range(start, stop))) * times + list(range(stop, n))
    return ModelSpec(
        config=c,
        embedding=PartSpec("embedding", "token_embedding", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size, tensor="embed")),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i) for i in order),
        final_norm=norm("norm"),
        head=PartSpec("head", "linear_head", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size, tensor="head")),
        names={"embedding": "", "final_norm": "final.", "head": ""},
    )
