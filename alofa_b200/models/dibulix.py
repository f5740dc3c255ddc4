"""Dibulix: a decoder whose layers, listed one by one in config.json, are
pre-norm sublayers (a mixer, then optionally a dense feed-forward) over several
copies of the residual stream ("hyper-connections": a sublayer reads a weighted
sum of the copies, and its output is written into all of them while they are
mixed among themselves; the model's output is their sum).  A layer's mixer is
one of

* ``parallel``: softmax attention (grouped heads, biases, rotation of
  neighbouring pairs on the first dimensions of each head, a sliding window, one
  added to the softmax's denominator) beside a minGRU recurrence, their outputs
  added with one factor each;
* ``channel_delta``: the gated delta rule with one decay per head and key
  channel, short convolutions on q, k and v, a gated norm on the output;
* ``latent_attention``: attention over a cached latent with one rotated key part
  shared by the heads (halves paired, YaRN-scaled frequencies), a sliding
  window, and a sigmoid gate per head on the output.

The feed-forward is ``W_down relu(W_up x)^2``; the head is the embedding table
and the logits are multiplied by ``logit_scale``.  This file only reads the
architecture's config keys and describes the model as a
:class:`~alofa_b200.config.spec.ModelSpec`; the parts it names live in
:mod:`alofa_b200.parts` and know nothing about Dibulix.

config.json keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``,
``streams`` (absent: one plain residual stream), ``logit_scale``,
``layers[i].type``, ``layers[i].mixer`` (parallel: ``left`` = ``heads, kv_heads,
dim, vdim, scale, rot.{base, dims}, mask.size``, ``right`` = ``width``,
``left_scale``, ``right_scale``; channel_delta: ``heads, kv_heads, dim, vdim,
conv``; latent_attention: ``heads, dim, rot_dim, vdim, kv_rank, scale,
rot.{base, dims, scaling.{factor, original, fast, slow}}, mask.size``) and
``layers[i].mlp`` (null or ``{kind: dense, ff}``).  Tensor names: ``embed``,
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.hc1.*``,
``l<i>.hc2.*``, ``final.norm``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ..config.json_reader import Keys
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..errors import AlofaError

NAME = "Dibulix"
MAX_POSITION = 1 << 24  # positions are fp32 in the kernels that turn: whole numbers are exact up to here
SINK_SCORE = 0.0  # "one added to the denominator": a sink whose score is 0


@dataclass
class Rotary:
    base: float
    dims: int
    scaling: Optional[dict] = None  # factor, original, fast, slow


@dataclass
class WindowedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[Rotary] = None
    window: Optional[int] = None


@dataclass
class ParallelConfig:
    left: WindowedAttentionConfig
    right_width: int
    left_scale: float
    right_scale: float


@dataclass
class DeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass
class LatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: Optional[Rotary] = None
    window: Optional[int] = None


@dataclass
class DibulixLayer:
    type: str
    mixer: object
    ff: Optional[int]  # the dense feed-forward's inner size, None for no feed-forward


@dataclass
class DibulixConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float = 1.0
    streams: Optional[int] = None  # None: one plain residual stream, no connection weights
    layers: list = field(default_factory=list)

    def validate(self, origin: str = "") -> None:
        def need(ok, what, detail):
            if not ok:
                raise AlofaError("parse", what, f"{detail} config={origin}")

        need(self.vocab > 0 and self.width > 0, "vocab and width must be positive", f"vocab={self.vocab} width={self.width}")
        need(self.eps > 0, "norm.eps must be positive", f"eps={self.eps}")
        need(self.streams is None or 1 <= self.streams <= 8, "streams must lie in [1, 8]", f"streams={self.streams}")
        need(len(self.layers) > 0, "layers must not be empty", "layers=[]")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            where = f"layers[{i}].mixer={m}"
            if layer.type == "parallel":
                a = m.left
                need(min(a.heads, a.kv_heads, a.dim, a.vdim) > 0 and a.heads % a.kv_heads == 0, "left: kv_heads must divide heads", where)
                need(a.rot is None or (a.rot.dims % 2 == 0 and 0 <= a.rot.dims <= a.dim and a.rot.base > 0), "left: rot.dims must be even and at most dim", where)
                need(a.window is None or a.window > 0, "left: mask.size must be positive", where)
                need(m.right_width > 0, "right: width must be positive", where)
            elif layer.type == "channel_delta":
                need(min(m.heads, m.kv_heads, m.dim, m.vdim, m.conv) > 0 and m.heads % m.kv_heads == 0, "kv_heads must divide heads, sizes must be positive", where)
            else:
                need(min(m.heads, m.vdim, m.kv_rank) > 0 and m.dim >= 0 and m.rot_dim >= 0 and m.dim + m.rot_dim > 0, "sizes must be positive", where)
                need(m.rot is None or (m.rot.dims % 2 == 0 and 0 <= m.rot.dims <= m.rot_dim and m.rot.base > 0), "rot.dims must be even and at most rot_dim", where)
                need(m.window is None or m.window > 0, "mask.size must be positive", where)
            need(layer.ff is None or layer.ff > 0, "mlp.ff must be positive", f"layers[{i}].mlp.ff={layer.ff}")


def _object(obj: dict, key: str, origin: str) -> dict:
    value = obj.get(key)
    if not isinstance(value, dict):
        raise AlofaError("parse", "config key must be an object", f"key={key} config={origin}")
    return value


def _read_rot(obj: dict, origin: str) -> Optional[Rotary]:
    rot = obj.get("rot")
    if not isinstance(rot, dict):
        return None
    k = Keys(rot, origin)
    scaling = None
    if isinstance(rot.get("scaling"), dict):
        sk = Keys(rot["scaling"], origin)
        scaling = {name: sk.number(name) for name in ("factor", "original", "fast", "slow")}
    return Rotary(k.number("base"), k.integer("dims"), scaling)


def _read_window(obj: dict, origin: str) -> Optional[int]:
    mask = obj.get("mask")
    return Keys(mask, origin).integer("size") if isinstance(mask, dict) else None


def _read_mixer(kind: str, obj: dict, origin: str):
    if kind == "parallel":
        lo = _object(obj, "left", origin)
        k = Keys(lo, origin)
        left = WindowedAttentionConfig(k.integer("heads"), k.integer("kv_heads"), k.integer("dim"), k.integer("vdim"), k.number("scale"), _read_rot(lo, origin),
                                       _read_window(lo, origin))
        top = Keys(obj, origin)
        return ParallelConfig(left, Keys(_object(obj, "right", origin), origin).integer("width"), top.number("left_scale"), top.number("right_scale"))
    if kind == "channel_delta":
        k = Keys(obj, origin)
        return DeltaConfig(k.integer("heads"), k.integer("kv_heads"), k.integer("dim"), k.integer("vdim"), k.integer("conv"))
    if kind == "latent_attention":
        k = Keys(obj, origin)
        return LatentConfig(k.integer("heads"), k.integer("dim"), k.integer("rot_dim"), k.integer("vdim"), k.integer("kv_rank"), k.number("scale"), _read_rot(obj, origin),
                            _read_window(obj, origin))
    raise AlofaError("parse", "unknown layer type", f"type={kind} config={origin}")


def _read_ff(obj, origin: str) -> Optional[int]:
    if obj is None:
        return None
    if not isinstance(obj, dict):
        raise AlofaError("parse", "mlp must be an object or null", f"config={origin}")
    k = Keys(obj, origin)
    if k.string("kind") != "dense":
        raise AlofaError("parse", "unknown mlp kind", f"kind={obj.get('kind')} config={origin}")
    return k.integer("ff")


def read_config(obj: dict, origin: str) -> DibulixConfig:
    k = Keys(obj, origin)
    layers = obj.get("layers")
    if not isinstance(layers, list):
        raise AlofaError("parse", "config key must be a list", f"key=layers config={origin}")
    cfg = DibulixConfig(vocab=k.integer("vocab"), width=k.integer("width"), eps=Keys(_object(obj, "norm", origin), origin).number("eps"),
                        logit_scale=k.number("logit_scale") if "logit_scale" in obj else 1.0, streams=k.integer("streams") if "streams" in obj else None)
    for i, entry in enumerate(layers):
        if not isinstance(entry, dict):
            raise AlofaError("parse", "a layer must be an object", f"layers[{i}] config={origin}")
        kind = Keys(entry, origin).string("type")
        cfg.layers.append(DibulixLayer(kind, _read_mixer(kind, _object(entry, "mixer", origin), origin), _read_ff(entry.get("mlp"), origin)))
    cfg.validate(origin)
    return cfg


def _rot_json(rot: Optional[Rotary]) -> dict:
    if rot is None:
        return {}
    out = {"base": rot.base, "dims": rot.dims}
    if rot.scaling:
        out["scaling"] = dict(rot.scaling)
    return {"rot": out}


def to_json(cfg: DibulixConfig) -> dict:
    layers = []
    for layer in cfg.layers:
        m = layer.mixer
        if layer.type == "parallel":
            a = m.left
            left = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale, **_rot_json(a.rot)}
            if a.window is not None:
                left["mask"] = {"size": a.window}
            mixer = {"left": left, "right": {"width": m.right_width}, "left_scale": m.left_scale, "right_scale": m.right_scale}
        elif layer.type == "channel_delta":
            mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
        else:
            mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale, **_rot_json(m.rot)}
            if m.window is not None:
                mixer["mask"] = {"size": m.window}
        layers.append({"type": layer.type, "mixer": mixer, "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}})
    out = {"architecture": NAME, "vocab": cfg.vocab, "width": cfg.width, "norm": {"eps": cfg.eps}, "logit_scale": cfg.logit_scale, "layers": layers}
    if cfg.streams is not None:
        out["streams"] = cfg.streams
    return out


def _position(rot: Optional[Rotary], layout: str) -> PartSpec:
    if rot is None or rot.dims == 0:
        return PartSpec("rotary_interleaved", {"dims": 0, "base": 1.0})
    return PartSpec("rotary_interleaved", {"dims": rot.dims, "base": rot.base, "layout": layout, "scaling": rot.scaling})


def build_spec(cfg: DibulixConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "parallel":
            a = m.left
            attention = PartSpec("normed_attention", {"hidden_size": width, "heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale,
                                                      "bias": True, "sink": SINK_SCORE, "window": a.window,
                                                      "position": _position(a.rot, "pairs") if a.rot is not None and a.rot.dims else None}, prefix=p + "mix.left.")
            gru = PartSpec("min_gru", {"hidden_size": width, "width": m.right_width}, prefix=p + "mix.right.")
            mixer = PartSpec("side_by_side", {"hidden_size": width, "eps": eps, "names": ["left", "right"], "branches": [attention, gru], "combine": "weighted",
                                              "scales": [m.left_scale, m.right_scale]}, prefix=p + "mix.")
        elif layer.type == "channel_delta":
            mixer = PartSpec("gated_delta", {"hidden_size": width, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv, "eps": eps},
                             prefix=p + "mix.")
        else:
            mixer = PartSpec("latent_attention", {"hidden_size": width, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                                                  "q_rank": 0, "gate": True, "scale": m.scale, "eps": eps, "sink": False, "window": m.window,
                                                  "position": _position(m.rot, "halves")}, prefix=p + "mix.")
        block = {"hidden_size": width, "streams": cfg.streams or 1, "connections": cfg.streams is not None, "mixer": mixer,
                 "mixer_norm": PartSpec("rmsnorm", {"size": width, "eps": eps, "weight_name": "norm1"}, prefix=p), "feed_forward": None}
        if layer.ff is not None:
            block["feed_forward"] = PartSpec("mlp", {"hidden_size": width, "intermediate_size": layer.ff, "activation": "relu_squared", "bias": False}, prefix=p + "mlp.")
            block["feed_forward_norm"] = PartSpec("rmsnorm", {"size": width, "eps": eps, "weight_name": "norm2"}, prefix=p)
        layers.append(LayerSpec(PartSpec("hyper_residual", block, prefix=p)))
    spec = ModelSpec(
        architecture=NAME, hidden_size=width, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": width, "weight_name": "embed"}),
        layers=layers, run=[RunEntry(i) for i in range(len(layers))],
        final_norm=PartSpec("rmsnorm", {"size": width, "eps": eps, "weight_name": "final.norm"}),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": width, "tied_to": "embed", "weight_name": "embed", "scale": cfg.logit_scale}),
    )
    spec.validate()
    return spec


register_architecture(Architecture(NAME, read_config, build_spec, to_json), replace=True)
