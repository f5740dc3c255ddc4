"""Kikerax: a decoder whose layers, listed one by one in config.json, put a
norm on the OUTPUT of each sublayer only, ``x += norm1(mixer(x)); x +=
norm2(ff(x))`` (the sublayers read the stream itself; the feed-forward may be
absent).  A layer's mixer is one of

* ``parallel``: softmax attention whose values are its keys as projected
  (weighted RMS norm of q and k per head, no rotation, queries that grow with
  the logarithm of the position, capped scores, a sigmoid gate per head on the
  output) beside a recurrent block with a real-gated linear recurrent unit,
  their outputs added with one factor each;
* ``attention``: differential attention, two softmax maps a head over the same
  values whose weighted difference is normed per head; biases, weighted RMS
  norm of q and k, neighbouring pairs turned by the position on the first
  dimensions of each map (YaRN-scaled frequencies), a mask in chunks counted
  from the sequence's start, a sigmoid gate per head.

The feed-forward is dense (``W_down gelu_tanh(W_up x)``) or a mixture of gated
experts chosen by sigmoid scores with a stored correction, among the best
groups of neighbouring experts only, plus a shared expert.  The head is the
embedding table; the logits are bounded by ``logit_softcap * tanh(. /
logit_softcap)``.  This file only reads the architecture's config keys and
describes the model as a :class:`~alofa_b200.config.spec.ModelSpec`; the parts
it names live in :mod:`alofa_b200.parts` and know nothing about Kikerax.

config.json keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``,
``logit_softcap`` (absent: none), ``layers[i].type``, ``layers[i].mixer``
(parallel: ``left`` = ``heads, kv_heads, dim, vdim, scale, softcap,
q_temp.{coef, every}``, ``right`` = ``width, blocks, conv``, ``left_scale``,
``right_scale``; attention: ``heads, kv_heads, dim, vdim, scale, diff,
rot.{base, dims, scaling.{factor, original, fast, slow}}, mask.size``) and
``layers[i].mlp`` (null, ``{kind: dense, ff}`` or ``{kind: moe, expert.ff,
router.{experts, top, scale, groups.{count, keep}}, shared.ff}``).  Keys that
switch a mechanism on may be absent (``softcap``, ``q_temp``, ``rot``,
``rot.scaling``, ``mask``, ``router.groups``, ``shared``).  Tensor names:
``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ..config.json_reader import Keys
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..errors import AlofaError

NAME = "Kikerax"
MAX_POSITION = 1 << 24  # positions are fp32 in the kernels that turn: whole numbers are exact up to here
LRU_DECAY_SCALE = 8.0  # log a = -8 * r * softplus(lam)
RENORM_EPS = 1e-20  # added to the sum the chosen experts' scores are divided by


@dataclass
class KeyedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float] = None
    q_temp: Optional[dict] = None  # coef, every


@dataclass
class RecurrentConfig:
    width: int
    blocks: int
    conv: int


@dataclass
class ParallelConfig:
    left: KeyedAttentionConfig
    right: RecurrentConfig
    left_scale: float
    right_scale: float


@dataclass
class DifferentialConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    rot: Optional[dict] = None  # base, dims, scaling (factor, original, fast, slow) or None
    chunk: Optional[int] = None


@dataclass
class FeedForwardConfig:
    kind: str  # "dense" or "moe"
    ff: int  # dense: the inner size; moe: one expert's
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0
    groups: Optional[dict] = None  # count, keep
    shared_ff: int = 0


@dataclass
class KikeraxLayer:
    type: str
    mixer: object
    mlp: Optional[FeedForwardConfig]


@dataclass
class KikeraxConfig:
    vocab: int
    width: int
    eps: float
    logit_softcap: Optional[float] = None
    layers: list = field(default_factory=list)

    def validate(self, origin: str = "") -> None:
        def need(ok, what, detail):
            if not ok:
                raise AlofaError("parse", what, f"{detail} config={origin}")

        need(self.vocab > 0 and self.width > 0, "vocab and width must be positive", f"vocab={self.vocab} width={self.width}")
        need(self.eps > 0, "norm.eps must be positive", f"eps={self.eps}")
        need(self.logit_softcap is None or self.logit_softcap > 0, "logit_softcap must be positive", f"logit_softcap={self.logit_softcap}")
        need(len(self.layers) > 0, "layers must not be empty", "layers=[]")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            where = f"layers[{i}].mixer={m}"
            if layer.type == "parallel":
                a, r = m.left, m.right
                need(min(a.heads, a.kv_heads, a.dim, a.vdim) > 0 and a.heads % a.kv_heads == 0, "left: kv_heads must divide heads, sizes must be positive", where)
                need(a.dim == a.vdim, "left: the keys are the values, so vdim must equal dim", where)
                need(a.softcap is None or a.softcap > 0, "left: softcap must be positive", where)
                need(a.q_temp is None or a.q_temp["every"] > 0, "left: q_temp.every must be positive", where)
                need(min(r.width, r.blocks, r.conv) > 0 and r.width % r.blocks == 0, "right: blocks must divide width, sizes must be positive", where)
            else:
                need(min(m.heads, m.kv_heads, m.dim, m.vdim) > 0 and m.heads % m.kv_heads == 0, "kv_heads must divide heads, sizes must be positive", where)
                need(m.rot is None or (m.rot["dims"] % 2 == 0 and 0 <= m.rot["dims"] <= m.dim and m.rot["base"] > 0), "rot.dims must be even and at most dim", where)
                need(m.chunk is None or m.chunk > 0, "mask.size must be positive", where)
            f = layer.mlp
            if f is not None:
                need(f.ff > 0, "the feed-forward's inner size must be positive", f"layers[{i}].mlp={f}")
                if f.kind == "moe":
                    need(0 < f.top <= f.experts, "router.top must lie in [1, experts]", f"layers[{i}].mlp={f}")
                    g = f.groups
                    need(g is None or (g["count"] > 0 and f.experts % g["count"] == 0 and 0 < g["keep"] <= g["count"] and g["keep"] * (f.experts // g["count"]) >= f.top),
                         "router.groups: count must divide experts, and the groups kept must hold at least top experts", f"layers[{i}].mlp={f}")


def _object(obj: dict, key: str, origin: str) -> dict:
    value = obj.get(key)
    if not isinstance(value, dict):
        raise AlofaError("parse", "config key must be an object", f"key={key} config={origin}")
    return value


def _read_rot(obj: dict, origin: str) -> Optional[dict]:
    rot = obj.get("rot")
    if not isinstance(rot, dict):
        return None
    k = Keys(rot, origin)
    scaling = None
    if isinstance(rot.get("scaling"), dict):
        sk = Keys(rot["scaling"], origin)
        scaling = {name: sk.number(name) for name in ("factor", "original", "fast", "slow")}
    return {"base": k.number("base"), "dims": k.integer("dims"), "scaling": scaling}


def _read_mixer(kind: str, obj: dict, origin: str):
    if kind == "parallel":
        lo, ro = _object(obj, "left", origin), _object(obj, "right", origin)
        k, r, top = Keys(lo, origin), Keys(ro, origin), Keys(obj, origin)
        q_temp = None
        if isinstance(lo.get("q_temp"), dict):
            tk = Keys(lo["q_temp"], origin)
            q_temp = {"coef": tk.number("coef"), "every": tk.integer("every")}
        left = KeyedAttentionConfig(k.integer("heads"), k.integer("kv_heads"), k.integer("dim"), k.integer("vdim"), k.number("scale"),
                                    k.number("softcap") if k.has("softcap") else None, q_temp)
        return ParallelConfig(left, RecurrentConfig(r.integer("width"), r.integer("blocks"), r.integer("conv")), top.number("left_scale"), top.number("right_scale"))
    if kind == "attention":
        k = Keys(obj, origin)
        mask = obj.get("mask")
        return DifferentialConfig(k.integer("heads"), k.integer("kv_heads"), k.integer("dim"), k.integer("vdim"), k.number("scale"), k.number("diff"), _read_rot(obj, origin),
                                  Keys(mask, origin).integer("size") if isinstance(mask, dict) else None)
    raise AlofaError("parse", "unknown layer type", f"type={kind} config={origin}")


def _read_mlp(obj, origin: str) -> Optional[FeedForwardConfig]:
    if obj is None:
        return None
    if not isinstance(obj, dict):
        raise AlofaError("parse", "mlp must be an object or null", f"config={origin}")
    k = Keys(obj, origin)
    kind = k.string("kind")
    if kind == "dense":
        return FeedForwardConfig("dense", k.integer("ff"))
    if kind == "moe":
        ro = _object(obj, "router", origin)
        r = Keys(ro, origin)
        groups = None
        if isinstance(ro.get("groups"), dict):
            gk = Keys(ro["groups"], origin)
            groups = {"count": gk.integer("count"), "keep": gk.integer("keep")}
        shared = obj.get("shared")
        return FeedForwardConfig("moe", Keys(_object(obj, "expert", origin), origin).integer("ff"), r.integer("experts"), r.integer("top"), r.number("scale", 1.0), groups,
                                 Keys(shared, origin).integer("ff") if isinstance(shared, dict) else 0)
    raise AlofaError("parse", "unknown mlp kind", f"kind={kind} config={origin}")


def read_config(obj: dict, origin: str) -> KikeraxConfig:
    k = Keys(obj, origin)
    layers = obj.get("layers")
    if not isinstance(layers, list):
        raise AlofaError("parse", "config key must be a list", f"key=layers config={origin}")
    cfg = KikeraxConfig(vocab=k.integer("vocab"), width=k.integer("width"), eps=Keys(_object(obj, "norm", origin), origin).number("eps"),
                        logit_softcap=k.number("logit_softcap") if k.has("logit_softcap") else None)
    for i, entry in enumerate(layers):
        if not isinstance(entry, dict):
            raise AlofaError("parse", "a layer must be an object", f"layers[{i}] config={origin}")
        kind = Keys(entry, origin).string("type")
        cfg.layers.append(KikeraxLayer(kind, _read_mixer(kind, _object(entry, "mixer", origin), origin), _read_mlp(entry.get("mlp"), origin)))
    cfg.validate(origin)
    return cfg


def to_json(cfg: KikeraxConfig) -> dict:
    layers = []
    for layer in cfg.layers:
        m = layer.mixer
        if layer.type == "parallel":
            a, r = m.left, m.right
            left = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
            if a.softcap is not None:
                left["softcap"] = a.softcap
            if a.q_temp is not None:
                left["q_temp"] = dict(a.q_temp)
            mixer = {"left": left, "right": {"width": r.width, "blocks": r.blocks, "conv": r.conv}, "left_scale": m.left_scale, "right_scale": m.right_scale}
        else:
            mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale, "diff": m.diff}
            if m.rot is not None:
                mixer["rot"] = {"base": m.rot["base"], "dims": m.rot["dims"], **({"scaling": dict(m.rot["scaling"])} if m.rot["scaling"] else {})}
            if m.chunk is not None:
                mixer["mask"] = {"size": m.chunk}
        f = layer.mlp
        if f is None:
            mlp = None
        elif f.kind == "dense":
            mlp = {"kind": "dense", "ff": f.ff}
        else:
            router = {"experts": f.experts, "top": f.top, "scale": f.route_scale}
            if f.groups is not None:
                router["groups"] = dict(f.groups)
            mlp = {"kind": "moe", "expert": {"ff": f.ff}, "router": router}
            if f.shared_ff:
                mlp["shared"] = {"ff": f.shared_ff}
        layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
    out = {"architecture": NAME, "vocab": cfg.vocab, "width": cfg.width, "norm": {"eps": cfg.eps}, "layers": layers}
    if cfg.logit_softcap is not None:
        out["logit_softcap"] = cfg.logit_softcap
    return out


def build_spec(cfg: KikeraxConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "parallel":
            a, r = m.left, m.right
            attention = PartSpec("normed_attention", {"hidden_size": width, "heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale,
                                                      "qk_norm": True, "norm_weight": True, "eps": eps, "values": "keys", "gate": True, "softcap": a.softcap,
                                                      "q_temp_coef": a.q_temp["coef"] if a.q_temp else None, "q_temp_every": a.q_temp["every"] if a.q_temp else None},
                                 prefix=p + "mix.left.")
            unit = PartSpec("gated_lru", {"hidden_size": width, "width": r.width, "blocks": r.blocks, "conv": r.conv, "decay_scale": LRU_DECAY_SCALE,
                                          "activation": "gelu_tanh"}, prefix=p + "mix.right.")
            mixer = PartSpec("side_by_side", {"hidden_size": width, "eps": eps, "names": ["left", "right"], "branches": [attention, unit], "combine": "weighted",
                                              "scales": [m.left_scale, m.right_scale]}, prefix=p + "mix.")
        else:
            position = None
            if m.rot is not None and m.rot["dims"]:
                position = PartSpec("rotary_interleaved", {"dims": m.rot["dims"], "base": m.rot["base"], "layout": "pairs", "scaling": m.rot["scaling"]})
            mixer = PartSpec("normed_attention", {"hidden_size": width, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                                                  "qk_norm": True, "norm_weight": True, "eps": eps, "bias": True, "out_bias": True, "gate": True, "maps": 2, "diff": m.diff,
                                                  "chunk": m.chunk, "position": position}, prefix=p + "mix.")
        block = {"hidden_size": width, "mixer": mixer, "mixer_post_norm": PartSpec("rmsnorm", {"size": width, "eps": eps, "weight_name": "norm1"}, prefix=p),
                 "feed_forward": None}
        f = layer.mlp
        if f is not None:
            if f.kind == "dense":
                block["feed_forward"] = PartSpec("mlp", {"hidden_size": width, "intermediate_size": f.ff, "activation": "gelu_tanh", "bias": False}, prefix=p + "mlp.")
            else:
                block["feed_forward"] = PartSpec("routed_experts", {"hidden_size": width, "experts": f.experts, "top": f.top, "expert_ff": f.ff, "shared_ff": f.shared_ff,
                                                                    "activation": "silu", "gated": True, "score": "sigmoid", "renormalize": True, "renorm_eps": RENORM_EPS,
                                                                    "correction": True, "route_scale": f.route_scale, "groups": f.groups["count"] if f.groups else 1,
                                                                    "keep": f.groups["keep"] if f.groups else 1}, prefix=p + "mlp.")
            block["feed_forward_post_norm"] = PartSpec("rmsnorm", {"size": width, "eps": eps, "weight_name": "norm2"}, prefix=p)
        layers.append(LayerSpec(PartSpec("postnorm_residual", block, prefix=p)))
    spec = ModelSpec(
        architecture=NAME, hidden_size=width, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": width, "weight_name": "embed"}),
        layers=layers, run=[RunEntry(i) for i in range(len(layers))],
        final_norm=PartSpec("rmsnorm", {"size": width, "eps": eps, "weight_name": "final.norm"}),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": width, "tied_to": "embed", "weight_name": "embed", "softcap": cfg.logit_softcap}),
    )
    spec.validate()
    return spec


register_architecture(Architecture(NAME, read_config, build_spec, to_json), replace=True)
