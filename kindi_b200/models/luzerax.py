"""The Luzerax decoder: its config.json keys, its typed configuration and its ``ModelSpec``.

What the architecture is. ``x = embed[token]``; a list of layers whose norms sit on the sub-layers' OUTPUTS:
``x += ls1 * norm1(mixer(x))`` and, where the layer has a feed-forward, ``x += ls2 * norm2(ff(x))``, the sub-layers
reading the stream x itself, ``norm`` an RMS norm with gains and ``ls`` a learned per-column scale; a final RMS norm
and an untied head. ``layers[i].type`` names the layer's mixer:

* ``attention``: differential attention without a position encoding. The query projection holds two maps per head
  and the key projection two per key/value head; every map of q and k passes an RMS norm over the head with shared
  gains (``q.norm``, ``k.norm``); queries carry a temperature ``1 + q_temp.coef ln(floor((p + 1) / q_temp.every) + 1)``;
  both maps are causal softmax attention over the same values, and head h is ``a1 - lambda a2`` with
  ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff``, divided by its root mean square and multiplied by ``1 - diff``.
* ``attention_2``: grouped-query attention whose q and k are rotated in adjacent pairs on their first ``rot.dims``
  elements (``f_i = rot.base^(-2i / rot.dims)``), then divided by their root mean square per head (no gains); causal
  softmax; head h's output is multiplied by ``sigmoid(W_g x)_h``.

Both take ``scale`` (the factor on ``q . k``), ``heads``, ``kv_heads``, ``dim`` and ``vdim`` from the configuration.

The feed-forward is dense (``mlp.kind`` = ``dense``: ``W_down (silu(W_gate x) * (W_up x))``) or a mixture of experts
(``moe``): ``router.experts`` experts ``W_down (g' sigmoid(1.702 g') (u' + 1))`` with ``g' = min(W_gate x, limit)`` and
``u' = clamp(W_up x, -limit, limit)`` (``expert.ff``, ``expert.limit``) plus ``router.identity`` experts that hand
their input through; scores are the softmax over all ``experts + identity`` router outputs, the choice of
``router.top`` goes by score + ``correction`` inside the ``router.groups.keep`` best of ``router.groups.count`` equal
groups of neighbours, the weights are the chosen scores over their sum; a shared expert of the same form
(``shared.ff``, ``shared.limit``) is added for every row.

config.json is nested: ``layers[i] = {"type", "mixer": {...}, "mlp": {...} | null}``, ``norm.eps``, ``vocab``,
``width``. Tensors: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``. Every size and constant comes from the configuration; nothing here knows a
particular model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, ConfigReader
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

GLU_ALPHA = 1.702               # the factor inside the experts' sigmoid: fixed by the design


@dataclass(frozen=True)
class LuzeraxMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    # attention (differential)
    diff: Optional[float] = None
    temp_coef: float = 0.0
    temp_every: int = 1
    # attention_2 (rotated, gated)
    rot_base: Optional[float] = None
    rot_dims: int = 0


@dataclass(frozen=True)
class LuzeraxExperts:
    experts: int
    identity: int
    top: int
    groups: int
    keep: int
    ff: int
    limit: float
    shared_ff: Optional[int]
    shared_limit: float


@dataclass(frozen=True)
class LuzeraxLayer:
    kind: str                   # "attention" | "attention_2"
    mixer: LuzeraxMixer
    ff: Any                     # None, an int (the dense feed-forward's inner size) or LuzeraxExperts


@dataclass(frozen=True)
class LuzeraxConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: Tuple[LuzeraxLayer, ...]

    def to_dict(self) -> dict:
        """the config.json that reads back as this configuration"""
        layers = []
        for l in self.layers:
            m = l.mixer
            mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
            if l.kind == "attention":
                mixer.update({"diff": m.diff, "q_temp": {"coef": m.temp_coef, "every": m.temp_every}})
            else:
                mixer["rot"] = {"base": m.rot_base, "dims": m.rot_dims}
            if l.ff is None:
                mlp = None
            elif isinstance(l.ff, int):
                mlp = {"kind": "dense", "ff": l.ff}
            else:
                f = l.ff
                mlp = {"kind": "moe", "expert": {"ff": f.ff, "limit": f.limit},
                       "router": {"experts": f.experts, "identity": f.identity, "top": f.top,
                                  "groups": {"count": f.groups, "keep": f.keep}},
                       "shared": None if f.shared_ff is None else {"ff": f.shared_ff, "limit": f.shared_limit}}
            layers.append({"type": l.kind, "mixer": mixer, "mlp": mlp})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "layers": layers}


def _positive(what: str, v):
    if not (v > 0):
        raise ConfigError("config.json: %s must be positive, found %r" % (what, v))
    return v


def _read_mixer(raw: Mapping[str, Any], where: str, kind: str) -> LuzeraxMixer:
    r = ConfigReader(raw, where)
    heads = _positive(where + ".heads", r.integer("heads"))
    kv = _positive(where + ".kv_heads", r.integer("kv_heads", heads))
    if heads % kv:
        raise ConfigError("%s: heads %d is not a multiple of kv_heads %d" % (where, heads, kv))
    dim = _positive(where + ".dim", r.integer("dim"))
    vdim = _positive(where + ".vdim", r.integer("vdim", dim))
    scale = float(_positive(where + ".scale", r.number("scale", dim ** -0.5)))
    if kind == "attention":
        diff = r.number("diff")
        coef, every = 0.0, 1
        traw = r.any("q_temp")
        if traw is not None:
            tr = ConfigReader(traw, where + ".q_temp")
            coef = float(tr.number("coef", 0.0))
            every = _positive(where + ".q_temp.every", tr.integer("every", 1))
            tr.finish(())
        r.neutral("rot", (None,), "this mixer has no position encoding")
        r.finish(())
        return LuzeraxMixer(heads, kv, dim, vdim, scale, diff=float(diff), temp_coef=coef, temp_every=every)
    rr = ConfigReader(r.any("rot") or {}, where + ".rot")
    base = float(_positive(where + ".rot.base", rr.number("base", 10000.0)))
    dims = rr.integer("dims", dim - dim % 2)
    rr.finish(())
    if dims < 0 or dims % 2 or dims > dim:
        raise ConfigError("%s.rot.dims must be even and at most dim = %d, found %d" % (where, dim, dims))
    r.neutral("diff", (None,), "this mixer has one softmax map per head")
    r.neutral("q_temp", (None,), "this mixer has no query temperature")
    r.finish(())
    return LuzeraxMixer(heads, kv, dim, vdim, scale, rot_base=base, rot_dims=dims)


def _read_mlp(raw: Optional[Mapping[str, Any]], where: str):
    if raw is None:
        return None
    fr = ConfigReader(raw, where)
    kind = fr.string("kind", "dense")
    if kind == "dense":
        ff = _positive(where + ".ff", fr.integer("ff"))
        fr.finish(())
        return ff
    if kind != "moe":
        raise ConfigError("%s: kind %r is not a feed-forward of this architecture (dense, moe)" % (where, kind))
    er = ConfigReader(fr.any("expert") or {}, where + ".expert")
    ff = _positive(where + ".expert.ff", er.integer("ff"))
    limit = float(_positive(where + ".expert.limit", er.number("limit")))
    er.finish(())
    rr = ConfigReader(fr.any("router") or {}, where + ".router")
    experts = _positive(where + ".router.experts", rr.integer("experts"))
    identity = rr.integer("identity", 0)
    top = _positive(where + ".router.top", rr.integer("top"))
    groups, keep = 1, 1
    graw = rr.any("groups")
    if graw is not None:
        gr = ConfigReader(graw, where + ".router.groups")
        groups = _positive(where + ".router.groups.count", gr.integer("count", 1))
        keep = _positive(where + ".router.groups.keep", gr.integer("keep", groups))
        gr.finish(())
    rr.finish(())
    n_out = experts + identity
    if identity < 0:
        raise ConfigError("%s.router.identity must not be negative, found %d" % (where, identity))
    if n_out % groups or keep > groups:
        raise ConfigError("%s.router: %d outputs do not form %d equal groups of which %d are kept"
                          % (where, n_out, groups, keep))
    if top > keep * (n_out // groups):
        raise ConfigError("%s.router.top = %d exceeds the %d outputs of the kept groups"
                          % (where, top, keep * (n_out // groups)))
    shared_ff, shared_limit = None, limit
    sraw = fr.any("shared")
    if sraw is not None:
        sr = ConfigReader(sraw, where + ".shared")
        shared_ff = _positive(where + ".shared.ff", sr.integer("ff"))
        shared_limit = float(_positive(where + ".shared.limit", sr.number("limit", limit)))
        sr.finish(())
    fr.finish(())
    return LuzeraxExperts(experts, identity, top, groups, keep, ff, limit, shared_ff, shared_limit)


_MIXERS = ("attention", "attention_2")


def read_config(raw: Mapping[str, Any]) -> LuzeraxConfig:
    r = ConfigReader(raw)
    arch = r.string("architecture")
    vocab = _positive("vocab", r.integer("vocab"))
    width = _positive("width", r.integer("width"))
    norm = ConfigReader(r.any("norm") or {}, "config.json: norm")
    eps = _positive("norm.eps", norm.number("eps"))
    norm.finish(())
    lraw = r.any("layers")
    if not isinstance(lraw, (list, tuple)) or not lraw:
        raise ConfigError("config.json: layers must be a non-empty list")
    layers = []
    for i, l in enumerate(lraw):
        where = "config.json: layers[%d]" % i
        lr = ConfigReader(l, where)
        kind = lr.string("type")
        if kind not in _MIXERS:
            raise ConfigError("%s: type %r is not a mixer of this architecture (%s)" % (where, kind, ", ".join(_MIXERS)))
        mixer = _read_mixer(lr.any("mixer") or {}, where + ".mixer", kind)
        ff = _read_mlp(lr.any("mlp"), where + ".mlp")
        lr.finish(())
        layers.append(LuzeraxLayer(kind, mixer, ff))
    r.finish()
    return LuzeraxConfig(arch, vocab, width, float(eps), tuple(layers))


EMBEDDING, HEAD, FINAL_NORM = "embed", "head", "final.norm"


def build_spec(cfg: LuzeraxConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": cfg.eps, "weight": ""})
    layers, schedule = [], []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        common = {"n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                  "scale": m.scale, "names": {"q": "q", "k": "k", "v": "v", "o": "o"}}
        if l.kind == "attention":
            mixer = PartSpec("headnorm_attention", dict(
                common, position=PartSpec("none", {}),
                head_norm={"eps": cfg.eps, "when": "before", "q": "q.norm", "k": "k.norm"},
                q_temp={"coef": m.temp_coef, "every": m.temp_every},
                differential={"diff": m.diff, "eps": cfg.eps, "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}))
        else:
            position = PartSpec("rotary", {"base": m.rot_base, "rotary_dim": m.rot_dims, "pairing": "interleaved"}) \
                if m.rot_dims else PartSpec("none", {})
            mixer = PartSpec("headnorm_attention", dict(
                common, position=position, head_norm={"eps": cfg.eps, "when": "after", "q": None, "k": None},
                head_gate="g"))
        ff = None
        if isinstance(l.ff, int):
            ff = PartSpec("swiglu", {"intermediate": l.ff, "activation": "silu",
                                     "names": {"gate": "gate", "up": "up", "down": "down"}})
        elif l.ff is not None:
            f = l.ff
            shared = None
            if f.shared_ff is not None:
                shared = {"intermediate": f.shared_ff, "activation": "glu_clamp", "limit": f.shared_limit,
                          "alpha": GLU_ALPHA,
                          "names": {"gate": "shared.gate", "up": "shared.up", "down": "shared.down"}}
            ff = PartSpec("moe", {
                "n_experts": f.experts, "top_k": f.top, "intermediate": f.ff, "gated": True,
                "activation": "glu_clamp", "limit": f.limit, "alpha": GLU_ALPHA, "score": "softmax_all",
                "router_bias": False, "correction": "correction", "identity": f.identity,
                "groups": {"count": f.groups, "keep": f.keep}, "shared": shared,
                "names": {"router": "router", "gate": "e%d.gate", "up": "e%d.up", "down": "e%d.down"}})
        block = PartSpec("postnorm", {"norm1": norm, "mixer": mixer, "norm2": norm, "feed_forward": ff,
                                      "layer_scale": {"mixer": "ls1", "feed_forward": "ls2"},
                                      "names": {"norm1": "norm1", "mixer": "mix.", "norm2": "norm2",
                                                "feed_forward": "mlp."}})
        layers.append(LayerSpec(block, "l%d." % i))
        schedule.append(ScheduleEntry(layer=i, cache=i))
    spec = ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, width=cfg.width, layers=tuple(layers),
        schedule=tuple(schedule), final_norm=norm, final_norm_prefix=FINAL_NORM,
        embedding=PartSpec("table", {"name": EMBEDDING, "vocab": cfg.vocab}),
        head=PartSpec("linear", {"name": HEAD, "vocab": cfg.vocab}),
        # a layer without a feed-forward has no use for a second norm or scale: a folder that stores them is accepted
        may_ignore=tuple(n for i, l in enumerate(cfg.layers) if l.ff is None
                         for n in ("l%d.norm2" % i, "l%d.ls2" % i)))
    spec.validate()
    return spec


register_architecture("Luzerax", build_spec, read_config)
