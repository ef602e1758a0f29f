"""The Medodra decoder: its config.json keys, its typed configuration and its ``ModelSpec``.

What the architecture is. ``x = embed[token] * embedding.scale`` plus a sinusoidal position vector; a list of layers,
each ``x += m * (mixer(norm1(x)) + ff(norm2(x)))`` with both norms reading the same x (``m`` = ``residual_mult``), the
norms being RMS norms whose gain is one plus the stored weight; a final norm of the same kind and an untied head.
``layers[i].type`` names the layer's mixer:

* ``delta``: the gated delta rule (short convolutions with silu on q, k, v; unit-norm q and k; a decay and a write
  strength per head; a per-head RMS norm and a silu gate on the output).
* ``parallel``: two mixers side by side whose RMS-normed outputs are averaged - ``left``: causal attention without a
  softmax (biases, short convolutions, a query temperature that grows with the position, RMS-normed values, a learned
  distance bias by buckets, sigmoid weights); ``right``: minGRU.

The feed-forward (``mlp.kind`` = ``moe``) is a mixture of gated silu experts: a 32-bit router, sigmoid scores, the
``top`` largest chosen, each expert run on its score times the input, plus a shared expert gated by one sigmoid per
row. A stretch of layers (``loop.start`` to ``loop.stop - 1``) runs ``loop.times`` times with the same weights and a
cache entry of its own for every run; right before the first layer of every pass the residual stream becomes
``W_in [x; x0]`` (``loop.in``), x0 being the embedding output.

config.json is nested: ``layers[i] = {"type", "mixer": {...}, "mlp": {...} | null}``, ``loop``, ``embedding.scale``,
``norm.eps``, ``residual_mult``, ``vocab``, ``width``. Tensors: ``embed``, ``loop.in``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.*``, ``l<i>.mlp.{router,e<j>.{gate,up,down},shared.{gate,up,down,sg}}``, ``final.norm``, ``head``. Every
size and constant comes from the configuration; nothing here knows a particular model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, ConfigReader
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

SINUSOID_BASE = 10000.0         # the position vector's frequencies are base^(-2i / width)
UNIT_EPS = 1e-6                 # inside the root of the delta rule's unit norms


@dataclass(frozen=True)
class MedodraDelta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class MedodraLeft:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    bias_max: float
    temp_coef: float
    temp_every: int


@dataclass(frozen=True)
class MedodraParallel:
    left: MedodraLeft
    right_width: int


@dataclass(frozen=True)
class MedodraMoE:
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class MedodraLayer:
    kind: str                   # "delta" | "parallel"
    mixer: Any
    mlp: Optional[MedodraMoE]


@dataclass(frozen=True)
class MedodraConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    residual_mult: float
    layers: Tuple[MedodraLayer, ...]
    loop: Optional[Tuple[int, int, int]] = None          # start, stop, times

    def run_order(self):
        """(layer, begins a pass) in the order the layers run"""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        order = [(i, False) for i in range(start)]
        for _ in range(times):
            order += [(i, i == start) for i in range(start, stop)]
        return order + [(i, False) for i in range(stop, n)]

    def to_dict(self) -> dict:
        """the config.json that reads back as this configuration"""
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.kind == "delta":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
            else:
                a = m.left
                mixer = {"left": {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim,
                                  "conv": a.conv, "scale": a.scale, "bias_max": a.bias_max,
                                  "q_temp": {"coef": a.temp_coef, "every": a.temp_every}},
                         "right": {"width": m.right_width}}
            mlp = None
            if l.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp.ff},
                       "router": {"experts": l.mlp.experts, "top": l.mlp.top},
                       "shared": None if l.mlp.shared_ff is None else {"ff": l.mlp.shared_ff}}
            layers.append({"type": l.kind, "mixer": mixer, "mlp": mlp})
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale},
               "residual_mult": self.residual_mult, "layers": layers}
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return out


def _positive(what: str, v):
    if not (v > 0):
        raise ConfigError("config.json: %s must be positive, found %r" % (what, v))
    return v


def _heads(r: ConfigReader, where: str):
    heads = _positive(where + ".heads", r.integer("heads"))
    kv = _positive(where + ".kv_heads", r.integer("kv_heads", heads))
    if heads % kv:
        raise ConfigError("%s: heads %d is not a multiple of kv_heads %d" % (where, heads, kv))
    dim = _positive(where + ".dim", r.integer("dim"))
    vdim = _positive(where + ".vdim", r.integer("vdim", dim))
    conv = r.integer("conv", 0)             # taps of the tensors '<projection>.conv'; absent or 0: no convolution
    if not (0 <= conv <= 8):
        raise ConfigError("%s: conv must lie between 0 (none) and 8 taps, found %d" % (where, conv))
    return heads, kv, dim, vdim, conv


def _read_delta(raw: Mapping[str, Any], where: str) -> MedodraDelta:
    r = ConfigReader(raw, where)
    out = MedodraDelta(*_heads(r, where))
    r.finish(())
    return out


def _read_parallel(raw: Mapping[str, Any], where: str) -> MedodraParallel:
    r = ConfigReader(raw, where)
    lw = where + ".left"
    lr = ConfigReader(r.any("left") or {}, lw)
    heads, kv, dim, vdim, conv = _heads(lr, lw)
    scale = float(_positive(lw + ".scale", lr.number("scale", dim ** -0.5)))
    bias_max = float(_positive(lw + ".bias_max", lr.number("bias_max")))
    coef, every = 0.0, 1
    traw = lr.any("q_temp")
    if traw is not None:
        tr = ConfigReader(traw, lw + ".q_temp")
        coef = float(tr.number("coef", 0.0))
        every = _positive(lw + ".q_temp.every", tr.integer("every", 1))
        tr.finish(())
    lr.finish(())
    rr = ConfigReader(r.any("right") or {}, where + ".right")
    right = _positive(where + ".right.width", rr.integer("width"))
    rr.finish(())
    r.finish(())
    return MedodraParallel(MedodraLeft(heads, kv, dim, vdim, conv, scale, bias_max, coef, every), right)


def _read_moe(raw: Mapping[str, Any], where: str) -> MedodraMoE:
    r = ConfigReader(raw, where)
    kind = r.string("kind", "moe")
    if kind != "moe":
        raise ConfigError("%s: kind %r is not a feed-forward of this architecture (moe)" % (where, kind))
    ex = ConfigReader(r.any("expert") or {}, where + ".expert")
    ff = _positive(where + ".expert.ff", ex.integer("ff"))
    ex.finish(())
    ro = ConfigReader(r.any("router") or {}, where + ".router")
    experts = _positive(where + ".router.experts", ro.integer("experts"))
    top = _positive(where + ".router.top", ro.integer("top"))
    ro.finish(())
    if top > experts:
        raise ConfigError("%s.router: top %d exceeds experts %d" % (where, top, experts))
    shared = None
    sraw = r.any("shared")
    if sraw is not None:
        sr = ConfigReader(sraw, where + ".shared")
        shared = _positive(where + ".shared.ff", sr.integer("ff"))
        sr.finish(())
    r.finish(())
    return MedodraMoE(experts, top, ff, shared)


_MIXERS = ("delta", "parallel")


def read_config(raw: Mapping[str, Any]) -> MedodraConfig:
    r = ConfigReader(raw)
    arch = r.string("architecture")
    vocab = _positive("vocab", r.integer("vocab"))
    width = _positive("width", r.integer("width"))
    norm = ConfigReader(r.any("norm") or {}, "config.json: norm")
    eps = float(_positive("norm.eps", norm.number("eps")))
    norm.finish(())
    emb = ConfigReader(r.any("embedding") or {}, "config.json: embedding")
    emb_scale = float(emb.number("scale", 1.0))
    emb.finish(())
    mult = float(r.number("residual_mult", 1.0))
    lraw = r.any("layers")
    if not isinstance(lraw, (list, tuple)) or not lraw:
        raise ConfigError("config.json: layers must be a non-empty list")
    layers = []
    for i, l in enumerate(lraw):
        where = "config.json: layers[%d]" % i
        lr = ConfigReader(l, where)
        kind = lr.string("type")
        mraw = lr.any("mixer") or {}
        if kind == "delta":
            mixer = _read_delta(mraw, where + ".mixer")
        elif kind == "parallel":
            mixer = _read_parallel(mraw, where + ".mixer")
        else:
            raise ConfigError("%s: type %r is not a mixer of this architecture (%s)" % (where, kind, ", ".join(_MIXERS)))
        fraw = lr.any("mlp")
        layers.append(MedodraLayer(kind, mixer, None if fraw is None else _read_moe(fraw, where + ".mlp")))
        lr.finish(())
    loop = None
    lraw = r.any("loop")
    if lraw is not None:
        lp = ConfigReader(lraw, "config.json: loop")
        start, stop, times = lp.integer("start", 0), lp.integer("stop", 0), lp.integer("times", 1)
        lp.finish(())
        if not (0 <= start < stop <= len(layers)) or times < 1:
            raise ConfigError("config.json: loop must have 0 <= start < stop <= %d layers and times >= 1, found "
                              "start %d, stop %d, times %d" % (len(layers), start, stop, times))
        loop = (start, stop, times)
    r.finish()
    return MedodraConfig(arch, vocab, width, eps, emb_scale, mult, tuple(layers), loop)


EMBEDDING, HEAD, FINAL_NORM, LOOP_IN = "embed", "head", "final.norm", "loop.in"


def build_spec(cfg: MedodraConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": cfg.eps, "weight": "", "one_plus": True})
    layers = []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        if l.kind == "delta":
            mixer = PartSpec("gated_delta", {"n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim,
                                             "v_head_dim": m.vdim, "conv": m.conv, "eps": cfg.eps,
                                             "unit_eps": UNIT_EPS})
        else:
            a = m.left
            left = PartSpec("sigmoid_attention", {
                "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
                "scale": a.scale, "conv": a.conv, "bias": True,
                "q_temp": {"coef": a.temp_coef, "every": a.temp_every}, "v_norm": cfg.eps,
                "rel": {"name": "rel", "far": a.bias_max}, "head_bias": "pb"})
            right = PartSpec("min_gru", {"inner": m.right_width, "bias": True})
            mixer = PartSpec("parallel", {"eps": cfg.eps, "branches": (
                {"mixer": left, "prefix": "left.", "gain": "left.out"},
                {"mixer": right, "prefix": "right.", "gain": "right.out"})})
        ff = None
        if l.mlp is not None:
            shared = None
            if l.mlp.shared_ff is not None:
                shared = {"intermediate": l.mlp.shared_ff, "activation": "silu", "row_gate": "shared.sg",
                          "names": {"gate": "shared.gate", "up": "shared.up", "down": "shared.down"}}
            ff = PartSpec("moe", {
                "n_experts": l.mlp.experts, "top_k": l.mlp.top, "intermediate": l.mlp.ff, "activation": "silu",
                "gated": True, "score": "sigmoid", "weight_on": "input", "router_bias": False, "shared": shared,
                "names": {"router": "router", "gate": "e%d.gate", "up": "e%d.up", "down": "e%d.down"}})
        block = PartSpec("parallel", {"norm1": norm, "mixer": mixer, "norm2": norm, "feed_forward": ff,
                                      "residual_mult": cfg.residual_mult,
                                      "names": {"norm1": "norm1", "mixer": "mix.", "norm2": "norm2",
                                                "feed_forward": "mlp."}})
        layers.append(LayerSpec(block, "l%d." % i))
    # every run has a cache entry of its own; a pass over the repeated stretch begins with the mixing product
    schedule = tuple(ScheduleEntry(layer=layer, cache=n, mix_embedding=LOOP_IN if begins else None)
                     for n, (layer, begins) in enumerate(cfg.run_order()))
    spec = ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, width=cfg.width, layers=tuple(layers),
        schedule=schedule, final_norm=norm, final_norm_prefix=FINAL_NORM,
        embedding=PartSpec("table", {"name": EMBEDDING, "vocab": cfg.vocab, "scale": cfg.embedding_scale,
                                     "sinusoid": {"base": SINUSOID_BASE}}),
        head=PartSpec("linear", {"name": HEAD, "vocab": cfg.vocab}),
        # a layer without a feed-forward has no use for a second norm: a folder that stores one all the same is accepted
        may_ignore=tuple("l%d.norm2" % i for i, l in enumerate(cfg.layers) if l.mlp is None)
        + (() if cfg.loop is not None else (LOOP_IN,)))
    spec.validate()
    return spec


register_architecture("Medodra", build_spec, read_config)
