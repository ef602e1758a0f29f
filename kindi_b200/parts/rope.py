"""Position encodings. The attention mixer hands its projections to its position encoding, which rotates queries
and keys and stores keys and values (one fused kernel); an encoding that is a rotation also offers its table
(``inv_freq[i]`` for each rotated pair and the number of rotated dimensions) to kernels that rotate on the fly.

Rotary (rotate-half pairing, for tensors in the safetensors layout): pair ``(i, i + rot/2)``, angle
``float(pos) * inv_freq[i]`` with ``inv_freq[i] = base ** (-2 i / rot)`` rounded to 32-bit; the reference's form
for such tensors is ``kindi/dspine.cu:151-174`` (angle in 32-bit, ``a c - b s`` / ``b c + a s``), its GGUF path
rotates adjacent pairs of permuted rows, which is the same function (``kindi/nbq.cu:497-520``); the base defaults
to 10000.0 (``kindi/nanbeige.py:256``). ``NoPosition`` rotates nothing.

Options of ``rotary``. ``pairing``: ``"half"`` (the default, above) or ``"interleaved"`` (element 2i with 2i + 1); the
rotate-and-store kernels take the half pairing only, so an interleaved rotation is for mixers that rotate with kernels
of their own (latent attention) and read ``inv_freq``, ``mult`` and ``pairing`` from the part. ``scaling`` (``factor``,
``original``, ``fast``, ``slow``): frequencies stretched for contexts beyond the one a model was trained at (YaRN,
Peng et al., "YaRN: Efficient Context Window Extension of Large Language Models"). With
``dim(t) = rot ln(original / (2 pi t)) / (2 ln base)``, ``lo = max(floor(dim(fast)), 0)``,
``hi = min(ceil(dim(slow)), rot - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` the frequency of
pair i becomes ``f_i / factor * ramp_i + f_i (1 - ramp_i)``, and cosines and sines are multiplied by
``mult = 0.1 ln(factor) + 1``.
"""
from __future__ import annotations

import math

import torch

from ..config.registry import register_part
from ..kernels import lib as K
from .base import PositionEncoding


class RotationEncoding(PositionEncoding):
    """a rotation of the pairs (i, i + rotary_dim / 2) by pos * inv_freq[i]; subclasses set ``inv_freq`` (float32
    ``[max(1, rotary_dim / 2)]`` on the device) and ``rotary_dim`` (even, at most the head size; 0 rotates nothing)"""

    # a hashable name of the frequency table when parts of other layers may have the very same one (then a step
    # computes its rows' cosines and sines once and every such part uses them); None: this part's table is its own
    angles_key = None

    mult = 1.0                  # factor on every cosine and sine
    pairing = "half"            # or "interleaved"

    def rotation(self):
        if self.pairing != "half" or self.mult != 1.0:
            return None         # kernels that rotate on the fly take the plain rotate-half form only
        return self.inv_freq, self.rotary_dim

    def encode_and_store(self, ctx, qkv, q_out, n_heads, n_kv_store, head_dim, pool, table, n_pages,
                         qk_norm=None) -> None:
        if self.pairing != "half" or self.mult != 1.0:
            raise NotImplementedError("the rotate-and-store kernels rotate the pairs (i, i + rot / 2) with unit "
                                      "cosines and sines; this encoding is for mixers that rotate themselves")
        if qk_norm is not None:
            # a norm over the whole query and key projections comes before the rotation: one kernel does both
            wq, wk, eps, nq_true, nk_true = qk_norm
            n_kv = wk.numel() // head_dim
            K.norm_rope_store(qkv, q_out, wq, wk, eps, nq_true, nk_true, self.inv_freq, self.rotary_dim, ctx.pos,
                              ctx.seq, ctx.slot, n_heads, n_kv, n_kv_store, head_dim, pool if n_kv_store else None,
                              table, n_pages, ctx.status)
            return
        angles = None
        if self.angles_key is not None and ctx.T >= K.rope_table_min_rows() and self.rotary_dim >= 16:
            angles = ctx.scratch.get(self.angles_key)
            if angles is None:
                angles = ctx.scratch[self.angles_key] = K.rope_table(ctx.pos, self.inv_freq, self.rotary_dim)
        K.rope_store(qkv, q_out, self.inv_freq, self.rotary_dim, ctx.pos, ctx.seq, ctx.slot, n_heads, n_kv_store,
                     head_dim, pool if n_kv_store else None, table, n_pages, ctx.status, angles)


class Rotary(RotationEncoding):
    def __init__(self, spec, width, weights, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.base = float(spec["base"])
        self.rotary_dim = int(spec["rotary_dim"])
        if self.rotary_dim % 2 or self.rotary_dim <= 0:
            raise ValueError("rotary_dim must be even and positive, found %d" % self.rotary_dim)
        self.pairing = str(spec.get("pairing") or "half")
        if self.pairing not in ("half", "interleaved"):
            raise ValueError("pairing must be 'half' or 'interleaved', found %r" % self.pairing)
        f, self.mult = yarn_frequencies(self.base, self.rotary_dim, spec.get("scaling"))
        self.inv_freq = f.to(torch.float32).to(device)
        self.inv_freq64 = f.to(device)          # for kernels of the true 32-bit path that take their angles in 64-bit
        self.angles_key = ("rotary", self.base, self.rotary_dim) if spec.get("scaling") is None else None


def yarn_frequencies(base: float, rot: int, scaling=None):
    """(frequency of each rotated pair, float64 [rot / 2]; the factor on cosines and sines). ``scaling`` None: the
    plain ``base ** (-2 i / rot)`` and 1.0"""
    i = torch.arange(0, rot // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / rot)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if not (factor > 0.0 and original > 0.0 and float(scaling["fast"]) > 0.0 and float(scaling["slow"]) > 0.0):
        raise ValueError("rotation scaling needs positive factor, original, fast and slow, found %r" % (dict(scaling),))

    def dim_of(turns: float) -> float:
        return rot * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), rot - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class NoPosition(RotationEncoding):
    def __init__(self, spec, width, weights, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.rotary_dim = 0
        self.inv_freq = torch.zeros(1, dtype=torch.float32, device=device)


register_part("position", "rotary", Rotary)
register_part("position", "none", NoPosition)
