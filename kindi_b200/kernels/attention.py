"""Attention over the cache: the choice of kernel by dtype and by the step's shape."""
from __future__ import annotations

from . import lib as K


def attention(ctx, q, out, nh, nkv, hd, scale, window, pool, table, n_pages, keep_first: int = 0, sink=None,
              gate=None) -> bool:
    """``out`` = attention of the (already position-encoded) query rows ``q`` over their sequences' cached keys and
    values, which include this step's: all positions up to the row's, or with ``window`` the last ``window`` of them
    and the sequence's first ``keep_first``. ``sink`` (float32 ``[nh]``): ``exp(sink_h)`` joins head h's softmax
    denominator. ``gate`` (rows or 32-bit planes laid out like ``out``): an output gate ``out *= sigmoid(gate)``; the
    return value says whether the kernel applied it (False: the caller still has to)"""
    if ctx.fast:
        from . import fast
        done = fast.attention_bf16(ctx, q, out, nh, nkv, hd, scale, window, pool, table, n_pages, keep_first, sink,
                                   gate)
        if done:
            return done == 2
    rows_gate = gate if gate is not None and gate.dim() == 2 and gate.dtype == q.dtype else None
    K.attn_generic(q, out, ctx.pos, ctx.seq, ctx.slot, nh, nkv, hd, scale, window, pool, table, n_pages, ctx.status,
                   keep_first, sink, rows_gate)
    return rows_gate is not None


def attention_from_planes(ctx, qkv, out, nh, nkv, hd, scale, window, rotation, pool, table, n_pages) -> bool:
    """a decode step of the serving kernels whose QKV product came as 32-bit planes: one kernel sums them, rotates
    queries and the newest key by ``rotation`` (``(inv_freq, rotary_dim)`` of the position encoding, None when it is
    no rotation), stores the newest key and value and attends. False: not taken (the caller encodes, stores and
    attends in separate steps)"""
    if not (ctx.fast and ctx.decode and qkv.dim() == 3 and rotation is not None):
        return False
    from . import fast
    inv_freq, rotary_dim = rotation
    return fast.attention_decode_rope(ctx, qkv, out, nh, nkv, hd, scale, window, inv_freq, rotary_dim, pool, True,
                                      table, n_pages)


def sigmoid_attention(ctx, q, out, nh, nkv, hd, scale, bias, pool, table, n_pages) -> None:
    """``out`` = causal attention whose weights are ``sigmoid(q . k * scale + bias[h][distance])``, not normalised
    over keys, of the query rows ``q`` over their sequences' cached keys and values (this step's included). ``bias``:
    float32 ``[nh, n]`` over the distance, the last entry standing for every larger one, or None"""
    if ctx.decode and (hd * pool.element_size()) % 16 == 0:
        # single tokens, in either dtype: every sequence's pages in splits side by side
        from . import fast
        K.sigattn_decode(q, out, ctx.slot, ctx.kv_len, ctx.B, nh, nkv, hd, scale, bias, pool, table, n_pages,
                         splits=fast.sigmoid_decode_splits(ctx, nkv, nh // nkv), status=ctx.status)
        return
    if ctx.fast:
        from . import fast
        if fast.sigmoid_attention_bf16(ctx, q, out, nh, nkv, hd, scale, bias, pool, table, n_pages):
            return
    K.sigmoid_attn(q, out, ctx.pos, ctx.seq, ctx.slot, nh, nkv, hd, scale, bias, pool, table, n_pages, ctx.status)
