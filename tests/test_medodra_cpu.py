"""The Medodra architecture without a GPU: its configuration reader, the order its layers run in and the cache every
run needs (pages, convolution tails and recurrent states of one entry), the distance table as the part folds it, and
the plain implementation's own sanity (the planted key decides a probe's logits; the forms the kernels for long
prompts rest on - the delta rule of a run as one triangular system, minGRU of a run as a linear map of the state it
starts from - are the same functions as the token-by-token definitions)."""
import copy
import math
import random

import numpy as np
import pytest
import torch

import plain_medodra as PM
import tiny_medodra as TM
from kindi_b200.cache.sequence_cache import SequenceCache
from kindi_b200.config import ConfigError
from kindi_b200.config.registry import model_from_config
from kindi_b200.parts.base import KVNeed, StateNeed
from kindi_b200.parts.model import cache_needs, expected_tensors, tensor_inits
from kindi_b200.parts.sigmoid_attention import distance_bucket

F64 = torch.float64


def test_config_reads_every_size_from_the_nested_keys():
    raw = TM.config("A")
    cfg, spec = model_from_config(raw)
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.embedding_scale, cfg.residual_mult) == (211, 64, 1e-5, 1.7, 1.0)
    assert [l.kind for l in cfg.layers] == ["parallel", "delta", "parallel"] and cfg.loop is None
    a = cfg.layers[0].mixer.left
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.conv, a.scale, a.bias_max, a.temp_coef, a.temp_every) == \
        (4, 2, 16, 24, 3, 0.3, 40, 0.5, 16)
    assert cfg.layers[0].mixer.right_width == 48
    m = cfg.layers[1].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.conv) == (4, 2, 16, 8, 2) and cfg.layers[1].mlp is None
    f = cfg.layers[0].mlp
    assert (f.experts, f.top, f.ff, f.shared_ff) == (4, 2, 24, 16) and cfg.layers[2].mlp.shared_ff is None
    assert cfg.to_dict() == raw
    for name in "BCDE":
        assert model_from_config(TM.config(name))[0].to_dict() == _with_defaults(TM.config(name))
    names = expected_tensors(spec)
    assert names["embed"] == (211, 64) and names["head"] == (211, 64) and names["final.norm"] == (64,)
    assert "loop.in" not in names
    assert names["l0.mix.left.q"] == (64, 64) and names["l0.mix.left.k"] == (32, 64) and names["l0.mix.left.v"] == (48, 64)
    assert names["l0.mix.left.o"] == (64, 96) and names["l0.mix.left.o.b"] == (64,) and names["l0.mix.left.v.b"] == (48,)
    assert names["l0.mix.left.k.conv"] == (32, 3) and names["l0.mix.left.pb"] == (4,) and names["l0.mix.left.out"] == (64,)
    assert names["l0.mix.left.rel"][1] == 4 and names["l0.mix.left.rel"][0] < 0        # the tensor's own rows
    assert names["l0.mix.right.z"] == (48, 64) and names["l0.mix.right.x.b"] == (48,) and names["l0.mix.right.o"] == (64, 48)
    assert names["l0.mlp.router"] == (4, 64) and names["l0.mlp.e3.down"] == (64, 24) and names["l0.mlp.shared.up"] == (16, 64)
    assert names["l1.mix.q"] == (32, 64) and names["l1.mix.v"] == (32, 64) and names["l1.mix.v.conv"] == (32, 2)
    assert names["l1.mix.b"] == (4, 64) and names["l1.mix.a"] == (4, 64) and names["l1.mix.A_log"] == (4,)
    assert names["l1.mix.norm"] == (8,) and names["l1.mix.g"] == (32, 64) and names["l1.mix.o"] == (64, 32)
    assert not any(n.startswith(("l1.mlp", "l1.norm2")) for n in names)
    assert not any(n.startswith("l2.mlp.shared") for n in names)
    assert tensor_inits(spec)["l1.mix.norm"] == "gain"


def _with_defaults(raw):
    """what to_dict writes for a layer that gave no ``conv``: none, as a number"""
    raw = copy.deepcopy(raw)
    for l in raw["layers"]:
        m = l["mixer"]["left"] if l["type"] == "parallel" else l["mixer"]
        m.setdefault("conv", 0)
    return raw


@pytest.mark.parametrize("change,word", [
    (lambda c: c.update(bogus=1), "bogus"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(window=64), "window"),
    (lambda c: c["layers"][0].update(type="attention"), "attention"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "dense"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].update(conv=9), "conv"),
    (lambda c: c["layers"][1]["mixer"].pop("dim"), "dim"),
    (lambda c: c.update(loop={"start": 2, "stop": 2, "times": 2}), "loop"),
    (lambda c: c.update(loop={"start": 0, "stop": 4, "times": 2}), "loop"),
    (lambda c: c.update(loop={"start": 0, "stop": 2, "times": 0}), "loop"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_config_errors_name_the_key(change, word):
    c = TM.config("A")
    change(c)
    with pytest.raises(ConfigError) as e:
        model_from_config(c)
    assert word in str(e.value)


@pytest.mark.parametrize("name", sorted(TM.TINY))
def test_every_run_of_a_layer_has_its_own_cache(name):
    raw = TM.config(name)
    cfg, spec = model_from_config(raw)
    order = PM.run_order(raw)
    assert [(e.layer, e.mix_embedding is not None) for e in spec.schedule] == order == cfg.run_order()
    assert [e.cache for e in spec.schedule] == list(range(len(order)))          # nothing shared between passes
    assert ("loop.in" in expected_tensors(spec)) == ("loop" in raw)
    if "loop" in raw:
        assert expected_tensors(spec)["loop.in"] == (raw["width"], 2 * raw["width"])
        assert sum(1 for _, starts in order if starts) == raw["loop"]["times"]
    needs = cache_needs(spec)
    for e in spec.schedule:
        layer, need = raw["layers"][e.layer], needs[e.cache]
        if layer["type"] == "delta":
            m = layer["mixer"]
            taps = m.get("conv", 0)
            want = [StateNeed((m["heads"], m["vdim"], m["dim"]))]
            if taps > 1:
                want.append(StateNeed((taps - 1, 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"])))
            assert list(need) == want
        else:
            a, w = layer["mixer"]["left"], layer["mixer"]["right"]["width"]
            taps = a.get("conv", 0)
            kv = need[0]
            assert isinstance(kv, KVNeed) and kv.n_kv_heads == a["kv_heads"] and kv.window is None
            assert kv.head_dim >= max(a["dim"], a["vdim"]) and kv.head_dim % 8 == 0
            rest = list(need[1:])
            if taps > 1:
                assert rest.pop(0) == StateNeed((taps - 1, (a["heads"] + a["kv_heads"]) * a["dim"] + a["kv_heads"] * a["vdim"]))
            assert rest == [StateNeed((w,))]
    assert SequenceCache.bytes_needed(needs, 1024, 4, torch.bfloat16, 256) > 0


@pytest.mark.parametrize("rows,far", [(6, 7.5), (8, 40), (16, 64), (12, 200), (32, 300), (7, 17), (16, 8.5)])
def test_distance_table(rows, far):
    """one row per distance below rows // 2, then rows spaced evenly in the logarithm; the last row is reached at
    `far` and never left; the part's function is the plain one"""
    half = rows // 2
    last = None
    for n in range(0, int(far) * 3 + 5):
        b = distance_bucket(n, rows, far)
        assert b == PM.distance_bucket(n, rows, far)
        assert 0 <= b <= rows - 1 and (last is None or b >= last)
        if n < half:
            assert b == n
        else:
            want = half + math.floor(math.log(n / half) / math.log(far / half) * (rows - half))
            assert b == min(rows - 1, want)
        if n >= far:
            assert b == rows - 1
        last = b
    assert distance_bucket(half, rows, far) == half


def test_the_delta_rule_of_a_run_is_one_triangular_system():
    """with G_t = g_0 .. g_t: U = (I + A)^-1 R, A[t][s] = beta_t (G_t / G_s)(k_t . k_s) below the diagonal,
    R_t = beta_t (v_t - G_t S0^T k_t); o_t = G_t S0^T q_t + sum_(s<=t) (G_t / G_s)(q_t . k_s) u_s;
    S_end = G_last S0 + sum_s (G_last / G_s) k_s u_s^T: what the kernel for long prompts computes a run"""
    g = torch.Generator().manual_seed(3)
    T, d, dv = 37, 12, 7
    q = torch.randn(T, 1, d, generator=g, dtype=F64)
    k = torch.randn(T, 1, d, generator=g, dtype=F64)
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(T, 1, dv, generator=g, dtype=F64)
    beta = torch.rand(T, 1, generator=g, dtype=F64)
    decay = 0.5 + 0.5 * torch.rand(T, 1, generator=g, dtype=F64)
    S0 = torch.randn(d, dv, generator=g, dtype=F64)
    states = [S0.clone()]
    want = PM.delta_recurrence(q, k, v, beta, decay, states)[:, 0]
    K_, Q_, V_, b_ = k[:, 0], q[:, 0], v[:, 0], beta[:, 0]
    G = torch.cumprod(decay[:, 0], 0)
    ratio = torch.tril(G[:, None] / G[None, :])
    A = torch.tril(b_[:, None] * ratio * (K_ @ K_.T), diagonal=-1)
    R = b_[:, None] * (V_ - G[:, None] * (K_ @ S0))
    U = torch.linalg.solve_triangular(torch.eye(T, dtype=F64) + A, R, upper=False)
    O = G[:, None] * (Q_ @ S0) + (ratio * (Q_ @ K_.T)) @ U
    S_end = G[-1] * S0 + (K_ * (G[-1] / G)[:, None]).T @ U
    assert float((O - want).abs().max()) < 1e-10
    assert float((S_end - states[0]).abs().max()) < 1e-10


def test_min_gru_of_a_run_is_linear_in_the_state_it_starts_from():
    g = torch.Generator().manual_seed(4)
    T, W = 50, 9
    z = torch.rand(T, W, generator=g, dtype=F64)
    u = torch.randn(T, W, generator=g, dtype=F64)
    S_in = torch.randn(W, generator=g, dtype=F64)
    from_zero = PM.min_gru_scan(z, u)[-1]
    A = torch.prod(1.0 - z, dim=0)
    assert float((PM.min_gru_scan(z, u, S_in)[-1] - (A * S_in + from_zero)).abs().max()) < 1e-12
    # the candidate: u + 1/2 from zero on, the logistic function below (both 1/2 at zero)
    one = PM.min_gru_scan(torch.ones(1, 3, dtype=F64), torch.tensor([[-2.0, 0.0, 3.0]], dtype=F64))[0]
    assert torch.allclose(one, torch.tensor([1.0 / (1.0 + math.exp(2.0)), 0.5, 3.5], dtype=F64))


def test_position_vector_and_norm():
    x = PM.sinusoid(torch.tensor([0, 1, 5]), 8)
    assert torch.allclose(x[0], torch.tensor([0.0, 1.0] * 4, dtype=F64))
    for i in range(4):
        a = 5 * 10000.0 ** (-2.0 * i / 8)
        assert abs(float(x[2, 2 * i]) - math.sin(a)) < 1e-12 and abs(float(x[2, 2 * i + 1]) - math.cos(a)) < 1e-12
    v = torch.tensor([[3.0, -4.0]], dtype=F64)
    n = PM.norm_one_plus(v, torch.tensor([0.5, -1.0], dtype=F64), 0.0)
    assert torch.allclose(n, torch.tensor([[3.0 / math.sqrt(12.5) * 1.5, 0.0]], dtype=F64))


@pytest.mark.parametrize("name,floor", [("A", 0.1), ("B", 0.1), ("E", 0.1), ("D", 0.01)])
def test_the_planted_key_decides_a_probes_logits(tmp_path, name, floor):
    """what the engine tests rest on: on the plain model, a probe row's logits move by more than the bfloat16
    tolerance when the needle is taken away, although hundreds of keys lie between them (in D, where one query head
    of five reads the needle and a layer's output counts a quarter, by hundreds of times the 32-bit tolerance)"""
    folder = TM.make_model(tmp_path, name, "float32")
    raw = TM.config(name)
    cfg, w = PM.load_model(folder)
    rng = random.Random(5)
    toks = TM.needle_request(raw["vocab"], 200, 20, list(range(194, 200)), rng)
    full = PM.forward(cfg, w, toks).numpy()
    gone = list(toks)
    gone[20] = 7
    hidden = PM.forward(cfg, w, gone).numpy()
    assert np.abs(full[194:] - hidden[194:]).max() > floor * np.abs(full).max()
