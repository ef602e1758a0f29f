"""Random Luzerax configurations - widths, layer orders, head counts, groups and sizes (also sizes no vector load
takes), rotated parts of any even size, temperatures, dense feed-forwards, experts in any grouping with and without
identity and shared experts, or no feed-forward at all - each against the plain implementation: whole prompts, their
last tokens one by one, and all requests as one unequal batch, in both dtypes."""
import random

import pytest

import tiny
import tiny_luzerax as TL
import test_luzerax_gpu as T

pytestmark = pytest.mark.gpu


def random_mlp(rng: random.Random):
    r = rng.random()
    if r < 0.15:
        return None
    if r < 0.35:
        return TL._dense(rng.choice([16, 24, 40, 96, 200]))
    groups = rng.choice([1, 1, 2, 3, 4])
    size = rng.choice([1, 2, 3, 4, 6])
    n_out = groups * size
    identity = rng.randint(0, min(3, n_out - 1))
    keep = rng.randint(1, groups)
    top = rng.randint(1, min(4, keep * size))
    shared = rng.choice([None, (16, 0.8), (72, 2.0)])
    return TL._moe(n_out - identity, identity, top, groups, keep, rng.choice([16, 20, 40, 96]),
                   rng.choice([0.5, 1.0, 3.0]), shared)


def random_config(rng: random.Random) -> dict:
    width = rng.choice([48, 64, 72, 96, 128, 136, 256])
    layers = []
    for _ in range(rng.randint(1, 5)):
        kv = rng.choice([1, 2, 3])
        heads = kv * rng.choice([1, 2, 4])
        dim = rng.choice([8, 10, 20, 32, 48, 64, 96, 128])
        vdim = rng.choice([dim, 8, 12, 40, 64, 100, 128])
        if rng.random() < 0.5:
            layers.append(TL._diff(heads, kv, dim, vdim, 0.1, rng.choice([0.2, 0.4, 0.55]), rng.choice([0.0, 0.3, 0.8]),
                                   rng.choice([1, 7, 64, 500]), random_mlp(rng)))
        else:
            layers.append(TL._rot(heads, kv, dim, vdim, 0.1, rng.choice([100.0, 10000.0, 250000.0]),
                                  rng.choice([0, 2, dim // 2 - dim // 2 % 2, dim - dim % 2]), random_mlp(rng)))
    return TL._config(rng.choice([97, 211, 512]), width, rng.choice([1e-6, 1e-5]), layers)


SEEDS = [2000, 2003, 2006, 2009, 2012, 2015, 2018, 2021]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("k", range(len(SEEDS)))
def test_random_configuration(tmp_path, k, dtype):
    rng = random.Random(SEEDS[k])
    cfg = random_config(rng)
    name = "R%d" % k
    TL.TINY[name] = (cfg, 500 + k)
    try:
        folder = TL.make_model(tmp_path, name, dtype)
    finally:
        del TL.TINY[name]
    reqs = T._edge_requests(cfg, seed=3, L=150)
    reqs = dict(list(reqs.items())[:4] + list(reqs.items())[-3:])
    want = T._plain(folder, reqs)
    steps = tiny.trace_whole(reqs)
    later = tiny.trace_last_n(reqs, 24)
    for s in later:
        s["step"] += len(steps)
    eng = T._engine(folder, steps + later, dtype)
    out = str(tmp_path / "out")
    tiny.run_replay(eng, steps, out)
    T._compare(tiny.collect(out, steps, cfg["vocab"]), reqs, want, T.TOL[dtype], "%s %s whole" % (name, dtype))
    tiny.run_replay(eng, later, out)
    T._compare(tiny.collect(out, later, cfg["vocab"]), reqs, want, T.TOL[dtype], "%s %s decoded" % (name, dtype))
    decode = {r: min(len(reqs[r]) - 1, rng.choice([0, 3, 9])) for r in reqs}
    group = tiny.trace_group(reqs, decode)
    eng = T._engine(folder, group, dtype)
    out = str(tmp_path / "batch")
    tiny.run_replay(eng, group, out)
    eng.check_status()
    eng.cache.check()
    T._compare(tiny.collect(out, group, cfg["vocab"]), reqs, want, T.TOL[dtype], "%s %s batch" % (name, dtype))
