"""Random Medodra configurations - widths, layer orders, repeated stretches, head counts, groups and sizes (also sizes
no vector load takes), taps or none, tables of 4 to 32 rows, experts and shared experts or none - each against the plain
implementation: whole prompts, their last tokens one by one, and all requests as one unequal batch, in both dtypes."""
import random

import pytest

import tiny
import tiny_medodra as TM
import test_medodra_gpu as T

pytestmark = pytest.mark.gpu


def random_config(rng: random.Random) -> dict:
    width = rng.choice([48, 64, 72, 96, 128, 136, 256])
    n_layers = rng.randint(1, 5)
    layers = []
    for _ in range(n_layers):
        mlp = None
        if rng.random() < 0.8:
            experts = rng.choice([2, 3, 5, 8, 12])
            mlp = TM._moe(experts, rng.randint(1, min(experts, 3)), rng.choice([16, 24, 40, 96]),
                          rng.choice([None, 16, 72, 128]))
        kv = rng.choice([1, 2, 3])
        if rng.random() < 0.5:
            dim = rng.choice([8, 20, 32, 48, 64, 96, 128])
            rows = rng.choice([4, 6, 8, 16, 32])
            far = rng.choice([rows / 2 + 0.5, rows / 2 + 3, 40, 64, 100, 240, 500.5])
            layers.append(TM._par(kv * rng.choice([1, 2, 4, 8]), kv, dim, rng.choice([dim, 16, 40, 96, 128]),
                                  rng.choice([None, 1, 2, 3, 4]), rng.choice([0.1, 0.25, dim ** -0.5]), far,
                                  rng.choice([0.0, 0.3, 0.5]), rng.choice([1, 7, 64, 128]),
                                  rng.choice([16, 40, width, 384]), mlp, rows=rows))
        else:
            layers.append(TM._delta(kv * rng.choice([1, 2, 4]), kv, rng.choice([8, 20, 32, 64, 128]),
                                    rng.choice([8, 12, 64, 100]), rng.choice([None, 1, 2, 3, 4]), mlp))
    loop = None
    if rng.random() < 0.6:
        a = rng.randrange(n_layers)
        loop = (a, rng.randint(a + 1, n_layers), rng.randint(1, 3))
    return TM._config(rng.choice([97, 211, 512]), width, rng.choice([1e-6, 1e-5]), rng.choice([0.5, 1.0, 3.0]),
                      rng.choice([0.5, 1.0, 0.25]), layers, loop)


# (seed 1018 is left out: its model has two router logits 1.4e-7 apart at one row, a close call that a 32-bit and a
# 64-bit router decide differently)
SEEDS = [1000, 1003, 1006, 1009, 1012, 1015, 1021, 1024]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("k", range(len(SEEDS)))
def test_random_configuration(tmp_path, k, dtype):
    rng = random.Random(SEEDS[k])
    cfg = random_config(rng)
    name = "R%d" % k
    TM.TINY[name] = (cfg, 500 + k)
    try:
        folder = TM.make_model(tmp_path, name, dtype)
    finally:
        del TM.TINY[name]
    reqs = T._edge_requests(cfg, seed=3, longest=300)
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
