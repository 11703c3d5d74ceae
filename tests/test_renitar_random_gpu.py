"""Random Renitar configurations — number and order of layers, head counts and sizes, taus and decays, taps, rotated
part, caps, blocks of positions, experts with and without those that hand their input on, shared experts, constants and
weights drawn per seed — with randomly cut traces, in both types against the plain implementation (GPU).  The second
family draws sizes that the fast kernels take (head sizes that are multiples of 16, widths that are multiples of 64)
with requests of a few hundred tokens, so that blocks of positions pass over page borders in the fast kernels too."""
import numpy as np
import pytest

import helpers as H
import plain_renitar as G
import renitar_models as M

pytestmark = pytest.mark.gpu
STORAGE = {"float32": "F32", "bfloat16": "BF16"}


def random_mixer(rng, dims, longest, most_kv=4):
    if rng.random() < 0.5:
        return M.gla(int(rng.integers(1, 5)), int(rng.choice(dims)), int(rng.choice(dims)), float(rng.choice([1.0, 4.0, 16.0, 64.0])))
    kv = int(rng.integers(1, most_kv + 1))
    heads = kv * int(rng.integers(1, 5))
    dim, vdim = int(rng.choice(dims)), int(rng.choice(dims))
    left = M.att(heads, kv, dim, vdim, scale=float(rng.uniform(0.5, 1.5)) * dim ** -0.5,
                 conv=int(rng.integers(1, 6)) if rng.random() < 0.8 else None,
                 chunk=int(rng.integers(1, longest)) if rng.random() < 0.85 else None,
                 rot_dims=int(rng.choice([d for d in (0, 2, 4, 6, 8, 16, 32, 64, 128) if d <= dim])),
                 base=float(rng.choice([50.0, 10000.0, 500000.0])),
                 softcap=float(rng.choice([2.0, 10.0, 30.0, 50.0])) if rng.random() < 0.8 else None)
    n_right = int(rng.integers(1, 5))
    right = M.lin(int(rng.choice(dims)), int(rng.choice(dims)), [float(rng.choice([0.3, 0.8, 0.95, 0.999, 1.0])) for _ in range(n_right)])
    return M.pair(left, right)


def random_mlp(rng, inners):
    if rng.random() < 0.2:
        return None
    experts = int(rng.integers(1, 13))
    identity = int(rng.integers(0, 4)) if rng.random() < 0.7 else None
    top = int(rng.integers(1, min(experts + (identity or 0), 6) + 1))
    return M.moe(int(rng.choice(inners)), experts, top, scale=float(rng.uniform(0.5, 3.0)), identity=identity,
                 shared=int(rng.choice(inners)) if rng.random() < 0.6 else None)


def random_config(rng, fast):
    if fast:
        width, dims, inners, longest = int(rng.choice([64, 128, 192, 256])), [16, 32, 48, 64, 96, 128], [64, 128, 192], 250
    else:
        width, dims, inners, longest = int(rng.choice([20, 36, 48, 50, 72, 100])), [3, 4, 6, 8, 10, 16, 24, 32, 48, 80], [8, 12, 22, 40, 64], 120
    layers = [(random_mixer(rng, dims, longest, 2 if fast else 4), random_mlp(rng, inners)) for _ in range(int(rng.integers(1, 5 if fast else 8)))]
    for (kind, m), _ in layers:                      # a rotation pairs entries: an odd head size rotates one entry less
        if kind == "parallel" and "rot" in m["left"]:
            m["left"]["rot"]["dims"] -= m["left"]["rot"]["dims"] % 2
    return M.config(width, int(rng.integers(30, 400)), layers, eps=float(rng.choice([1e-6, 1e-5, 1e-3])),
                    mult=float(rng.choice([0.3, 0.5, 1.0])))


def run(cfg, rng, seed, dtype, lengths, folder):
    import llmi_b200 as L
    w = M.write_model(folder, cfg, M.make_weights(cfg, seed, rank=int(rng.integers(1, 20))), STORAGE[dtype])
    model = L.load(folder, dtype)
    reqs = {f"r{i}": rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate(lengths)}
    refs = {r: G.forward(cfg, w, t) for r, t in reqs.items()}
    cuts = [H.trace_whole(reqs), H.trace_portions(reqs, int(rng.integers(2, 70)), n_last=int(rng.integers(1, 20))),
            H.trace_last_decoded(reqs, n_last=int(rng.integers(20, 60))),
            H.trace_batches(reqs, int(rng.integers(2, 5)), {r: int(rng.integers(1, len(t) + 1)) for r, t in reqs.items()}),
            H.trace_mixed(reqs, {r: int(rng.integers(1, len(t) + 1)) for r, t in reqs.items()},
                          {r: int(rng.choice([1, 1, 2, 9])) for r in reqs})]
    for steps, most in cuts:
        got = H.collect(steps, H.replay(model, steps, most), cfg["vocab"])
        errs = []
        for r in refs:
            assert np.isfinite(got[r]).all(), (cfg, r)
            errs.extend((np.abs(got[r] - refs[r]).max(axis=1) / np.abs(refs[r]).max()).tolist())
        if dtype == "float32":
            assert max(errs) < 5e-5, (cfg, max(errs))
        else:
            # bf16 rounds every layer's activations to 2^-9 of their size: the typical row stays within a bound that grows
            # with the root of the depth.  A router whose corrected scores nearly tie chooses otherwise than the float64
            # oracle in a few rows, and such a row, and what follows it through the states, is off by a large part of a
            # logit: those rows are counted, not bounded
            e, deep = np.asarray(errs), len(cfg["layers"]) ** 0.5
            assert float(np.median(e)) < 1.2e-2 * deep and float(np.quantile(e, 0.9)) < 5e-2 * deep and float((e > 0.25).mean()) < 0.05, (
                cfg, float(np.median(e)), float(np.quantile(e, 0.9)), float((e > 0.25).mean()), float(e.max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(8))
def test_random_configuration_and_trace(seed, dtype, tmp_path):
    rng = np.random.default_rng(7000 + seed)
    cfg = random_config(rng, fast=False)
    lengths = [int(n) for n in rng.integers(1, 150, 4)] + [int(rng.choice([63, 64, 65, 128, 129]))]
    run(cfg, rng, seed, dtype, lengths, str(tmp_path / "m"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(4))
def test_random_configuration_at_the_fast_kernels_sizes(seed, dtype, tmp_path):
    rng = np.random.default_rng(8000 + seed)
    cfg = random_config(rng, fast=True)
    lengths = [int(rng.integers(130, 330)), int(rng.choice([255, 256, 257]))]
    run(cfg, rng, seed, dtype, lengths, str(tmp_path / "m"))
