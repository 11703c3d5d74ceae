"""Small Gemosun configurations and weights for the tests: sizes unlike one another (and unlike any model the library
ships numbers for), and weights large enough that every mechanism matters."""
import numpy as np

from fusazen_models import write_model  # noqa: F401  (config.json + model.safetensors from a dict of arrays)


def att(heads, kv_heads, dim, window=None, pool=None, rot_dims=None, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": float(scale if scale is not None else dim ** -0.5)}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if window is not None:
        m["mask"] = {"size": window}
        if pool is not None:
            m["mask"]["pool"] = pool
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def config(width, vocab, layers, eps=1e-5):
    return {"architecture": "Gemosun", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [{"type": "attention", "mixer": m, "mlp": f} for m, f in layers]}


# one mechanism at a time
WINDOW_POOL = config(48, 97, [(att(4, 2, 12, window=10, pool=3, rot_dims=6, base=300.0, scaling=(3.0, 16, 8.0, 0.5)), None)])
WINDOW_ONLY = config(40, 83, [(att(2, 2, 10, window=7, rot_dims=10), None)])                       # a window and nothing beyond it; a whole-head rotation
NO_MASK = config(36, 71, [(att(3, 1, 8), None)])                                                   # every earlier position; no rotation
DENSE = config(32, 61, [(att(2, 1, 8, window=5, pool=5, rot_dims=4, base=50.0), dense(72))])       # a block as long as the window
EXPERTS = config(40, 90, [(att(2, 2, 8, window=9, pool=2, rot_dims=8), moe(16, 6, 2, groups=(3, 2), shared=24)),
                          (att(2, 1, 8, window=4, pool=1, rot_dims=2), moe(12, 5, 3)),               # no groups, no shared expert; blocks of one position
                          (att(4, 4, 4, window=3, pool=7), moe(8, 4, 1, groups=(4, 2), shared=8))])  # groups of one expert; a block longer than the window
# layers unlike each other; blocks that divide no page, a window of one position, a window longer than a page,
# blocks longer than a page
MIXED = config(56, 120, [(att(4, 2, 12, window=70, pool=5, rot_dims=12, base=1000.0, scaling=(8.0, 32, 4.0, 1.0)), dense(64)),
                         (att(2, 1, 16, window=1, pool=3, rot_dims=8), moe(24, 8, 3, groups=(2, 1), shared=16)),
                         (att(6, 3, 8, window=33, pool=66, rot_dims=4, base=77.0), None),
                         (att(2, 2, 20, window=130, pool=11, rot_dims=20, scaling=(2.0, 64, 16.0, 2.0)), dense(40)),
                         (att(3, 3, 12, window=64, pool=64), moe(16, 4, 2, groups=(2, 2)))], eps=1e-4)
# sizes of the kind the fast kernels take (multiples of 16 and 64), several layers
WIDE = config(128, 300, [(att(4, 2, 64, window=100, pool=16, rot_dims=32, scaling=(4.0, 128, 16.0, 1.0)), dense(256)),
                         (att(8, 2, 32, window=64, pool=4, rot_dims=32), moe(64, 8, 2, groups=(4, 2), shared=128)),
                         (att(2, 2, 128, window=150, pool=24, rot_dims=64, base=50000.0), moe(32, 16, 4, groups=(2, 1))),
                         (att(4, 1, 64, window=40, pool=10, rot_dims=16), dense(192))])
# sizes that fit no fast kernel: rows of odd byte counts, head counts that divide nothing
ODD = config(36, 77, [(att(5, 5, 6, window=11, pool=4, rot_dims=2, base=50.0), moe(10, 3, 2, shared=7)),
                      (att(3, 1, 10, window=6, pool=9, rot_dims=6, scaling=(5.0, 8, 2.0, 0.25)), dense(22))], eps=1e-6)
# heads larger than the tensor-core kernels' 64 and 128, and between them
BIG_HEADS = config(192, 211, [(att(2, 1, 96, window=50, pool=6, rot_dims=48, scaling=(4.0, 64, 16.0, 1.0)), dense(128)),
                              (att(2, 2, 160, window=70, pool=9, rot_dims=160), moe(128, 6, 2, groups=(3, 2), shared=64)),
                              (att(3, 1, 192, window=33, pool=4, rot_dims=64), None),
                              (att(2, 1, 256, window=90, pool=16, rot_dims=128, scaling=(8.0, 32, 8.0, 1.0)), moe(256, 4, 2))])
CONFIGS = {"big_heads": BIG_HEADS, "odd": ODD, "window_pool": WINDOW_POOL, "window": WINDOW_ONLY, "no_mask": NO_MASK, "dense": DENSE, "experts": EXPERTS,
           "mixed": MIXED, "wide": WIDE}


def make_weights(cfg, seed):
    """name -> float32 array: sharp attention, routers with spread-out scores, mixtures over the depth with unequal
    (also negative) shares."""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]
    w = {}

    def mat(name, out, inp, gain=1.0):
        w[name] = (rng.standard_normal((out, inp)) * gain / np.sqrt(inp)).astype(np.float32)

    def vec(name, n, mean=0.0, std=1.0):
        w[name] = (mean + std * rng.standard_normal(n)).astype(np.float32)

    w["embed"] = rng.standard_normal((V, W)).astype(np.float32)
    mat("head", V, W, 2.0)
    vec("final.norm", W, 1.0, 0.2)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, G, D = m["heads"], m["kv_heads"], m["dim"]
        vec(p + "norm1", W, 1.0, 0.2)
        mat(p + "mix.q", H * D, W, 3.0)
        mat(p + "mix.k", G * D, W, 3.0)
        mat(p + "mix.g", H, W, 2.0)
        mat(p + "mix.o", W, H * D)
        mlp = layer["mlp"]
        if mlp is not None:
            vec(p + "norm2", W, 1.0, 0.2)
            if mlp["kind"] == "dense":
                mat(p + "mlp.gate", mlp["ff"], W, 2.0)
                mat(p + "mlp.up", mlp["ff"], W, 2.0)
                mat(p + "mlp.down", W, mlp["ff"])
            else:
                F = mlp["expert"]["ff"]
                for e in range(mlp["router"]["experts"]):
                    mat(f"{p}mlp.e{e}.up", F, W, 2.0)
                    mat(f"{p}mlp.e{e}.down", W, F)
                mat(p + "mlp.router", mlp["router"]["experts"], W, 4.0)
                if mlp.get("shared"):
                    mat(p + "mlp.shared.up", mlp["shared"]["ff"], W, 2.0)
                    mat(p + "mlp.shared.down", W, mlp["shared"]["ff"])
                    mat(p + "mlp.shared.sg", 1, W, 2.0)
        c = rng.uniform(0.2, 1.0, i + 2) * rng.choice([1.0, 1.0, 1.0, -0.5], i + 2)
        c[-1] = abs(c[-1]) + 0.3
        w[p + "dwa"] = (c / np.abs(c).sum() * 1.5).astype(np.float32)
    return w
