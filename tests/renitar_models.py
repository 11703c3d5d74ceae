"""Small Renitar configurations and weights for the tests: sizes unlike one another (and unlike any model the library
ships numbers for), and weights large enough that every mechanism matters: sharp attention, decays spread between fast
forgetting and none, routers with decisive scores and corrections that change the choice."""
import numpy as np

from fusazen_models import write_model  # noqa: F401  (config.json + model.safetensors from a dict of arrays)


def gla(heads, dim, vdim, tau):
    return "gla", {"heads": heads, "dim": dim, "vdim": vdim, "tau": float(tau)}


def pair(left, right):
    return "parallel", {"left": left, "right": right}


def att(heads, kv_heads, dim, vdim, scale=None, conv=None, chunk=None, rot_dims=None, base=10000.0, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5)}
    if conv is not None:
        m["conv"] = conv
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    if softcap is not None:
        m["softcap"] = float(softcap)
    return m


def lin(dim, vdim, decay):
    return {"heads": len(decay), "dim": dim, "vdim": vdim, "decay": [float(d) for d in decay]}


def moe(ff, experts, top, scale=1.0, identity=None, shared=None):
    r = {"experts": experts, "top": top, "scale": float(scale)}
    if identity is not None:
        r["identity"] = identity
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def config(width, vocab, layers, eps=1e-5, mult=1.0):
    return {"architecture": "Renitar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": float(mult),
            "layers": [{"type": t, "mixer": m, "mlp": f} for (t, m), f in layers]}


# one mechanism at a time
GLA = config(40, 83, [(gla(3, 12, 20, 4.0), None)], mult=0.8)                                       # the general recurrence kernel (20 values a head)
GLA_LANES = config(48, 71, [(gla(2, 40, 32, 10.0), None), (gla(1, 96, 48, 1.0), None)], mult=0.6)   # the register form: one and two chunks of key channels
PAIR = config(48, 97, [(pair(att(4, 2, 8, 12, scale=0.9, conv=3, chunk=10, rot_dims=4, base=300.0, softcap=5.0), lin(8, 8, [0.5, 0.97])), None)],
              mult=0.5)
PAIR_BARE = config(36, 61, [(pair(att(3, 3, 6, 10), lin(12, 4, [1.0])), None)], mult=1.0)           # no convolution, mask, rotation or cap; a head that forgets nothing
EXPERTS = config(40, 90, [(gla(2, 8, 8, 2.0), moe(16, 5, 3, scale=2.0, identity=2, shared=24)),
                          (gla(1, 16, 16, 8.0), moe(12, 4, 1, scale=0.5)),                           # no identity, no shared expert, one choice
                          (gla(2, 4, 12, 3.0), moe(8, 2, 4, scale=1.0, identity=3, shared=8))],      # more experts that hand on than experts with matrices; all but one chosen
                 mult=0.7)
# layers unlike each other; blocks of positions that divide no page, of one position, as long as a page, longer than a page;
# one, two and five taps
MIXED = config(56, 120, [(pair(att(4, 2, 12, 8, conv=5, chunk=70, rot_dims=12, base=1000.0, softcap=20.0), lin(8, 12, [0.9, 0.6, 0.999])), moe(24, 6, 2, scale=1.5, identity=1, shared=16)),
                         (gla(2, 12, 16, 5.0), None),
                         (pair(att(2, 1, 16, 16, conv=1, chunk=1, rot_dims=8), lin(16, 8, [0.3, 0.8])), moe(16, 3, 2, scale=2.5)),
                         (pair(att(6, 3, 8, 4, conv=2, chunk=64, softcap=3.0), lin(4, 4, [0.95])), None),
                         (gla(4, 8, 4, 32.0), moe(8, 8, 3, scale=1.0, identity=2)),
                         (pair(att(2, 2, 20, 12, chunk=130, rot_dims=20, base=77.0), lin(12, 20, [0.99, 0.5])), moe(16, 4, 2, scale=1.0, shared=40))],
               eps=1e-4, mult=0.4)
# sizes of the kind the fast kernels take (multiples of 16 and 64), several layers
WIDE = config(128, 300, [(gla(2, 64, 64, 12.0), moe(64, 8, 2, scale=1.25, identity=3, shared=128)),
                         (pair(att(4, 1, 64, 32, scale=0.2, conv=4, chunk=100, rot_dims=32, softcap=15.0), lin(64, 64, [0.7, 0.99])), moe(128, 4, 2, scale=1.0, identity=1)),
                         (gla(4, 32, 32, 8.0), None),
                         (pair(att(8, 2, 32, 64, conv=4, chunk=40, rot_dims=16, base=50000.0), lin(32, 16, [0.9, 0.8, 0.95, 0.999])), moe(64, 16, 4, scale=2.0, shared=64))],
              mult=0.5)
# sizes that fit no fast kernel: rows of odd byte counts, head counts that divide nothing
ODD = config(36, 77, [(gla(5, 6, 7, 3.0), moe(10, 3, 2, scale=1.3, identity=1, shared=7)),
                      (pair(att(5, 5, 6, 9, conv=3, chunk=11, rot_dims=2, base=50.0, softcap=7.0), lin(5, 3, [0.8, 0.6, 0.9])), moe(22, 5, 2, scale=0.9))],
             eps=1e-6, mult=0.9)
# a width and sizes that are no multiples of four: nothing is aligned to 16 bytes
UNALIGNED = config(50, 101, [(gla(3, 7, 9, 6.0), moe(11, 3, 2, scale=1.1, identity=2, shared=13)),
                             (pair(att(2, 1, 10, 6, conv=2, chunk=9, rot_dims=6, softcap=9.0), lin(5, 7, [0.7, 0.93])), moe(9, 2, 1, scale=1.7))],
                   mult=0.6)
CONFIGS = {"unaligned": UNALIGNED, "gla": GLA, "gla_lanes": GLA_LANES, "pair": PAIR, "pair_bare": PAIR_BARE, "experts": EXPERTS, "mixed": MIXED,
           "wide": WIDE, "odd": ODD}


def make_weights(cfg, seed, rank=None):
    """name -> float32 array.  ``rank``: the size of the decay's low-rank path (default: unlike width / 16)."""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]
    w = {}

    def mat(name, out, inp, gain=1.0):
        w[name] = (rng.standard_normal((out, inp)) * gain / np.sqrt(inp)).astype(np.float32)

    def vec(name, n, mean=0.0, std=1.0):
        w[name] = (mean + std * rng.standard_normal(n)).astype(np.float32)

    w["embed"] = rng.standard_normal((V, W)).astype(np.float32)
    mat("head", V, W, 2.0)
    vec("final.norm", W, 0.0, 0.2)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        vec(p + "norm1", W, 0.0, 0.2)
        if layer["type"] == "gla":
            H, D, Dv = m["heads"], m["dim"], m["vdim"]
            R = rank or (W // 16 + 3)
            mat(p + "mix.q", H * D, W, 2.0)
            mat(p + "mix.k", H * D, W, 2.0)
            mat(p + "mix.v", H * Dv, W)
            mat(p + "mix.g", H * Dv, W, 2.0)
            mat(p + "mix.o", W, H * Dv)
            vec(p + "mix.norm", Dv, 1.0, 0.2)
            mat(p + "mix.a1", R, W)
            mat(p + "mix.a2", H * D, R, 2.0)
            # logistic(z)^(1/tau) from about 0.3 to 0.999: biases that grow with tau
            w[p + "mix.a2.b"] = (rng.uniform(-1.0, 4.0, H * D) + np.log(m["tau"])).astype(np.float32)
        else:
            a, r = m["left"], m["right"]
            H, G, D, Dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            q = p + "mix.left."
            mat(q + "q", H * D, W, 3.0)
            mat(q + "k", G * D, W, 3.0)
            mat(q + "v", G * Dv, W)
            mat(q + "g", H * Dv, W, 2.0)
            mat(q + "o", W, H * Dv)
            vec(q + "q.b", H * D, 0.0, 0.3)
            vec(q + "k.b", G * D, 0.0, 0.3)
            vec(q + "v.b", G * Dv, 0.0, 0.3)
            vec(q + "o.b", W, 0.0, 0.3)
            vec(q + "q.norm", H * D, 1.5, 0.3)
            vec(q + "k.norm", G * D, 1.5, 0.3)
            if a.get("conv"):
                for n, c in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                    w[q + n + ".conv"] = (rng.standard_normal((c, a["conv"])) * 0.6).astype(np.float32)
            Hr, Dr, Dvr = r["heads"], r["dim"], r["vdim"]
            q = p + "mix.right."
            mat(q + "q", Hr * Dr, W, 2.0)
            mat(q + "k", Hr * Dr, W, 2.0)
            mat(q + "v", Hr * Dvr, W)
            mat(q + "g", Hr * Dvr, W, 2.0)
            mat(q + "o", W, Hr * Dvr)
            vec(q + "norm", Hr * Dvr, 1.0, 0.2)
            vec(p + "mix.left.out", W, 1.0, 0.2)
            vec(p + "mix.right.out", W, 1.0, 0.2)
        mlp = layer["mlp"]
        if mlp is not None:
            F, r = mlp["expert"]["ff"], mlp["router"]
            n_out = r["experts"] + (r.get("identity") or 0)
            for e in range(r["experts"]):
                mat(f"{p}mlp.e{e}.up", F, W, 2.0)
                mat(f"{p}mlp.e{e}.down", W, F)
            mat(p + "mlp.router", n_out, W, 4.0)
            vec(p + "mlp.correction", n_out, 0.0, 0.15)
            if mlp.get("shared"):
                mat(p + "mlp.shared.up", mlp["shared"]["ff"], W, 2.0)
                mat(p + "mlp.shared.down", W, mlp["shared"]["ff"])
                mat(p + "mlp.shared.sg", 1, W, 2.0)
    return w
