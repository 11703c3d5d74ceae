"""The Renitar design on the CPU: its configuration and what it refuses, the recipe and its tensor table, random
folders, and the plain implementation's own mechanisms."""
import copy

import numpy as np
import pytest

import plain_renitar as G
import renitar_models as M


def test_configuration_reads_every_size_and_refuses_what_is_missing():
    from llmi_b200.config import ConfigError
    from llmi_b200.config.registry import parse_config
    arch, c = parse_config(M.MIXED)
    assert arch.name == "Renitar" and c.width == 56 and c.vocab == 120 and c.norm_eps == 1e-4 and len(c.layers) == 6
    assert c.residual_mult == 0.4
    a, r = c.layers[0].mixer.left, c.layers[0].mixer.right
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.taps, a.chunk, a.rot_dims, a.rot_base, a.softcap) == (4, 2, 12, 8, 5, 70, 12, 1000.0, 20.0)
    assert (r.heads, r.dim, r.vdim, r.decay) == (3, 8, 12, (0.9, 0.6, 0.999))
    g = c.layers[1].mixer
    assert (g.heads, g.dim, g.vdim, g.tau, g.rank) == (2, 12, 16, 5.0, 0) and c.layers[1].mlp is None
    f = c.layers[0].mlp
    assert (f.ff, f.experts, f.identity, f.top, f.scale, f.shared_ff) == (24, 6, 1, 2, 1.5, 16)
    assert c.layers[2].mlp.identity == 0 and c.layers[2].mlp.shared_ff == 0
    bare = parse_config(M.PAIR_BARE)[1].layers[0].mixer.left
    assert (bare.taps, bare.chunk, bare.rot_dims, bare.softcap) == (0, 0, 0, 0.0)
    zeros = copy.deepcopy(M.PAIR)                      # 0 says "none" as well as a missing key does
    zeros["layers"][0]["mixer"]["left"].update(conv=0, softcap=0, rot={"dims": 0})
    z = parse_config(zeros)[1].layers[0].mixer.left
    assert (z.taps, z.rot_dims, z.softcap) == (0, 0, 0.0)
    for path, value in ((("width",), None), (("residual_mult",), None), (("norm",), {}), (("layers", 0, "type"), "delta"),
                        (("layers", 0, "mixer", "left", "heads"), 0), (("layers", 0, "mixer", "left", "kv_heads"), 3),
                        (("layers", 0, "mixer", "left", "rot", "dims"), 14), (("layers", 0, "mixer", "left", "rot", "dims"), 5),
                        (("layers", 0, "mixer", "left", "scale"), "x"), (("layers", 0, "mixer", "left", "mask", "size"), 0),
                        (("layers", 0, "mixer", "left", "conv"), 17), (("layers", 0, "mixer", "left", "softcap"), -1.0),
                        (("layers", 0, "mixer", "right", "decay"), [0.5, 0.5]), (("layers", 0, "mixer", "right", "decay"), [0.5, 0.5, -0.5]),
                        (("layers", 0, "mixer", "right"), None), (("layers", 1, "mixer", "tau"), 0), (("layers", 1, "mixer", "vdim"), None),
                        (("layers", 0, "mlp", "router", "top"), 8), (("layers", 0, "mlp", "kind"), "dense"),
                        (("layers", 0, "mlp", "router", "scale"), None), (("layers", 0, "mlp", "expert"), None)):
        bad = copy.deepcopy(M.MIXED)
        node = bad
        for key in path[:-1]:
            node = node[key]
        if value is None:
            del node[path[-1]]
        else:
            node[path[-1]] = value
        with pytest.raises(ConfigError):
            parse_config(bad)


def test_recipe_and_tensor_table():
    from llmi_b200.config.registry import parse_config
    from llmi_b200.parts.build import expected_tensors
    from llmi_b200.parts.registry import FreeDim, resolved_shape
    for name, cfg in M.CONFIGS.items():
        arch, c = parse_config(cfg)
        spec = arch.model_spec(c)
        assert [e.layer for e in spec.schedule] == list(range(len(cfg["layers"])))
        assert all(ls.block == "parallel_scaled" and ls.block_params == {"residual_mult": cfg["residual_mult"]} for ls in spec.layers)
        assert all(ls.ffn_norm is None and ls.mixer_norm.params["one_plus"] for ls in spec.layers)
        decl = expected_tensors(spec)
        made = M.make_weights(cfg, 1)
        assert set(decl) == set(made), name
        for n, d in decl.items():
            want = tuple(made[n].shape)
            assert len(d.shape) == len(want), n
            for a, b in zip(d.shape, want):
                assert isinstance(a, FreeDim) or a == b, (name, n, d.shape, want)      # (the low-rank path's size is the file's)
            assert len(resolved_shape(d.shape)) == len(want)


def test_a_random_folder_has_the_recipes_tensors(tmp_path):
    from llmi_b200.config.registry import parse_config
    from llmi_b200.parts.build import expected_tensors
    from llmi_b200.parts.registry import resolved_shape
    from llmi_b200.weights.random_weights import write_random_model
    from llmi_b200.weights.safetensors_io import SafetensorsFile
    cfg = M.CONFIGS["mixed"]
    write_random_model(str(tmp_path), cfg, seed=3)
    arch, c = parse_config(cfg)
    decl = expected_tensors(arch.model_spec(c))
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    try:
        assert set(f.names()) == set(decl)
        for n, d in decl.items():
            assert tuple(f.tensor(n).shape) == resolved_shape(d.shape), n
    finally:
        f.close()


# ---------------------------------------------------------------------------------- the oracle's own mechanisms

def test_the_recurrence_is_linear_attention_with_decayed_weights():
    """o_t = sum_{j <= t} (q_t * prod_{j < i <= t} w_i) . k_j  v_j: the recurrence against the sum written out."""
    rng = np.random.default_rng(0)
    T, dk, dv = 9, 5, 3
    q, k, v = rng.standard_normal((T, dk)), rng.standard_normal((T, dk)), rng.standard_normal((T, dv))
    w = rng.uniform(0.2, 1.0, (T, dk))
    o = G.linear_recurrence(q, k, v, w)
    for t in range(T):
        ref = np.zeros(dv)
        for j in range(t + 1):
            ref += ((q[t] * np.prod(w[j + 1:t + 1], axis=0)) @ k[j]) * v[j]
        assert np.abs(o[t] - ref).max() < 1e-12
    o1 = G.linear_recurrence(q, k, v, 0.7)
    assert np.abs(o1 - G.linear_recurrence(q, k, v, np.full((T, dk), 0.7))).max() < 1e-12


def test_blocks_of_positions_rotation_convolution_and_routing():
    assert [j for j in range(12) if G.sees(11, j, 5)] == [10, 11] and [j for j in range(12) if G.sees(9, j, 5)] == [5, 6, 7, 8, 9]
    assert all(G.sees(7, j, 0) for j in range(8)) and not G.sees(3, 4, 0) and not G.sees(5, 4, 5)
    x = np.arange(1.0, 13.0).reshape(2, 6)
    y = G.rotate_half(x, 3, 100.0, 4)
    assert np.allclose(y[:, 4:], x[:, 4:]) and np.allclose(np.hypot(y[:, 0], y[:, 2]), np.hypot(x[:, 0], x[:, 2]))
    assert np.allclose(y[0, 0], x[0, 0] * np.cos(3.0) - x[0, 2] * np.sin(3.0)) and np.allclose(G.rotate_half(x, 0, 100.0, 4), x)
    assert np.allclose(y[0, 1], x[0, 1] * np.cos(0.3) - x[0, 3] * np.sin(0.3))
    u = np.arange(1.0, 9.0).reshape(4, 2)
    w = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 2.0]])
    c = G.short_conv(u, w)
    assert np.allclose(c[:, 1], 2 * u[:, 1]) and np.allclose(c[:, 0], [100.0, 310.0, 531.0, 753.0])
    z = np.array([1.0, 0.9, 0.0, -1.0])
    s = G.softmax(z)
    assert G.route(z, np.zeros(4), 2, 3.0) == ([0, 1], [3 * s[0], 3 * s[1]])
    chosen, wts = G.route(z, np.array([0.0, 0.0, 0.5, 0.0]), 2, 1.0)        # the correction changes the choice, not the weights
    assert chosen == [2, 0] and np.allclose(wts, [s[2], s[0]])
    assert G.route(np.zeros(3), np.zeros(3), 2, 1.0)[0] == [0, 1]           # ties: the lower index


def test_experts_that_hand_their_input_on():
    cfg = M.CONFIGS["experts"]
    w = {k: v.astype(np.float64) for k, v in M.make_weights(cfg, 2).items()}
    mlp = copy.deepcopy(cfg["layers"][2]["mlp"])
    h = np.random.default_rng(1).standard_normal((7, cfg["width"]))
    full = G.mixture(mlp, w, "l2.mlp.", h)
    for n in ("router", "correction"):                     # only the outputs that stand for experts without tensors
        w["x." + n] = w["l2.mlp." + n][2:]
    for n in ("shared.up", "shared.down", "shared.sg"):
        w["x." + n] = w["l2.mlp." + n]
    only = copy.deepcopy(mlp)
    only["router"].update(experts=0, identity=3, top=3)
    y = G.mixture(only, w, "x.", h)
    shared = G.expert(w, "x.shared.", h) * G.sigmoid(h @ w["x.shared.sg"].T)
    assert np.allclose(y - shared, h)                      # all three chosen: their scores sum to one
    assert full.shape == h.shape and np.isfinite(full).all()
