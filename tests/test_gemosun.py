"""The Gemosun design on the CPU: its configuration and what it refuses, the recipe and its tensor table, random
folders, the cache's rows per block of positions, and the plain implementation's own mechanisms."""
import copy

import numpy as np
import pytest

import gemosun_models as M
import plain_gemosun as G


def test_configuration_reads_every_size_and_refuses_what_is_missing():
    from llmi_b200.config import ConfigError
    from llmi_b200.config.registry import parse_config
    arch, c = parse_config(M.MIXED)
    assert arch.name == "Gemosun" and c.width == 56 and c.vocab == 120 and c.norm_eps == 1e-4 and len(c.layers) == 5
    a = c.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.window, a.pool, a.rot_dims, a.rot_base) == (4, 2, 12, 70, 5, 12, 1000.0)
    assert a.rot_scaling.factor == 8.0 and a.rot_scaling.original == 32 and c.layers[1].mixer.rot_scaling is None
    f = c.layers[1].mlp
    assert (f.kind, f.ff, f.experts, f.top, f.groups, f.keep, f.shared_ff) == ("moe", 24, 8, 3, 2, 1, 16)
    assert c.layers[2].mlp is None and c.layers[4].mlp.shared_ff == 0 and c.layers[2].mixer.rot_dims == 4
    no_mask = parse_config(M.NO_MASK)[1].layers[0].mixer
    assert (no_mask.window, no_mask.pool, no_mask.rot_dims) == (0, 0, 0)
    for path, value in ((("width",), None), (("layers", 0, "mixer", "heads"), 0), (("layers", 0, "mixer", "kv_heads"), 3),
                        (("layers", 0, "mixer", "vdim"), 13), (("layers", 0, "mixer", "rot", "dims"), 14),
                        (("layers", 0, "mixer", "rot", "dims"), 5), (("layers", 0, "mixer", "scale"), "x"),
                        (("layers", 0, "mixer", "mask", "size"), 0), (("layers", 0, "mixer", "rot", "scaling", "factor"), None),
                        (("layers", 1, "mlp", "router", "top"), 9), (("layers", 1, "mlp", "router", "groups", "count"), 3),
                        (("layers", 1, "mlp", "router", "groups", "keep"), 3), (("layers", 1, "mlp", "kind"), "sparse"),
                        (("layers", 1, "mlp", "expert"), None), (("layers", 0, "type"), "delta"), (("norm",), {})):
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
    few = copy.deepcopy(M.MIXED)
    few["layers"][1]["mlp"]["router"].update(top=5)           # the one kept group holds four experts
    with pytest.raises(ConfigError):
        parse_config(few)


def test_recipe_and_tensor_table():
    from llmi_b200.config.registry import parse_config
    from llmi_b200.parts.build import expected_tensors
    from llmi_b200.parts.registry import resolved_shape
    for name, cfg in M.CONFIGS.items():
        arch, c = parse_config(cfg)
        spec = arch.model_spec(c)
        assert [e.layer for e in spec.schedule] == list(range(len(cfg["layers"])))
        assert all(e.after.kind == "depth_average" and e.after.params["index"] == i for i, e in enumerate(spec.schedule))
        decl = expected_tensors(spec)
        made = M.make_weights(cfg, 1)
        assert set(decl) == set(made), name
        for n, d in decl.items():
            assert resolved_shape(d.shape) == made[n].shape, (name, n)
        assert all(layer.block == "parallel" for layer in spec.layers)
    spec = parse_config(M.WINDOW_POOL)[0].model_spec(parse_config(M.WINDOW_POOL)[1])
    assert spec.layers[0].ffn is None and spec.layers[0].ffn_norm is None
    assert spec.layers[0].mixer.params["position"].kind == "rotary_pairs"
    assert parse_config(M.NO_MASK)[0].model_spec(parse_config(M.NO_MASK)[1]).layers[0].mixer.params["position"].kind == "none"


def test_random_folder_round_trip(tmp_path):
    import torch
    from llmi_b200 import write_random_model
    from llmi_b200.config.registry import read_model_config
    from llmi_b200.parts.build import expected_tensors
    from llmi_b200.weights.safetensors_io import SafetensorsFile
    d = write_random_model(str(tmp_path / "m"), M.EXPERTS, seed=3, dtype=torch.bfloat16)
    arch, c = read_model_config(d)
    f = SafetensorsFile(str(tmp_path / "m" / "model.safetensors"))
    try:
        assert set(f.names()) == set(expected_tensors(arch.model_spec(c)))
    finally:
        f.close()


def test_rows_per_block_of_positions_in_the_page_pool():
    """A group that keeps one row per block of ``every`` positions takes a page when a block's row opens one, counts
    lengths in positions, and undoes a reserved position exactly."""
    from llmi_b200.cache.pages import CacheError, PagePool
    for every in (1, 3, 8, 64, 100):
        pool = PagePool(6, page_size=4, every=every)
        pool.open(0)
        held = []
        for n in range(1, 4 * every * 5 + 1):
            need = pool.pages_needed(0, 1)
            base = np.array([n - 1])
            takes, gives = pool.page_events(base)
            assert bool(takes[0]) == (need == 1) and gives[0] == 0
            before = len(pool.table(0))
            pool.extend(0, 1)
            assert len(pool.table(0)) == -(-(n // every) // 4) == before + need
            pool.extend(0, 1)
            pool.shrink_by_one(0)                               # a position reserved ahead and taken back
            assert pool.length(0) == n and len(pool.table(0)) == -(-(n // every) // 4)
            held.append(len(pool.table(0)))
        pool.check()
        pool.close(0)
        assert pool.n_free == 6
        pool.open(1)
        assert pool.extend(1, 4 * every * 6) == 0 and len(pool.table(1)) == 6      # many positions at once
        with pytest.raises(CacheError):
            pool.extend(1, 4 * every)
    with pytest.raises(CacheError):
        PagePool(4, page_size=4, window=8, every=2)


def test_what_a_query_sees():
    assert G.visible(5, None, None) == (list(range(6)), [])
    assert G.visible(9, 4, None) == ([6, 7, 8, 9], [])
    assert G.visible(9, 4, 3) == ([6, 7, 8, 9], [0, 1])          # block 1 ends at 5 = 9 - 4
    assert G.visible(10, 4, 3) == ([7, 8, 9, 10], [0, 1])        # position 6 has left the window; its block (6..8) is not whole before it
    assert G.visible(12, 4, 3) == ([9, 10, 11, 12], [0, 1, 2])
    assert G.visible(2, 4, 3) == ([0, 1, 2], [])
    assert G.visible(7, 1, 1) == ([7], list(range(7)))


def test_routing_of_the_plain_implementation():
    s = np.array([0.9, 0.1, 0.2, 0.8, 0.85, 0.3])
    assert G.route(s, 2, None)[0] == [0, 4]
    chosen, wt = G.route(s, 2, {"count": 3, "keep": 1})           # runs (0,1) (2,3) (4,5): sums 1.0, 1.0, 1.15
    assert chosen == [4, 5] and abs(wt.sum() - 1) < 1e-12 and abs(wt[0] - 0.85 / 1.15) < 1e-12
    assert G.route(s, 3, {"count": 3, "keep": 2})[0] == [0, 4, 5]   # a tie of two runs goes to the lower one
    assert G.route(s, 1, {"count": 6, "keep": 2})[0] == [0]       # runs of one expert


def test_rotation_frequencies_of_the_plain_implementation():
    f, mult = G.rotation_frequencies({"dims": 8, "base": 100.0})
    assert mult == 1.0 and np.allclose(f, [1.0, 100 ** -0.25, 0.1, 100 ** -0.75])
    f2, mult2 = G.rotation_frequencies({"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    assert abs(mult2 - (0.1 * np.log(4.0) + 1)) < 1e-12
    assert f2[0] == f[0] and abs(f2[-1] - f[-1] / 4) < 1e-15 and np.all(f2 <= f) and np.all(f2 >= f / 4)
    x = np.arange(6, dtype=np.float64)[None, :] + 1
    y = G.rotate_pairs(x, 3, np.array([0.5, 0.25]), 2.0, 4)
    assert np.allclose(y[0, 4:], x[0, 4:]) and np.allclose(np.hypot(y[0, 0], y[0, 1]), 2 * np.hypot(1, 2))
