"""The Gemosun design in the library against the plain implementation of tests/plain_gemosun.py (GPU).

Every mechanism alone and together, however the work is cut: whole prompts, token by token, portions down to two
tokens, unequal batches, slots and pages that are used again (caches are poisoned with NaN before a replay), lengths at
page borders and at the borders of windows and pooled blocks, the first tokens, long decoding, greedy generation through
the library's own entry point.  32-bit runs must agree with the float64 oracle row by row; bf16 runs agree to bf16's
precision.
"""
import numpy as np
import pytest

import gemosun_models as M
import helpers as H
import plain_gemosun as G

pytestmark = pytest.mark.gpu

TOL32 = 3e-5
TOL16 = 5e-2
STORAGE = {"float32": "F32", "bfloat16": "BF16"}
LENGTHS = [1, 2, 3, 5, 31, 63, 64, 65, 100, 129, 200]


def requests_for(cfg, lengths=LENGTHS, seed=5):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def loaded(tmp_path_factory):
    import llmi_b200 as L
    made = {}

    def get(name, dtype, lengths=LENGTHS):
        key = (name, dtype, tuple(lengths))
        if key not in made:
            cfg = M.CONFIGS[name]
            d = str(tmp_path_factory.mktemp(f"gemosun_{name}_{dtype}"))
            w = M.write_model(d, cfg, M.make_weights(cfg, 7), STORAGE[dtype])
            reqs = requests_for(cfg, lengths)
            refs = {r: G.forward(cfg, w, t) for r, t in reqs.items()}
            made[key] = (L.load(d, dtype), reqs, refs, cfg, w)
        return made[key]
    return get


def check(got, refs, dtype):
    assert set(got) == set(refs)
    errs = []
    for r in refs:
        assert got[r].shape == refs[r].shape
        assert np.isfinite(got[r]).all(), f"{r}: non-finite logits (something outside the sequence's own positions was read)"
        err = np.abs(got[r] - refs[r]).max(axis=1) / np.abs(refs[r]).max()
        if dtype == "float32":
            assert err.max() < TOL32, (r, int(err.argmax()), float(err.max()))
        errs.extend(err.tolist())
    if dtype != "float32":
        # bf16 rounds activations to 2^-9 of their size: the typical row is well inside, nine of ten inside, and all but
        # one row in fifty near — a router whose best scores nearly tie may choose another expert in bf16 than the
        # float64 oracle does, and such a row (and what follows it through the cache) is off by more
        e = np.asarray(errs)
        assert float(np.median(e)) < TOL16 / 4 and float(np.quantile(e, 0.9)) < TOL16 and float(np.quantile(e, 0.98)) < 5 * TOL16, (
            float(np.median(e)), float(np.quantile(e, 0.9)), float(np.quantile(e, 0.98)), float(e.max()))


ALL = list(M.CONFIGS)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ALL)
def test_whole_prompts(loaded, name, dtype):
    model, reqs, refs, _, _ = loaded(name, dtype)
    steps, most = H.trace_whole(reqs)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ALL)
def test_prompt_then_token_by_token(loaded, name, dtype):
    """Most of a request in one step, its last 40 tokens one by one: windows pass over decoded tokens, blocks are
    completed by single tokens."""
    model, reqs, refs, _, _ = loaded(name, dtype)
    steps, most = H.trace_last_decoded(reqs, n_last=40)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("portion", [2, 3, 7, 64, 100])
@pytest.mark.parametrize("name", ["window_pool", "window", "dense", "experts", "mixed", "wide"])
def test_prompts_in_portions(loaded, name, portion):
    """A block of positions whose first positions came in an earlier portion is summed up when its last one comes."""
    model, reqs, refs, _, _ = loaded(name, "float32")
    if portion < 7:
        reqs = {r: t for r, t in reqs.items() if len(t) <= 70}
    steps, most = H.trace_portions(reqs, portion, n_last=3)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), {r: refs[r] for r in reqs}, "float32")


@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_prompts_in_portions_bf16(loaded, name):
    model, reqs, refs, _, _ = loaded(name, "bfloat16")
    steps, most = H.trace_portions(reqs, 33, n_last=3)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["window_pool", "experts", "mixed", "wide", "odd"])
def test_unequal_batches_one_after_another(loaded, name, dtype):
    """Batches of four requests of unequal lengths, prompts of unequal parts of them, decoded together; the next batch
    takes the slots and pages (of positions and of pooled blocks) that the one before gave back."""
    model, reqs, refs, _, _ = loaded(name, dtype)
    prompt_lens = {r: max(1, len(t) * (i % 3 + 1) // 4) for i, (r, t) in enumerate(reqs.items())}
    steps, most = H.trace_batches(reqs, 4, prompt_lens)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("name", ["window_pool", "experts", "mixed", "wide"])
def test_portions_beside_decoding(loaded, name):
    model, reqs, refs, _, _ = loaded(name, "float32")
    ids = list(reqs)
    first = {r: max(1, len(reqs[r]) // 3) for r in ids}
    portion = {r: (1, 5, 2, 33)[i % 4] for i, r in enumerate(ids)}
    steps, most = H.trace_mixed(reqs, first, portion)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(loaded, dtype):
    """Two tokens of prompt, then 300 steps of one token: pages are taken at 64, 128, ..., pages behind the window go
    back while decoding, and every pooled block is made by a single token."""
    model, reqs, refs, _, _ = loaded("mixed", dtype, lengths=[302, 150])
    steps, most = H.trace_batches(reqs, 2, {r: 2 for r in reqs})
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


def test_pages_behind_the_window_go_back_early(loaded):
    """A cache with far fewer pages than the request has positions holds it all the same: the window's pages and one
    row per pooled block are all a sequence keeps."""
    import llmi_b200 as L
    from llmi_b200.engine.batch import SequenceStep
    model, _, _, cfg, w = loaded("window_pool", "float32")
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], 700).tolist()
    ref = G.forward(cfg, w, toks)
    cache = model.new_cache(4 * 64, n_slots=2)             # four pages for 700 positions
    slot = cache.alloc_slot()
    got = [model.step(cache, [SequenceStep(slot, toks[:100], list(range(100)))]).cpu().numpy().copy()]
    for a in range(100, 700, 50):
        got.append(model.step(cache, [SequenceStep(slot, toks[a:a + 50], list(range(50)))]).cpu().numpy().copy())
    check({"a": np.concatenate(got)}, {"a": ref}, "float32")
    cache.free_slot(slot)
    cache.check()
    assert all(g.pool.n_free == g.pool.n_pages for g in cache.kv_groups)
    assert L is not None


@pytest.mark.parametrize("name", ["experts", "wide", "mixed"])
def test_greedy_generation_through_the_entry_point(loaded, name):
    """generate(): the scheduler's batches, recorded decode steps, the device's argmax — against the oracle's greedy loop."""
    import llmi_b200 as L
    model, _, _, cfg, w = loaded(name, "float32")
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (1, 9, 70, 4, 33)]
    new = [12, 5, 12, 1, 9]
    out = L.generate(model, prompts, max_new=new, max_batch=3)
    ref = [G.generate_greedy(cfg, w, p, n) for p, n in zip(prompts, new)]
    assert out == ref
    assert L.generate(model, prompts, max_new=new, max_batch=3, use_graphs=False) == ref


def test_recorded_steps_in_bf16_follow_the_plain_steps(loaded):
    """bf16 serving pads and records its steps (decode graphs, padded prompt steps): generation with and without them
    gives the same tokens, three times over (from the second time on everything is replayed)."""
    import llmi_b200 as L
    model, _, _, cfg, _ = loaded("wide", "bfloat16")
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (3, 40, 130, 17)]
    plain = L.generate(model, prompts, max_new=20, max_batch=4, use_graphs=False)
    for _ in range(3):
        assert L.generate(model, prompts, max_new=20, max_batch=4) == plain


def test_programs_as_a_user_calls_them(loaded, tmp_path):
    """bin/llmi-generate and bin/trace_run on a Gemosun folder, as subprocesses: the design is chosen by config.json."""
    import json
    import os
    import subprocess
    import sys
    from conftest import ROOT
    cfg = M.CONFIGS["experts"]
    d = str(tmp_path / "model")
    w = M.write_model(d, cfg, M.make_weights(cfg, 7), "F32")
    prompt = [3, 17, 80, 4, 4, 56]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llmi-generate"), d, "--ids", ",".join(map(str, prompt)),
                        "--max-new", "6", "--json", "--dtype", "fp32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1])["generated_ids"] == G.generate_greedy(cfg, w, prompt, 6)
    reqs = requests_for(cfg, [5, 70, 33])
    steps, _ = H.trace_batches(reqs, 3, {"r0": 2, "r1": 40, "r2": 33})
    out = tmp_path / "out"
    most = sum(len(t) for t in reqs.values())
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", str(most)],
                       input="".join(json.dumps(s_) + "\n" for s_ in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    outs = []
    for s_ in steps:
        n = sum(len(e["want"]) for e in s_["entries"])
        outs.append(np.fromfile(out / f"{s_['step']}.f32", dtype="<f4").reshape(n, -1) if n else None)
    check(H.collect(steps, outs, cfg["vocab"]), {r: G.forward(cfg, w, t) for r, t in reqs.items()}, "float32")


def test_a_file_that_keeps_a_norm_for_a_missing_feed_forward_loads(tmp_path):
    import llmi_b200 as L
    cfg = M.CONFIGS["window_pool"]
    w = M.make_weights(cfg, 3)
    w["l0.norm2"] = np.ones(cfg["width"], dtype=np.float32)
    d = str(tmp_path / "m")
    wf = M.write_model(d, cfg, w, "F32")
    model = L.load(d, "float32")
    toks = list(range(40))
    steps, most = H.trace_whole({"a": toks})
    check(H.collect(steps, H.replay(model, steps, most), cfg["vocab"]), {"a": G.forward(cfg, wf, toks)}, "float32")


# ----------------------------------------------------------------------------- kernels alone

class _Ctx:
    pass


def _one_sequence_ctx(n_rows, first_pos, decode):
    """The index arrays of a step that brings ``n_rows`` tokens of one sequence from position ``first_pos`` on."""
    import torch
    ctx = _Ctx()
    ctx.decode = decode
    ctx.n_seqs = 1
    ctx.tok_seq = torch.zeros(n_rows, dtype=torch.int32, device="cuda:0")
    ctx.tok_pos = torch.arange(first_pos, first_pos + n_rows, dtype=torch.int32, device="cuda:0")
    ctx.seq_q_start = torch.tensor([0, n_rows], dtype=torch.int32, device="cuda:0")
    ctx.seq_kv_len = torch.tensor([first_pos + n_rows], dtype=torch.int32, device="cuda:0")
    ctx.seq_slot = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    ctx.n_real_seqs = 1
    ctx.host_q_lens, ctx.host_kv_lens = [n_rows], [first_pos + n_rows]
    return ctx


def _paged(rows, order, page, dt, first_row=0):
    """rows [N, heads, d] -> a cache tensor [pages, heads, page, d] with the sequence's pages at ``order``; rows before
    ``first_row`` stay NaN (pages that were given back)."""
    import torch
    N, heads, d = rows.shape
    cache = torch.full((int(max(order)) + 2, heads, page, d), float("nan"), dtype=dt, device="cuda:0")
    for i, pg in enumerate(order):
        lo, hi = max(i * page, first_row), min((i + 1) * page, N)
        if hi > lo:
            cache[pg, :, lo - i * page:hi - i * page] = rows[lo:hi].permute(1, 0, 2).to("cuda:0")
    return cache


def _window_pool_reference(q, k, v, scale, window, pool, gate):
    """q [N, H, d], k, v [N, G, d] float64 -> [N, H, d]: the plain sums over what :func:`G.visible` lists."""
    N, Hq, d = q.shape
    Gk = k.shape[1]
    out = np.zeros((N, Hq, v.shape[2]))
    for t in range(N):
        toks, blocks = G.visible(t, window, pool)
        for h in range(Hq):
            g = h // (Hq // Gk)
            keys = np.array([k[pool * b:pool * (b + 1), g].mean(0) for b in blocks] + [k[j, g] for j in toks])
            vals = np.array([v[pool * b:pool * (b + 1), g].mean(0) for b in blocks] + [v[j, g] for j in toks])
            out[t, h] = G.softmax(keys @ q[t, h] * scale) @ vals * (G.sigmoid(gate[t, h]) if gate is not None else 1.0)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(2, 1, 16), (4, 2, 64), (2, 2, 128), (6, 2, 24)])
@pytest.mark.parametrize("window,pool,key", [
    (96, 8, 0), (96, 8, 199), (96, 8, 200), (96, 8, 203), (96, 8, 204),      # the query at 299 sees positions 204.. and blocks up to 25 (200..207 is block 25: not wholly before 204)
    (100, 8, 199), (100, 8, 200),                                            # 299 - 100 = 199: block 24 (192..199) is the last one seen
    (64, 64, 63), (64, 64, 191), (64, 64, 192), (64, 64, 235), (64, 64, 236),
    (37, 5, 259), (37, 5, 260), (37, 5, 262), (37, 5, 263), (1, 3, 296), (1, 3, 297), (1, 3, 298), (1, 3, 299),
    (130, 70, 69), (130, 70, 139), (130, 70, 140), (130, 70, 169), (130, 70, 170), (50, 0, 249), (50, 0, 250)])
def test_attention_sees_its_window_and_the_blocks_before_it(window, pool, key, sizes, dtype):
    """300 cached positions on pages that are not in order (pages behind the window and the newest block given back:
    NaN), pooled rows made by the library's own kernel from the cache, one position (``key``) made to stand out for the
    last head by scaling it and the query.  The query at 299 (as a single token, and as the last of a portion of 70
    tokens) must return that position's own value row when it lies in the window, the mean value of its block when the
    block lies wholly before the window, and must not see it at all in between; every row is compared with the plain sums."""
    import torch
    from llmi_b200.engine.runtime import Runtime
    from llmi_b200.ops import kernels
    Hq, Gk, d = sizes
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rng = np.random.default_rng(key + 7 * window + pool)
    N, page = 300, 64
    k = torch.tensor(rng.standard_normal((N, Gk, d)).astype(np.float32)).to(dt)
    v = torch.tensor(rng.standard_normal((N, Gk, d)).astype(np.float32)).to(dt)
    q = torch.tensor((rng.standard_normal((N, Hq, d)) * 0.3).astype(np.float32))
    others = np.arange(N) != key
    # the other keys of that head are short: short enough that none of them, seen alone, comes near the score that
    # `key` still has after it was averaged with its block's other keys
    k[others, Gk - 1] *= min(0.25, 0.05 * d ** 0.5 / max(pool, 1))
    q[:, -1] = k[key, Gk - 1].float() * (200.0 * max(pool, 1) / d)  # the score of `key` for the last head, also through its block's mean: about 100
    q = q.to(dt)
    gate = torch.tensor(rng.standard_normal((N, Hq + 3)).astype(np.float32), device="cuda:0")
    order = rng.permutation(9)[:5]
    rt = Runtime(dt, "cuda:0")
    pages = torch.tensor(order[None, :].astype(np.int32), device="cuda:0")
    pooled = None
    if pool:
        # the pooled rows, made as the model makes them: by the library's kernel, from the whole cache, in steps
        kc_all, vc_all = _paged(k, order, page, dt), _paged(v, order, page, dt)
        porder = rng.permutation(7)[:3] + 1
        k_pool = torch.full((9, Gk, page, d), float("nan"), dtype=dt, device="cuda:0")
        v_pool = torch.full((9, Gk, page, d), float("nan"), dtype=dt, device="cuda:0")
        ppages = torch.tensor(porder[None, :].astype(np.int32), device="cuda:0")
        for a, b in ((0, 1), (1, 2), (2, 131), (131, 132), (132, N)):
            kernels.pool_rows(kc_all, vc_all, pages, k_pool, v_pool, ppages, page, pool, _one_sequence_ctx(b - a, a, b - a == 1))
        pooled = (pool, k_pool, v_pool, ppages)
    kk, vv, qq = (x.float().numpy().astype(np.float64) for x in (k, v, q))
    ref = _window_pool_reference(qq, kk, vv, 0.5, window, pool, gate.cpu().numpy().astype(np.float64))
    tol = 2e-5 if dtype == "float32" else 3e-2
    for n_rows in (1, 70):
        # what the pages of positions still hold: nothing that lies wholly before the first query's window (and newest block)
        first_held = max(0, (N - n_rows) - max(window, pool) + 1) // page * page
        kc, vc = _paged(k, order, page, dt, first_held), _paged(v, order, page, dt, first_held)
        ctx = _one_sequence_ctx(n_rows, N - n_rows, n_rows == 1)
        out = torch.full((n_rows, Hq * d), float("nan"), dtype=dt, device="cuda:0")
        kernels.attention_maps(q[N - n_rows:].reshape(n_rows, -1).to("cuda:0").contiguous(), out, kc, vc, ctx, pages, page,
                               Hq, Gk, 1, d, d, 0.5, None, window, 0, rt=rt, pooled=pooled, gate=gate[N - n_rows:])
        got = out.float().cpu().numpy().reshape(n_rows, Hq, d)
        assert np.abs(got - ref[N - n_rows:]).max() < tol
        g_last = G.sigmoid(float(gate[N - 1, Hq - 1]))
        alone = np.abs(got[-1, -1] / g_last - vv[key, Gk - 1]).max() < max(tol, 1e-3) * 4
        in_window = 299 - key < window
        assert alone == in_window, (key, window)
        if pool and not in_window:
            b = key // pool
            as_block = np.abs(got[-1, -1] / g_last - vv[b * pool:(b + 1) * pool, Gk - 1].mean(0)).max() < (1e-3 if dtype == "float32" else 6e-2)
            assert as_block == (b * pool + pool - 1 <= 299 - window), (key, b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,extra", [(9, 5), (150, 4)])
@pytest.mark.parametrize("heads,kv,d,rot", [(2, 1, 8, 8), (3, 3, 12, 6), (4, 2, 64, 32), (2, 2, 10, 0), (5, 1, 128, 64), (2, 2, 16, 0)])
def test_rotation_of_neighbours_and_values_from_keys(heads, kv, d, rot, dtype, T, extra):
    """qkv_prepare with neighbouring pairs, an amplitude on cos and sin, and values that are the keys before the
    rotation, against the plain rotation; positions up to a few thousand.  Few tokens take the kernel of one entry a
    thread; many tokens with sizes in multiples of eight (and rows of whole 16 bytes: ``extra`` columns behind the
    keys) the one of eight entries a thread."""
    import torch
    from llmi_b200.ops import kernels
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rng = np.random.default_rng(d + rot)
    page, first = 64, 3000
    rot_cfg = {"dims": rot, "base": 500.0, "scaling": {"factor": 6.0, "original": 40, "fast": 4.0, "slow": 0.5}}
    f, mult = G.rotation_frequencies(rot_cfg) if rot else (np.zeros(0), 1.0)
    proj = torch.tensor(rng.standard_normal((T, (heads + kv) * d + extra)).astype(np.float32), device="cuda:0")
    n_pages = (first + T) // page + 1
    pages = torch.arange(n_pages, dtype=torch.int32, device="cuda:0")[None, :].contiguous()
    kc = torch.zeros((n_pages, kv, page, d), dtype=dt, device="cuda:0")
    vc = torch.zeros_like(kc)
    qo = torch.zeros((T, heads * d), dtype=dt, device="cuda:0")
    inv = torch.tensor(f.astype(np.float32), device="cuda:0") if rot else None
    kernels.qkv_prepare(proj, heads, kv, d, kv, d, None, None, 0.0, inv, rot, _one_sequence_ctx(T, first, False), pages, page, kc, vc, qo,
                        pairing=1, amplitude=float(mult), v_from_k=True)
    pr = proj.cpu().numpy().astype(np.float64)
    tol = 2e-4 if dtype == "float32" else 2e-2          # (an angle of thousands of radians in fp32 is good to about 1e-4)
    for t in range(T):
        pos = first + t
        qr, kr = pr[t, :heads * d].reshape(heads, d), pr[t, heads * d:(heads + kv) * d].reshape(kv, d)
        q_ref = G.rotate_pairs(qr, pos, f.astype(np.float32).astype(np.float64), mult, rot) if rot else qr
        k_ref = G.rotate_pairs(kr, pos, f.astype(np.float32).astype(np.float64), mult, rot) if rot else kr
        assert np.abs(qo[t].float().cpu().numpy().reshape(heads, d) - q_ref).max() < tol * 5
        assert np.abs(kc[pos // page, :, pos % page].float().cpu().numpy() - k_ref).max() < tol * 5
        assert np.abs(vc[pos // page, :, pos % page].float().cpu().numpy() - kr).max() < (1e-6 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("E,top,groups", [(6, 2, (3, 2)), (12, 3, (2, 1)), (8, 3, None), (5, 5, None), (16, 2, (16, 3)), (64, 6, (8, 4)), (40, 1, (4, 4))])
def test_experts_are_chosen_by_score_within_the_best_groups(E, top, groups):
    import torch
    from llmi_b200.ops import kernels
    rng = np.random.default_rng(E + top)
    T = 50
    z = rng.standard_normal((T, E + 1)).astype(np.float32) * 2
    logits = torch.tensor(z, device="cuda:0")
    ctx = _one_sequence_ctx(T, 0, False)
    ctx.tok_seq[7] = -1
    idx = torch.zeros((T, top), dtype=torch.int32, device="cuda:0")
    wt = torch.zeros((T, top), dtype=torch.float32, device="cuda:0")
    kernels.moe_route(logits, top, ctx, idx, wt, kernels.ROUTE_LOGISTIC_NORMALISED, groups[0] if groups else 0,
                      groups[1] if groups else 0, experts=E)
    idx, wt = idx.cpu().numpy(), wt.cpu().numpy()
    for t in range(T):
        if t == 7:
            assert (idx[t] == -1).all() and (wt[t] == 0).all()
            continue
        chosen, weights = G.route(G.sigmoid(z[t, :E].astype(np.float64)), top, {"count": groups[0], "keep": groups[1]} if groups else None)
        assert idx[t].tolist() == chosen
        assert np.abs(wt[t] - weights).max() < 1e-6


@pytest.mark.parametrize("act", ["relu2", "silu"])
@pytest.mark.parametrize("T,E,top,W,F", [(600, 4, 2, 128, 128), (1500, 8, 2, 256, 192), (520, 3, 2, 136, 200), (300, 12, 4, 384, 136),
                                         (700, 5, 2, 64, 256), (2100, 16, 1, 192, 320)])
def test_experts_without_a_gate_matrix_for_many_tokens(T, E, top, W, F, act):
    """The grouped form for many (token, choice) items — from 1,024 items on and 128-wide sizes the tcgen05 tiles, else
    the mma.sync tiles — against the sum written out in float64: experts with most of the items, with a few, with none;
    sizes that end inside a tile in every direction; rows of no sequence get zeros."""
    import torch
    from llmi_b200.engine.runtime import Runtime
    from llmi_b200.ops import kernels
    rt = Runtime(torch.bfloat16, "cuda:0")
    gen = torch.Generator(device="cuda:0").manual_seed(T + E)

    def rnd(*shape, gain=1.0):
        return (torch.randn(*shape, generator=gen, device="cuda:0") * gain).to(torch.bfloat16)
    h, wu, wd = rnd(T, W), rnd(E, F, W, gain=W ** -0.5), rnd(E, W, F, gain=F ** -0.5)
    # unequal loads: expert 0 is in most tokens' choices, the last expert in none
    score = torch.rand(T, E, generator=gen, device="cuda:0")
    score[:, 0] += 0.7
    score[:, E - 1] = -1.0
    idx = score.topk(top, dim=1).indices.to(torch.int32).contiguous()
    wt = torch.rand(T, top, generator=gen, device="cuda:0")
    idx[7] = -1
    idx[T - 1] = -1
    y = torch.full((T, W), float("nan"), device="cuda:0")
    kernels.moe_experts_grouped(h, None, wu, wd, idx, wt, kernels.EXPERT_ACTIVATIONS[act], rt, y)
    kernels.check_device_errors(torch.device("cuda:0"))
    ref = torch.zeros(T, W, dtype=torch.float64, device="cuda:0")
    hd = h.double()
    for e in range(E):
        for j in range(top):
            rows = (idx[:, j] == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            z = hd[rows] @ wu[e].double().T
            a = torch.relu(z) ** 2 if act == "relu2" else z * torch.sigmoid(z)
            ref[rows] += wt[rows, j].double()[:, None] * (a @ wd[e].double().T)
    assert torch.isfinite(y).all() and (y[7] == 0).all() and (y[T - 1] == 0).all()
    err = (y.double() - ref).abs().max(dim=1).values / ref.abs().max()
    assert float(err.max()) < 1.5e-2, (int(err.argmax()), float(err.max()))
    # added to what is there, the same sum
    y2 = torch.ones((T, W), device="cuda:0")
    kernels.moe_experts_grouped(h, None, wu, wd, idx, wt, kernels.EXPERT_ACTIVATIONS[act], rt, y2, add=True)
    assert float((y2 - 1.0 - y).abs().max()) < 1e-5 * max(1.0, float(y.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [20, 36, 128, 260, 328, 2048, 2500, 4096, 4100])
def test_layer_norm_alone_and_as_a_pair(width, dtype):
    import torch
    from llmi_b200.ops import kernels
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rng = np.random.default_rng(width)
    x = (rng.standard_normal((11, width)) * 3 + 40.0).astype(np.float32)       # a large mean: the variance must be taken around it
    w1, w2 = rng.standard_normal(width).astype(np.float32), rng.standard_normal(width).astype(np.float32)
    xd, w1d, w2d = (torch.tensor(a, device="cuda:0") for a in (x, w1, w2))
    a, b = torch.zeros((11, width), dtype=dt, device="cuda:0"), torch.zeros((11, width), dtype=dt, device="cuda:0")
    kernels.layernorm(xd, w1d, a, 1e-5, None, w2d, b)
    rows = torch.tensor([4, -1, 0, 10], dtype=torch.int32, device="cuda:0")
    c = torch.full((4, width), float("nan"), dtype=dt, device="cuda:0")
    kernels.layernorm(xd, w1d, c, 1e-5, rows)
    r1, r2 = G.layer_norm(x.astype(np.float64), w1, 1e-5), G.layer_norm(x.astype(np.float64), w2, 1e-5)
    tol = 1e-4 if dtype == "float32" else 8e-3          # bf16 rounds a result to 2^-9 of its own size

    def off(got_, ref_):
        return (np.abs(got_ - ref_) / (1.0 + np.abs(ref_))).max()
    assert off(a.float().cpu().numpy(), r1) < tol and off(b.float().cpu().numpy(), r2) < tol
    got = c.float().cpu().numpy()
    assert off(got[[0, 2, 3]], r1[[4, 0, 10]]) < tol and (got[1] == 0).all()


@pytest.mark.parametrize("shape", [(5, 24), (3, 7), (64, 128)])
def test_mixture_over_the_depth(shape):
    import torch
    from llmi_b200.ops import kernels
    rng = np.random.default_rng(shape[0])
    n_calls = 4
    hist = torch.full((n_calls + 1, *shape), float("nan"), device="cuda:0")
    xs = [rng.standard_normal(shape).astype(np.float32) for _ in range(n_calls + 1)]
    hist[0] = torch.tensor(xs[0], device="cuda:0")
    for i in range(n_calls):
        c = rng.standard_normal(i + 2).astype(np.float32)
        x = torch.tensor(xs[i + 1], device="cuda:0")
        kernels.depth_mix(x, hist, i + 1, torch.tensor(c, device="cuda:0"))
        ref = sum(float(c[j]) * xs[j].astype(np.float64) for j in range(i + 2))
        assert np.abs(x.cpu().numpy() - ref).max() < 1e-5
        assert np.array_equal(hist[i + 1].cpu().numpy(), xs[i + 1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(5, 24), (3, 7), (9, 328), (64, 2048), (2, 4096), (3, 4100)])
def test_mixture_over_the_depth_with_the_next_norms(shape, dtype):
    """The mixture and the norms that read it next in one pass: the same stream and record as the mixture alone leaves
    (to the bit), and the norms of that stream; sizes the fused form does not take fall back to the two kernels."""
    import torch
    from llmi_b200.engine.runtime import Runtime
    import llmi_b200  # noqa: F401  (registers the parts)
    from llmi_b200.parts.registry import get_part
    from llmi_b200.parts.spec import PartSpec
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rt = Runtime(dt, "cuda:0")
    T, W = shape
    rng = np.random.default_rng(W)
    w1, w2 = (rng.standard_normal(W).astype(np.float32) for _ in range(2))
    norm_spec = PartSpec("layernorm", {"width": W, "eps": 1e-4, "tensor": ""}, "n")
    norms = [get_part("norm", "layernorm")(norm_spec, {"": torch.tensor(w)}, rt) for w in (w1, w2)]
    n_calls = 3
    xs = [(rng.standard_normal(shape) * 2 + 5.0).astype(np.float32) for _ in range(n_calls + 1)]
    hist_a = torch.full((n_calls + 1, T, W), float("nan"), device="cuda:0")
    hist_b = hist_a.clone()
    hist_a[0] = hist_b[0] = torch.tensor(xs[0], device="cuda:0")
    tol = 1e-4 if dtype == "float32" else 8e-3
    for i in range(n_calls):
        c = rng.standard_normal(i + 2).astype(np.float32)
        exit_ = get_part("pass_exit", "depth_average")(PartSpec("depth_average", {"index": i, "tensor": "dwa"}, "l."), {"dwa": torch.tensor(c)}, rt)
        xa, xb = torch.tensor(xs[i + 1], device="cuda:0"), torch.tensor(xs[i + 1], device="cuda:0")
        assert exit_.forward(xa, hist_a, i, None) is None
        then = (norms[0], norms[1]) if i != 1 else (norms[0],)
        done = exit_.forward(xb, hist_b, i, None, then=then)
        assert torch.equal(xa, xb) and torch.equal(hist_a[i + 1], hist_b[i + 1])
        mixed = xa.cpu().numpy().astype(np.float64)
        if done is None:
            assert W % 4 or W > 4096
            continue
        outs = done if isinstance(done, tuple) else (done,)
        assert len(outs) == len(then)
        for o, w in zip(outs, (w1, w2)):
            ref = G.layer_norm(mixed, w, 1e-4)
            assert (np.abs(o.float().cpu().numpy() - ref) / (1.0 + np.abs(ref))).max() < tol
