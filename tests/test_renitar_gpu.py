"""The Renitar design in the library against the plain implementation of tests/plain_renitar.py (GPU).

Every mechanism alone and together, however the work is cut: whole prompts, token by token, portions down to two
tokens, unequal batches, slots and pages that are used again (caches are poisoned with NaN before a replay), lengths at
page borders and at the borders of blocks of positions, the first tokens, long decoding, greedy generation through the
library's own entry point.  32-bit runs must agree with the float64 oracle row by row; bf16 runs agree to bf16's
precision.
"""
import numpy as np
import pytest

import helpers as H
import plain_renitar as G
import renitar_models as M

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
            d = str(tmp_path_factory.mktemp(f"renitar_{name}_{dtype}"))
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
        # float64 oracle does, and such a row (and what follows it through the state) is off by more
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
    """Most of a request in one step, its last 40 tokens one by one: blocks of positions begin and end under decoded
    tokens, the states and the convolution's rows are carried from step to step."""
    model, reqs, refs, _, _ = loaded(name, dtype)
    steps, most = H.trace_last_decoded(reqs, n_last=40)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("portion", [2, 3, 7, 64, 100])
@pytest.mark.parametrize("name", ["unaligned", "gla", "gla_lanes", "pair", "pair_bare", "experts", "mixed", "wide"])
def test_prompts_in_portions(loaded, name, portion):
    """A portion's first rows take the convolution's taps from the rows the portion before left, its recurrences go on
    from the states, and blocks of positions are counted from the sequence's start, not the portion's."""
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
@pytest.mark.parametrize("name", ["unaligned", "pair", "experts", "mixed", "wide", "odd"])
def test_unequal_batches_one_after_another(loaded, name, dtype):
    """Batches of four requests of unequal lengths, prompts of unequal parts of them, decoded together; the next batch
    takes the slots (states, convolution rows) and pages that the one before gave back."""
    model, reqs, refs, _, _ = loaded(name, dtype)
    prompt_lens = {r: max(1, len(t) * (i % 3 + 1) // 4) for i, (r, t) in enumerate(reqs.items())}
    steps, most = H.trace_batches(reqs, 4, prompt_lens)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("name", ["pair", "experts", "mixed", "wide"])
def test_portions_beside_decoding(loaded, name):
    model, reqs, refs, _, _ = loaded(name, "float32")
    ids = list(reqs)
    first = {r: max(1, len(reqs[r]) // 3) for r in ids}
    portion = {r: (1, 5, 2, 33)[i % 4] for i, r in enumerate(ids)}
    steps, most = H.trace_mixed(reqs, first, portion)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(loaded, dtype):
    """Two tokens of prompt, then 300 steps of one token: pages are taken at 64, 128, ..., every block of positions is
    begun by a single token, and the states run through hundreds of steps."""
    model, reqs, refs, _, _ = loaded("mixed", dtype, lengths=[302, 150])
    steps, most = H.trace_batches(reqs, 2, {r: 2 for r in reqs})
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("name", ["experts", "wide", "mixed"])
def test_greedy_generation_through_the_entry_point(loaded, name):
    """generate(): the scheduler's batches, recorded decode steps, the device's argmax — against the oracle's greedy loop."""
    import llmi_b200 as L
    model, _, _, cfg, w = loaded(name, "float32")
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (1, 9, 70, 4, 33)]
    new = [12, 5, 12, 1, 9]
    out = L.generate(model, prompts, max_new=new, max_batch=3)
    ref = [G.greedy(cfg, w, p, n) for p, n in zip(prompts, new)]
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
    """bin/llmi-generate and bin/trace_run on a Renitar folder, as subprocesses: the design is chosen by config.json."""
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
    assert json.loads(r.stdout.strip().splitlines()[-1])["generated_ids"] == G.greedy(cfg, w, prompt, 6)
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


@pytest.mark.parametrize("rank", [1, 2, 40])
def test_the_file_decides_the_size_of_the_decays_low_rank_path(tmp_path, rank):
    import llmi_b200 as L
    cfg = M.CONFIGS["gla"]
    d = str(tmp_path / "m")
    w = M.write_model(d, cfg, M.make_weights(cfg, 3, rank=rank), "F32")
    model = L.load(d, "float32")
    toks = list(range(70))
    steps, most = H.trace_portions({"a": toks}, 17, n_last=5)
    check(H.collect(steps, H.replay(model, steps, most), cfg["vocab"]), {"a": G.forward(cfg, w, toks)}, "float32")


# ----------------------------------------------------------------------------- kernels alone

class _Ctx:
    pass


def _ctx(q_lens, first_pos, slots=None):
    """The index arrays of a step in which sequence s brings ``q_lens[s]`` tokens from position ``first_pos[s]`` on."""
    import torch
    ctx = _Ctx()
    ctx.decode = all(n == 1 for n in q_lens)
    ctx.n_seqs = ctx.n_real_seqs = len(q_lens)
    dev = "cuda:0"
    ctx.tok_seq = torch.tensor(np.repeat(np.arange(len(q_lens)), q_lens).astype(np.int32), device=dev)
    ctx.tok_pos = torch.tensor(np.concatenate([np.arange(p, p + n) for p, n in zip(first_pos, q_lens)]).astype(np.int32), device=dev)
    ctx.seq_q_start = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32), device=dev)
    ctx.seq_kv_len = torch.tensor([p + n for p, n in zip(first_pos, q_lens)], dtype=torch.int32, device=dev)
    ctx.seq_slot = torch.tensor(list(slots) if slots is not None else list(range(len(q_lens))), dtype=torch.int32, device=dev)
    ctx.host_q_lens, ctx.host_kv_lens = list(q_lens), [p + n for p, n in zip(first_pos, q_lens)]
    return ctx


def _paged(rows, order, page, dt):
    """rows [N, heads, d] -> a cache tensor [pages, heads, page, d] with the sequence's pages at ``order``; everything
    else NaN."""
    import torch
    N, heads, d = rows.shape
    cache = torch.full((int(max(order)) + 2, heads, page, d), float("nan"), dtype=dt, device="cuda:0")
    for i, pg in enumerate(order):
        lo, hi = i * page, min((i + 1) * page, N)
        if hi > lo:
            cache[pg, :, :hi - lo] = rows[lo:hi].permute(1, 0, 2).to("cuda:0")
    return cache


def _block_attention_reference(q, k, v, scale, chunk, cap, gate):
    """q [N, H, dk], k [N, G, dk], v [N, G, dv] float64, gate [N, H*dv] -> [N, H, dv]: the plain sums over what
    :func:`G.sees` allows."""
    N, Hq, _ = q.shape
    Gk, dv = k.shape[1], v.shape[2]
    out = np.zeros((N, Hq, dv))
    for t in range(N):
        js = [j for j in range(t + 1) if G.sees(t, j, chunk)]
        for h in range(Hq):
            g = h // (Hq // Gk)
            s = k[js, g] @ q[t, h] * scale
            if cap:
                s = cap * np.tanh(s / cap)
            out[t, h] = G.softmax(s) @ v[js, g] * G.sigmoid(gate[t, h * dv:(h + 1) * dv])
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(2, 1, 16, 16), (4, 2, 64, 48), (2, 2, 128, 32), (6, 2, 24, 40), (3, 3, 32, 64)])
@pytest.mark.parametrize("chunk,key", [
    (100, 0), (100, 199), (100, 200), (100, 201), (100, 299),       # the query at 299 sees 200 .. 299
    (64, 191), (64, 192), (64, 255), (64, 256), (64, 257),          # blocks as long as a page: 299 sees 256 .. 299
    (37, 258), (37, 259), (37, 260), (300, 0), (300, 63), (300, 64), (1, 298), (1, 299), (0, 0), (0, 128),
    (150, 149), (150, 150), (299, 298), (299, 0)])
def test_attention_sees_its_block_of_positions(chunk, key, sizes, dtype):
    """300 cached positions on pages that are not in order, one position (``key``) made to stand out for the last head by
    scaling it and the query; scores are capped and every output entry has a gate of its own.  The query at 299 (as a
    single token, and as the last of a portion of 70 tokens) must return that position's own value row when it lies in
    the query's block of positions and must not see it otherwise; every row is compared with the plain sums."""
    import torch
    from llmi_b200.engine.runtime import Runtime
    from llmi_b200.ops import kernels
    Hq, Gk, dk, dv = sizes
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rng = np.random.default_rng(key + 7 * chunk)
    N, page, cap = 300, 64, 50.0
    k = torch.tensor(rng.standard_normal((N, Gk, dk)).astype(np.float32)).to(dt)
    v = torch.tensor(rng.standard_normal((N, Gk, dv)).astype(np.float32)).to(dt)
    q = torch.tensor((rng.standard_normal((N, Hq, dk)) * 0.3).astype(np.float32))
    others = np.arange(N) != key
    k[others, Gk - 1] *= 0.05
    q[:, -1] = k[key, Gk - 1].float() * (200.0 / dk)     # the score of `key` for the last head: about 100, capped near 48
    q = q.to(dt)
    gate = torch.tensor(rng.standard_normal((N, Hq * dv)).astype(np.float32), device="cuda:0")
    order = rng.permutation(9)[:5]
    rt = Runtime(dt, "cuda:0")
    pages = torch.tensor(order[None, :].astype(np.int32), device="cuda:0")
    kk, vv, qq = (x.float().numpy().astype(np.float64) for x in (k, v, q))
    ref = _block_attention_reference(qq, kk, vv, 0.5, chunk, cap, gate.cpu().numpy().astype(np.float64))
    tol = 2e-5 if dtype == "float32" else 3e-2
    kc, vc = _paged(k, order, page, dt), _paged(v, order, page, dt)
    for n_rows in (1, 70):
        ctx = _ctx([n_rows], [N - n_rows])
        out = torch.full((n_rows, Hq * dv), float("nan"), dtype=dt, device="cuda:0")
        kernels.attention_maps(q[N - n_rows:].reshape(n_rows, -1).to("cuda:0").contiguous(), out, kc, vc, ctx, pages, page,
                               Hq, Gk, 1, dk, dv, 0.5, None, 0, chunk, rt=rt, gate=gate[N - n_rows:], softcap=cap)
        got = out.float().cpu().numpy().reshape(n_rows, Hq, dv)
        assert np.abs(got - ref[N - n_rows:]).max() < tol
        g_last = G.sigmoid(gate[N - 1, (Hq - 1) * dv:].cpu().numpy().astype(np.float64))
        alone = np.abs(got[-1, -1] / g_last - vv[key, Gk - 1]).max() < max(tol, 1e-3) * 4
        assert alone == G.sees(299, key, chunk), (key, chunk)


@pytest.mark.parametrize("H_,D,Dv", [(2, 64, 64), (3, 12, 20), (2, 40, 32), (1, 96, 48), (4, 128, 16), (2, 4, 12), (1, 200, 8), (5, 6, 7),
                                     (1, 256, 32), (2, 160, 16)])
@pytest.mark.parametrize("per_head", [False, True])
def test_recurrence_with_a_decay(H_, D, Dv, per_head):
    """S <- w S + k v^T, o = scale S^T q for three sequences of unequal lengths in slots that are not in order, cut into
    steps of many tokens, of one token, and of two; the states start as NaN where no sequence lives and as zero where one
    starts.  Head 0 forgets nothing in one key channel (with a decay per head: in all of them), which the first token
    writes and only the last token asks for again: what was written there comes back after hundreds of tokens."""
    import torch
    from llmi_b200.ops import kernels
    rng = np.random.default_rng(H_ * 1000 + D + Dv)
    lens, slots, scale, dev = [301, 17, 130], [4, 1, 2], 0.37, "cuda:0"
    N, Nv = H_ * D, H_ * Dv
    state = torch.full((6, N * Dv + 8), float("nan"), device=dev)
    state[slots] = 0.0
    head_w = np.concatenate([[1.0], rng.uniform(0.5, 0.99, H_ - 1)]).astype(np.float32)
    data, refs = [], []
    for n in lens:
        q, k = (rng.standard_normal((n, H_, D)) * 0.5 for _ in range(2))
        v = rng.standard_normal((n, H_, Dv))
        w = np.broadcast_to(head_w[None, :, None], (n, H_, D)).copy() if per_head else rng.uniform(0.3, 1.0, (n, H_, D))
        w[:, 0, 0], q[:, 0, 0], k[:, 0, 0] = 1.0, 0.0, 0.0
        k[0, 0, 0], q[-1, 0, 0] = 30.0, 30.0
        q, k, v, w = (x.astype(np.float32) for x in (q, k, v, w))
        data.append((q, k, v, w))
        refs.append(np.stack([G.linear_recurrence(*(x[:, a].astype(np.float64) for x in (q, k, v, w))) for a in range(H_)], axis=1) * scale)
    got = [np.zeros((n, H_, Dv)) for n in lens]
    done = [0, 0, 0]
    for step in ([250, 17, 100], [1, 0, 1], [2, 0, 2], [48, 0, 27]):          # tokens of each sequence per step
        live = [s for s in range(3) if step[s]]

        def rows(j):
            return np.concatenate([data[s][j][done[s]:done[s] + step[s]].reshape(step[s], -1) for s in live])
        proj = np.concatenate([np.zeros((sum(step), 4), np.float32), rows(0), rows(1), rows(2)], axis=1)     # (q does not start a row)
        ctx = _ctx([step[s] for s in live], [done[s] for s in live], [slots[s] for s in live])
        o = torch.full((sum(step), Nv), float("nan"), device=dev)
        decay = {"head_decay": torch.tensor(head_w, device=dev)} if per_head else {"dec": torch.tensor(rows(3), device=dev)}
        kernels.decay_recurrence(torch.tensor(proj, device=dev), 4, 4 + N, 4 + 2 * N, H_, D, Dv, state, ctx, o, q_scale=scale, **decay)
        o = o.cpu().numpy()
        at = 0
        for s in live:
            got[s][done[s]:done[s] + step[s]] = o[at:at + step[s]].reshape(step[s], H_, Dv)
            at += step[s]
            done[s] += step[s]
    assert done == lens
    for s in range(3):
        assert np.isfinite(got[s]).all()
        assert np.abs(got[s] - refs[s]).max() < 2e-5 * max(1.0, np.abs(refs[s]).max()), (s, float(np.abs(got[s] - refs[s]).max()))
        # the far key: the last token's read-out of head 0 holds 900 * scale * v_0 from channel 0, far above the rest
        far = 900.0 * scale * data[s][2][0, 0]
        assert np.abs(got[s][-1, 0] - far).max() < 0.2 * np.abs(far).max() + 40.0
        assert np.abs(refs[s][-1, 0] - far).max() < 0.2 * np.abs(far).max() + 40.0
    assert torch.isnan(state[[0, 3, 5]]).all() and torch.isfinite(state[slots, :N * Dv]).all()


@pytest.mark.parametrize("T,N,R,tau", [(5, 96, 16, 16.0), (70, 40, 3, 1.0), (9, 2048, 64, 4.0), (1100, 24, 1, 32.0)])
def test_decays_of_the_key_channels(T, N, R, tau):
    import torch
    from llmi_b200.ops import kernels
    rng = np.random.default_rng(T + N)
    low = rng.standard_normal((T, R + 5)).astype(np.float32)
    w2 = rng.standard_normal((N, R)).astype(np.float32)
    b = (rng.standard_normal(N) * 4).astype(np.float32)
    ctx = _ctx([T], [0])
    dec = torch.full((T, N), float("nan"), device="cuda:0")
    kernels.channel_decay(torch.tensor(low, device="cuda:0")[:, 2:2 + R], torch.tensor(w2.T.copy(), device="cuda:0"),
                          torch.tensor(b, device="cuda:0"), tau, ctx, dec)
    dec2 = torch.full((T, N), float("nan"), device="cuda:0")      # with the matrix as stored too: a handful of tokens read that
    kernels.channel_decay(torch.tensor(low, device="cuda:0")[:, 2:2 + R], torch.tensor(w2.T.copy(), device="cuda:0"),
                          torch.tensor(b, device="cuda:0"), tau, ctx, dec2, torch.tensor(w2, device="cuda:0"))
    assert torch.equal(dec, dec2)
    z = low[:, 2:2 + R].astype(np.float64) @ w2.astype(np.float64).T + b
    ref = G.sigmoid(z) ** (1.0 / tau)
    got = dec.cpu().numpy()
    assert np.abs(got - ref).max() < 3e-6
    assert np.abs(np.log(got) - np.log(ref)).max() < 2e-4 * max(1.0, np.abs(np.log(ref)).max())      # also where logistic(z) is tiny


@pytest.mark.parametrize("C,K", [(20, 4), (96, 1), (37, 2), (256, 5), (8, 16)])
def test_convolution_without_its_input_in_portions(C, K):
    """Rows of a wider fp32 matrix through the taps, two sequences cut into unequal portions (down to one token), the
    rows before a portion from the state; against the plain sum."""
    import torch
    from llmi_b200.ops import kernels
    rng = np.random.default_rng(C + K)
    lens = [45, 7]
    u = [rng.standard_normal((n, C)).astype(np.float32) for n in lens]
    w = rng.standard_normal((C, K)).astype(np.float32)
    refs = [G.short_conv(x.astype(np.float64), w.astype(np.float64)) for x in u]
    dev = "cuda:0"
    carry = torch.full((4, max(K - 1, 1) * C + 3), float("nan"), device=dev)
    slots = [2, 0]
    carry[slots] = 0.0
    wt = torch.tensor(w.T.copy(), device=dev)
    got = [np.zeros((n, C)) for n in lens]
    done = [0, 0]
    for step in ([20, 3], [1, 1], [2, 3], [1, 0], [1, 0], [1, 0], [1, 0], [1, 0], [17, 0]):
        live = [s for s in range(2) if step[s]]
        rows = np.concatenate([u[s][done[s]:done[s] + step[s]] for s in live])
        wide = torch.tensor(np.concatenate([rows, np.full((rows.shape[0], 6), 9.0, np.float32)], axis=1), device=dev)
        ctx = _ctx([step[s] for s in live], [done[s] for s in live], [slots[s] for s in live])
        out = torch.full((rows.shape[0], C), float("nan"), device=dev)
        if all(step[s] == 1 for s in live) and K > 1:      # single tokens: the kernel that also brings the state up to date
            kernels.conv_token(wide[:, :C], wt, carry, ctx, out)
        else:
            kernels.conv_add(wide[:, :C], wt, carry, ctx, out, add_input=False)
        o = out.cpu().numpy()
        at = 0
        for s in live:
            got[s][done[s]:done[s] + step[s]] = o[at:at + step[s]]
            at += step[s]
            done[s] += step[s]
    for s in range(2):
        assert np.abs(got[s] - refs[s]).max() < 1e-5


@pytest.mark.parametrize("E,n_id,top,scale", [(5, 2, 3, 2.0), (8, 0, 2, 1.0), (2, 3, 4, 0.5), (40, 1, 6, 1.5), (3, 0, 3, 1.0), (1, 1, 1, 3.0)])
def test_experts_are_chosen_by_corrected_scores_and_weighted_by_plain_ones(E, n_id, top, scale):
    import torch
    from llmi_b200.ops import kernels
    rng = np.random.default_rng(E + top)
    T, n_out = 60, E + n_id
    z = (rng.standard_normal((T, n_out + 1)) * 2).astype(np.float32)
    corr = (rng.standard_normal(n_out) * 0.3).astype(np.float32)         # large enough to change many choices
    ctx = _ctx([T], [0])
    ctx.tok_seq[7] = -1
    idx = torch.zeros((T, top), dtype=torch.int32, device="cuda:0")
    wt = torch.zeros((T, top), dtype=torch.float32, device="cuda:0")
    idw = torch.full((T,), float("nan"), device="cuda:0")
    kernels.moe_route(torch.tensor(z, device="cuda:0"), top, ctx, idx, wt, kernels.ROUTE_SOFTMAX_ALL, experts=n_out,
                      correction=torch.tensor(corr, device="cuda:0"), scale=scale, identity=n_id, id_wt=idw)
    idx, wt, idw = idx.cpu().numpy(), wt.cpu().numpy(), idw.cpu().numpy()
    changed = 0
    for t in range(T):
        if t == 7:
            assert (idx[t] == -1).all() and (wt[t] == 0).all() and idw[t] == 0
            continue
        chosen, weights = G.route(z[t, :n_out].astype(np.float64), corr.astype(np.float64), top, scale)
        changed += chosen != G.route(z[t, :n_out].astype(np.float64), 0 * corr, top, scale)[0]
        assert idx[t].tolist() == [e if e < E else -1 for e in chosen]
        assert np.abs(wt[t] - weights).max() < 1e-6
        assert abs(idw[t] - sum(c for e, c in zip(chosen, weights) if e >= E)) < 1e-6
    assert changed > 0 or top == n_out


@pytest.mark.parametrize("T,E,top,W,F", [(3, 4, 2, 64, 48), (600, 4, 2, 128, 128), (1500, 8, 2, 256, 192), (300, 5, 3, 136, 72)])
def test_experts_with_the_exact_gelu_on_every_kind_of_tile(T, E, top, W, F):
    """Streamed weights (a few tokens), mma.sync tiles, tcgen05 tiles (from 1,024 items on): the same sum, with choices
    that are skipped (index -1: experts that hand their input on, added by a kernel of their own)."""
    import torch
    from llmi_b200.engine.runtime import Runtime
    from llmi_b200.ops import kernels
    rt = Runtime(torch.bfloat16, "cuda:0")
    gen = torch.Generator(device="cuda:0").manual_seed(T + E)

    def rnd(*shape, gain=1.0):
        return (torch.randn(*shape, generator=gen, device="cuda:0") * gain).to(torch.bfloat16)
    h, wu, wd = rnd(T, W), rnd(E, F, W, gain=2 * W ** -0.5), rnd(E, W, F, gain=F ** -0.5)
    score = torch.rand(T, E + 1, generator=gen, device="cuda:0")
    idx = score.topk(top, dim=1).indices.to(torch.int32)
    idx[idx == E] = -1                                                   # the last "expert" has no tensors
    idx = idx.contiguous()
    wt = torch.rand(T, top, generator=gen, device="cuda:0")
    idw = (wt * (idx < 0)).sum(1).contiguous()
    y = torch.full((T, W), float("nan"), device="cuda:0")
    act = kernels.EXPERT_ACTIVATIONS["gelu"]
    if kernels.moe_grouped_applies(h, W, F, E):          # (the grouped form adds the handed-on inputs in the kernel that forms the sum)
        kernels.moe_experts_grouped(h, None, wu, wd, idx, wt, act, rt, y, id_wt=idw)
    else:
        a = torch.empty((T, top, F), device="cuda:0")
        kernels.moe_experts_streamed(h, None, wu, wd, idx, wt, act, a, y)
        kernels.moe_identity_add(h, idw, y)
    kernels.check_device_errors(torch.device("cuda:0"))
    hd = h.double()
    ref = idw.double()[:, None] * hd
    for e in range(E):
        for j in range(top):
            rows = (idx[:, j] == e).nonzero().flatten()
            if rows.numel():
                z = hd[rows] @ wu[e].double().T
                ref[rows] += wt[rows, j].double()[:, None] * ((0.5 * z * (1 + torch.erf(z / 2 ** 0.5))) @ wd[e].double().T)
    err = (y.double() - ref).abs().max(dim=1).values / ref.abs().max()
    assert torch.isfinite(y).all() and float(err.max()) < 1.5e-2, (int(err.argmax()), float(err.max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,N,K", [(3, 96, 64), (40, 200, 128), (700, 256, 192), (9, 40, 36)])
def test_products_that_end_in_the_exact_gelu(T, N, K, dtype):
    """Every product kernel that can take the step (weight streaming, tcgen05, fp32 FMA) finishes gelu(x W^T + b)."""
    import torch
    from llmi_b200.ops import kernels
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    gen = torch.Generator(device="cuda:0").manual_seed(T + N)
    x = (torch.randn(T, K, generator=gen, device="cuda:0")).to(dt)
    w = (torch.randn(N, K, generator=gen, device="cuda:0") * 2 * K ** -0.5).to(dt)
    b = torch.randn(N, generator=gen, device="cuda:0")
    out = torch.full((T, N), float("nan"), dtype=dt, device="cuda:0")
    kernels.linear(x, w, out, b, kernels.OUT_GELU)
    z = x.double() @ w.double().T + b.double()
    ref = 0.5 * z * (1 + torch.erf(z / 2 ** 0.5))
    assert float((out.double() - ref).abs().max()) < (2e-5 if dtype == "float32" else 3e-2) * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,W", [(5, 36), (70, 256), (3, 2048), (600, 1000)])
def test_joining_the_branches(T, W, dtype):
    """The mean of two normed rows; x += m y with and without the next norm in the same pass."""
    import torch
    from llmi_b200.ops import kernels
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rng = np.random.default_rng(T + W)
    a, b, x, y = (rng.standard_normal((T, W)).astype(np.float32) * s for s in (3.0, 0.2, 1.0, 2.0))
    wa, wb, wn = (1.0 + 0.3 * rng.standard_normal(W).astype(np.float32) for _ in range(3))
    dev = "cuda:0"
    ta, tb, tx, ty, twa, twb, twn = (torch.tensor(v, device=dev) for v in (a, b, x, y, wa, wb, wn))
    eps = 1e-3
    ref = 0.5 * (G.rms_norm(a.astype(np.float64), wa, eps) + G.rms_norm(b.astype(np.float64), wb, eps))
    out = torch.full((T, W), float("nan"), device=dev)
    kernels.normed_pair(ta, twa, tb, twb, eps, 0.5, out)
    assert np.abs(out.cpu().numpy() - ref).max() < 1e-5
    out2 = tx.clone()
    kernels.normed_pair(ta, twa, tb, twb, eps, 0.5, out2, add=True)
    assert np.abs(out2.cpu().numpy() - (x + ref)).max() < 1e-5
    x1 = tx.clone()
    kernels.stream_axpy_norm(x1, ty, 0.7)
    x_ref = x.astype(np.float64) + 0.7 * y
    assert np.abs(x1.cpu().numpy() - x_ref).max() < 1e-6
    x2, h = tx.clone(), torch.full((T, W), float("nan"), dtype=dt, device=dev)
    kernels.stream_axpy_norm(x2, ty, 0.7, twn, eps, h)
    assert torch.equal(x1, x2)
    assert np.abs(h.float().cpu().numpy() - G.rms_norm(x_ref, wn, eps)).max() < (1e-5 if dtype == "float32" else 3e-2)
