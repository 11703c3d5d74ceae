"""Decode and prefill throughput of the library at SmolLM2-1.7B shape (random bf16 weights, one B200).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --workload smollm2-360m|smollm2-135m [--workload-dtypes bfloat16,float32]
    python bench.py --design garodra|fusazen|gemosun|renitar [--design-sizes 2048,1024]          (its own JSON line: that design's prefill and
                                                                                  decode beside the Llama decoder (renitar: beside the
                                                                                  Fusazen design) at equal size; garodra also has the
                                                                                  size 2048-looped)

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 and context 4096 (a
"step" is one decode step of the whole batch), timed on the device with CUDA events around
exactly K steps after W warm-up steps.  ``e2e`` is the same through the public entry point
(``Model.step_and_choose``): host token ids in, host token ids out, every step.  ``prefill`` is
one 2,048-token prompt; ``points`` are decode at batch 1 and 64; ``roofline`` relates the decode
step to HBM bandwidth: (every weight once + the cache of the live requests) / step time.
Peaks come from MEASURED_PEAKS.json beside this file when present, else from the fallback
figures (6.65 TB/s copy, 1.59 PFLOP/s bf16).  Token ids are seeded uniform random numbers and
the cache of the decode runs is filled with random keys and values instead of a real prefill
(the time of a step does not depend on their values).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# SmolLM2-1.7B layer sizes (BASELINE.json configs[2])
CONFIG = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 32,
    "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 49152, "rope_theta": 130000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192, "hidden_act": "silu",
}
FULL_LAYERS = 24
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None
        self.begin = self.end = None

    def start(self):
        """Start sampling (the tool takes a moment to come up: call this before the warm-up)."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                                          "-i", "0", "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def mark_begin(self):
        self.begin = len(self.rows)

    def mark_end(self):
        self.end = len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        rows = self.rows[self.begin:self.end] if self.begin is not None and self.end is not None else self.rows
        where = "timed region"
        if not rows:                      # a region shorter than one sampling period: the samples around it
            rows, where = self.rows[max(0, (self.begin or 0) - 2):(self.end or 0) + 2], "around the timed region"
        sm = sorted(int(r[0]) for r in rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm), "sampled": where}


def fill_cache(cache, model, batch, start_len):
    """Slots whose caches hold ``start_len`` positions of random keys and values."""
    import torch
    for g in cache.kv_groups:
        g.k.normal_(0, 0.5)
        if g.v is not None:
            g.v.normal_(0, 0.5)
    slots = []
    for _ in range(batch):
        s = cache.alloc_slot()
        cache.extend(s, start_len)
        slots.append(s)
    torch.cuda.synchronize()
    return slots


def decode_run(model, batch, context, steps, warmup, e2e=False, clocks=None):
    """Decode `steps` steps ending at `context`; returns (ms per step, launches, h2d, d2h bytes per step)."""
    import torch
    from llmi_b200 import SamplingParams, SequenceStep
    from llmi_b200.engine.graphs import DecodeGraphs
    from llmi_b200.ops import kernels
    from llmi_b200.sampling import Sampler
    total = warmup + steps
    start = context - total
    cache = model.new_cache(batch * ((context + 63) // 64) * 64, n_slots=batch)
    slots = fill_cache(cache, model, batch, start)
    sampler = Sampler(SamplingParams(), model.rt)
    if model._graphs is None:
        model._graphs = DecodeGraphs(model)
    rng = torch.Generator().manual_seed(batch)
    toks = torch.randint(0, model.vocab_size, (batch,), generator=rng).tolist()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = h2d = d2h = 0
    for i in range(total):
        if i == warmup:
            torch.cuda.synchronize()
            if clocks:
                clocks.mark_begin()
            launches0 = kernels.launch_count()
            e0.record()
        seqs = [SequenceStep(s, [t], [0]) for s, t in zip(slots, toks)]
        if e2e:
            ids = model.step_and_choose(cache, seqs, sampler)          # host ids in, host ids out
            toks = ids.tolist()
            if i >= warmup:
                h2d += model.last_h2d_bytes
                d2h += ids.numel() * 4
        else:
            model._graphs.step(cache, seqs, sampler)
    e1.record()
    torch.cuda.synchronize()
    if clocks:
        clocks.mark_end()
    ms = e0.elapsed_time(e1) / steps
    launches = kernels.launch_count() - launches0
    kernels.check_device_errors(model.device)
    cache_bytes = batch * (context - steps / 2.0) * cache.bytes_per_token()
    for s in slots:
        cache.free_slot(s)
    del cache
    torch.cuda.empty_cache()
    return ms, launches, h2d / max(steps, 1), d2h / max(steps, 1), cache_bytes


def prefill_run(model, tokens, iters=5):
    import torch
    from llmi_b200 import SequenceStep
    cache = model.new_cache(((tokens + 63) // 64) * 64)
    ids = torch.randint(0, model.vocab_size, (tokens,), generator=torch.Generator().manual_seed(1)).tolist()
    times = []
    for i in range(iters + 2):
        s = cache.alloc_slot()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        model.step(cache, [SequenceStep(s, ids, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        cache.free_slot(s)
        if i >= 2:
            times.append(e0.elapsed_time(e1))
    return sorted(times)[len(times) // 2]


def prefill_flops(cfg, layers, T):
    H, nh, nkv, hd, F, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                            cfg["intermediate_size"], cfg["vocab_size"])
    per_token = layers * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * F)
    attn = layers * 4 * nh * hd * (T * (T + 1) // 2)          # QK^T and PV over the causal half
    return 2 * T * per_token + attn + 2 * H * V              # the head runs on the last row only


# The other two shapes of the benchmark set: whole requests through generate() (prefill and decoding in one time)
WORKLOADS = {
    "smollm2-360m": {
        "config": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 32, "hidden_size": 960, "num_attention_heads": 15,
                   "num_key_value_heads": 5, "head_dim": 64, "intermediate_size": 2560, "vocab_size": 49152, "rope_theta": 100000.0,
                   "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192, "hidden_act": "silu"},
        "prompts": lambda rng: [int(n) for n in rng.integers(16, 1025, 8)], "max_new": 256, "max_new_fp32": 256,
        "what": "8 prompts of 16..1,024 uniform random ids, 256 new tokens each"},
    "smollm2-135m": {
        "config": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 30, "hidden_size": 576, "num_attention_heads": 9,
                   "num_key_value_heads": 3, "head_dim": 64, "intermediate_size": 1536, "vocab_size": 49152, "rope_theta": 100000.0,
                   "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192, "hidden_act": "silu"},
        "prompts": lambda rng: [512] * 64, "max_new": 512, "max_new_fp32": 64,
        "what": "64 prompts of 512 uniform random ids, 512 new tokens each (64 in fp32)"},
}


def workload_run(name, dtypes):
    """One of the other benchmark shapes through the public entry point; prints one JSON line."""
    import numpy as np
    import torch
    import llmi_b200 as L
    wl = WORKLOADS[name]
    rng = np.random.default_rng(0)
    lens = wl["prompts"](rng)
    V = wl["config"]["vocab_size"]
    prompts = [rng.integers(0, V, n).tolist() for n in lens]
    out = {"workload": name, "what": wl["what"], "impl": "ours", "data": "synthetic (random weights, uniform random token ids)",
           "prompt_tokens": int(sum(lens)), "runs": {}}
    for dtype in dtypes:
        max_new = wl["max_new"] if dtype == "bfloat16" else wl["max_new_fp32"]
        model = L.random_model(wl["config"], seed=0, dtype=dtype, on_device=True)
        L.generate(model, prompts[:2], max_new=4, ignore_eos=True)          # builds the kernels' one-time state
        best = None
        for _ in range(2):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            got, info = L.generate(model, prompts, max_new=max_new, ignore_eos=True, return_details=True)
            torch.cuda.synchronize()
            sec = time.perf_counter() - t0
            best = sec if best is None else min(best, sec)
        new = sum(len(g) for g in got)
        out["runs"][dtype] = {"seconds": round(best, 4), "new_tokens": new, "new_tokens_per_s": round(new / best, 1),
                              "steps": info["steps"], "batches": info["batches"]}
        del model
        torch.cuda.empty_cache()
    print(json.dumps(out))
    return 0


# --design garodra: the Garodra design at sizes that resemble a real model's layers, beside the Llama decoder at equal
# width, depth and feed-forward size.  Layers of the design alternate its two mixers and its two feed-forwards.
def garodra_config(width, heads, dim, rot_dim, kv_rank, q_rank, d_heads, d_kv, ff, experts, top, expert_ff, layers, vocab, loop):
    att = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": dim, "kv_rank": kv_rank, "q_rank": q_rank,
           "scale": (dim + rot_dim) ** -0.5, "rot": {"base": 10000.0, "dims": rot_dim}}
    dlt = {"heads": d_heads, "kv_heads": d_kv, "dim": dim, "vdim": dim, "conv": 4}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}}
    kinds = [("latent_attention", att, dense), ("latent_attention", att, moe), ("delta", dlt, dense), ("delta", dlt, moe)]
    cfg = {"architecture": "Garodra", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
           "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in (kinds[i % 4] for i in range(layers))]}
    if loop:
        cfg["loop"] = {"start": 0, "stop": layers, "times": loop}
    return cfg


DESIGN_SIZES = {
    # name: (garodra config, llama config of equal width, layer runs and feed-forward size)
    "2048": (garodra_config(2048, 16, 128, 64, 512, 1024, 16, 8, 8192, 8, 2, 2048, 8, 49152, 0),
             dict(CONFIG, num_hidden_layers=8)),
    "2048-looped": (garodra_config(2048, 16, 128, 64, 512, 1024, 16, 8, 8192, 8, 2, 2048, 4, 49152, 2),
                    dict(CONFIG, num_hidden_layers=8)),
    "1024": (garodra_config(1024, 8, 64, 32, 256, 384, 8, 4, 4096, 8, 2, 1024, 8, 49152, 0),
             dict(CONFIG, num_hidden_layers=8, hidden_size=1024, num_attention_heads=16, num_key_value_heads=16,
                  intermediate_size=4096)),
}


# --design fusazen: the Fusazen design at sizes that resemble a real model's layers, beside the Llama decoder at equal
# width, depth and feed-forward size.  Eight layers: two-map attention, delta rule, normed attention, delta rule, two-map
# attention on the first layer's keys and values, delta rule, normed attention, delta rule.  The masks' blocks span the
# whole context of the decode runs, so that attention reads as many positions as the Llama decoder's.
def fusazen_config(width, heads, kv_heads, dim, d_heads, ff, vocab, block):
    diff = {"heads": heads // 2, "kv_heads": kv_heads // 2, "dim": dim, "vdim": 2 * dim, "diff": 0.5, "mask": {"size": block},
            "rot": {"base": 10000.0, "dims": dim // 2}, "scale": dim ** -0.5}
    normed = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": block}, "scale": 1.0 / dim}
    dlt = {"heads": d_heads, "dim": dim}
    mlp = {"kind": "dense", "ff": ff}
    kinds = [("attention", diff), ("general_delta", dlt), ("attention_2", normed), ("general_delta", dlt),
             ("attention", dict(diff, kv_from=0)), ("general_delta", dlt), ("attention_2", normed), ("general_delta", dlt)]
    return {"architecture": "Fusazen", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "canon": {"taps": 4}, "layers": [{"type": t, "mixer": m, "mlp": mlp} for t, m in kinds]}


FUSAZEN_SIZES = {
    "2048": (fusazen_config(2048, 32, 8, 64, 32, 8192, 49152, 8192), None),
    "1024": (fusazen_config(1024, 16, 4, 64, 16, 4096, 49152, 8192), None),
}


# --design gemosun: the Gemosun design at sizes that resemble a real model's layers, beside the Llama decoder at equal
# width, depth and dense feed-forward size.  Eight layers whose feed-forwards alternate: gated dense, then routed experts
# (eight, two a token, in four groups of which two can be chosen, plus a gated shared expert).  Every mixer is the
# design's attention: four query heads per key/value head, values that are the keys, a stretched rotation of half a head,
# a gate per head.  The sizes differ in the mask: a window of 1,024 positions with blocks of 16 pooled behind it (what the
# design is for: a decode step at 4,096 positions reads 1,024 positions and 192 pooled rows a layer), or ("-full") a
# window that spans the whole context, so that attention reads as many positions as the Llama decoder's.
def gemosun_config(width, heads, kv_heads, dim, ff, experts, top, expert_ff, groups, shared, window, pool, layers, vocab):
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
           "rot": {"base": 10000.0, "dims": dim // 2, "scaling": {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}},
           "mask": {"size": window, "pool": pool}}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top, "groups": {"count": groups[0], "keep": groups[1]}},
           "shared": {"ff": shared}}
    return {"architecture": "Gemosun", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [{"type": "attention", "mixer": att, "mlp": (dense, moe)[i % 2]} for i in range(layers)]}


GEMOSUN_SIZES = {
    "2048": (gemosun_config(2048, 16, 4, 128, 8192, 8, 2, 2048, (4, 2), 2048, 1024, 16, 8, 49152), None),
    "2048-full": (gemosun_config(2048, 16, 4, 128, 8192, 8, 2, 2048, (4, 2), 2048, 8192, 16, 8, 49152), None),
    "1024": (gemosun_config(1024, 16, 4, 64, 4096, 8, 2, 1024, (4, 2), 1024, 1024, 16, 8, 49152), None),
}


# --design renitar: the Renitar design at sizes that resemble a real model's layers, beside the Fusazen design (the
# closest of the library's models: a recurrence with a decay per key channel, attention masked to blocks of positions
# with whole-row q and k norms, a short convolution) at equal width and depth.  Eight layers: linear attention with a
# decay per key channel, then two mixers side by side (attention with a convolution on q, k, v, capped scores and a gate
# per output entry; linear attention with a decay per head), and so on in turn; every layer has routed experts (eight
# with matrices and two that hand their input on, three a token, a gated shared expert).  The attention's blocks of
# positions span the whole context of the decode runs, so that it reads as many positions as the other model's.
def renitar_config(width, heads, kv_heads, dim, r_heads, experts, identity, top, expert_ff, shared, vocab, block, layers=8):
    gla = {"heads": r_heads, "dim": dim, "vdim": dim, "tau": 8.0, "rank": max(16, width // 32)}
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "conv": 4, "softcap": 50.0,
            "mask": {"size": block}, "rot": {"base": 10000.0, "dims": dim // 2}}
    right = {"heads": r_heads, "dim": dim, "vdim": dim, "decay": [1.0 - 2.0 ** (-1.0 - 7.0 * h / max(r_heads - 1, 1)) for h in range(r_heads)]}
    moe = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": 2.0},
           "shared": {"ff": shared}}
    kinds = [("gla", gla), ("parallel", {"left": left, "right": right})]
    return {"architecture": "Renitar", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.7,
            "layers": [{"type": kinds[i % 2][0], "mixer": kinds[i % 2][1], "mlp": moe} for i in range(layers)]}


RENITAR_SIZES = {
    # name: (renitar config, the other model's config, the other model's label)
    "2048": (renitar_config(2048, 32, 8, 64, 32, 8, 2, 3, 2048, 2048, 49152, 8192), FUSAZEN_SIZES["2048"][0], "fusazen"),
    "1024": (renitar_config(1024, 16, 4, 64, 16, 8, 2, 3, 1024, 1024, 49152, 8192), FUSAZEN_SIZES["1024"][0], "fusazen"),
}


class KernelTimes:
    """Device time per entry point of ops.kernels inside real steps (CUDA events around every call; steps run launch
    by launch while this is on, so the figures are shares of a step, not a benchmark of it)."""
    NAMES = ("embed", "rmsnorm", "swiglu", "linear", "rope_store", "attention", "dyt", "dyt_add", "stream_add", "linear_batched",
             "latent_prepare", "latent_q_rotate", "attention_latent", "delta_step", "delta_finish", "moe_route",
             "moe_experts_streamed", "moe_experts_grouped", "conv_add", "qkv_prepare", "attention_maps", "diff_combine",
             "gdelta_prepare", "dplr_recurrence", "activate", "layernorm", "depth_mix", "pool_rows", "gate_rows", "tanh_rows",
             "channel_decay", "rows_silu", "decay_recurrence", "normed_pair", "stream_axpy_norm", "moe_identity_add")

    def __init__(self):
        self.spans, self.saved = [], {}

    def __enter__(self):
        import torch
        from llmi_b200.ops import kernels
        for name in self.NAMES:
            fn = getattr(kernels, name, None)
            if fn is None:
                continue
            self.saved[name] = fn

            def timed(*a, _fn=fn, _name=name, **k):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                r = _fn(*a, **k)
                e1.record()
                self.spans.append((_name, e0, e1))
                return r
            setattr(kernels, name, timed)
        return self

    def __exit__(self, *exc):
        from llmi_b200.ops import kernels
        for name, fn in self.saved.items():
            setattr(kernels, name, fn)

    def table(self):
        import torch
        torch.cuda.synchronize()
        out = {}
        for name, e0, e1 in self.spans:
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        return {k: round(v, 3) for k, v in sorted(out.items(), key=lambda kv: -kv[1])}


def design_run(name, steps, warmup, batch, context, tokens, sizes):
    """Prefill and decode throughput of a design beside the closest existing model at equal size; one JSON line."""
    import torch
    import llmi_b200 as L
    from llmi_b200 import SequenceStep
    tables = {"garodra": DESIGN_SIZES, "fusazen": FUSAZEN_SIZES, "gemosun": GEMOSUN_SIZES, "renitar": RENITAR_SIZES}
    if name not in tables:
        print(f"bench.py: unknown design {name!r}")
        return 2
    table = tables[name]
    pk, pk_kind = peaks()
    out = {"design": name, "impl": "ours", "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids, random cache contents)",
           "batch": batch, "context": context, "prefill_tokens": tokens, "steps": steps, "warmup": warmup, "peaks": pk_kind,
           "sizes": {}}
    for size in sizes:
        g_cfg, l_cfg, *other = table[size]
        if l_cfg is None:
            l_cfg = DESIGN_SIZES[size.split("-")[0]][1]
        row = {}
        for label, cfg in ((name, g_cfg), (other[0] if other else "llama", l_cfg)):
            model = L.random_model(cfg, seed=0, dtype="bfloat16", on_device=True)
            pre_ms = prefill_run(model, tokens, iters=3)
            ms, launches, _, _, cache_bytes = decode_run(model, batch, context, steps, warmup)
            ms1, *_ = decode_run(model, 1, context, min(steps, 32), warmup)
            entry = {"params": model.parameter_count, "weight_bytes": model.weight_bytes(),
                     "prefill_ms": round(pre_ms, 3), "prefill_tokens_per_s": round(tokens * 1000.0 / pre_ms, 1),
                     "decode_ms_per_step": round(ms, 4), "decode_tokens_per_s": round(batch * 1000.0 / ms, 1),
                     "decode_b1_tokens_per_s": round(1000.0 / ms1, 1), "decode_launches": launches,
                     "cache_bytes_per_token": model.new_cache(64).bytes_per_token()}
            # shares of one prompt step and of one decode step, kernel by kernel (launch by launch)
            os.environ["LLMI_GRAPHS"] = "0"
            from llmi_b200.engine import graphs
            graphs.RECORD = False
            cache = model.new_cache(((tokens + 63) // 64) * 64 + 64)
            ids = torch.randint(0, model.vocab_size, (tokens,), generator=torch.Generator().manual_seed(1)).tolist()
            for final in (False, True):                  # the first round sizes every scratch buffer; the second is read
                slot = cache.alloc_slot()
                with KernelTimes() as kt:
                    model.step(cache, [SequenceStep(slot, ids, [tokens - 1])])
                if final:
                    entry["prefill_kernel_ms"] = kt.table()
                for _ in range(2):
                    with KernelTimes() as kt:
                        model.step(cache, [SequenceStep(slot, [1], [0])])
                if final:
                    entry["decode_b1_kernel_ms_at_%d" % tokens] = kt.table()
                cache.free_slot(slot)
            graphs.RECORD = True
            os.environ.pop("LLMI_GRAPHS", None)
            row[label] = entry
            del model, cache
            torch.cuda.empty_cache()
        out["sizes"][size] = row
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the full model (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="with --only prefill: another prompt length")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one part only and print its numbers (for profiling one kernel class; not a bench line)")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=None,
                    help="run one of the other benchmark shapes whole, through generate(), and print its own JSON line")
    ap.add_argument("--workload-dtypes", default="bfloat16", help="comma-separated: bfloat16, float32")
    ap.add_argument("--kv-heads", type=int, default=None,
                    help="with --only: another number of key/value heads (grouped queries), to profile their kernels")
    ap.add_argument("--design", default=None,
                    help="'garodra', 'fusazen', 'gemosun' or 'renitar': that design's prefill and decode throughput at layer sizes of a real model, beside the "
                         "Llama decoder (renitar: beside the Fusazen design) at equal size (its own JSON line; the default workload is untouched)")
    ap.add_argument("--design-sizes", default="2048,1024", help="with --design: which of " + ", ".join(sorted(set(DESIGN_SIZES) | set(GEMOSUN_SIZES))))
    args = ap.parse_args()

    if args.design:
        if args.gpus != 1:
            print("bench.py: this library runs on one GPU; --gpus must be 1")
            return 2
        return design_run(args.design, max(args.steps, 1) if args.steps != 256 else 64, max(args.warmup, 3), args.batch,
                          args.context, args.prefill_tokens, [x.strip() for x in args.design_sizes.split(",") if x.strip()])
    if args.impl == "reference":
        if args.gpus != 1:
            print(json.dumps({"impl": "reference", "unavailable": "the reference runs on the CPU of one machine; --gpus must be 1"}))
            return 0
        # the unmodified reference through its own command line (a CMake C++ project: the offline pip install has
        # nothing to install — 'Neither setup.py nor pyproject.toml found' — so it is built with its own CMake files)
        from baseline import reference_arm
        return reference_arm.main(dict(CONFIG, num_hidden_layers=args.layers), args.batch, args.context, PREFILL_TOKENS,
                                  args.steps, args.warmup, FULL_LAYERS)
    if args.gpus != 1:
        print("bench.py: this library runs on one GPU; --gpus must be 1")
        return 2
    if args.workload:
        return workload_run(args.workload, [d.strip() for d in args.workload_dtypes.split(",") if d.strip()])
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)

    import torch
    import llmi_b200 as L
    pk, pk_kind = peaks()
    cfg = dict(CONFIG, num_hidden_layers=args.layers)
    if args.kv_heads is not None:
        if args.only is None:
            print("bench.py: --kv-heads changes the model's shape; it goes with --only (no bench line)")
            return 2
        cfg["num_key_value_heads"] = args.kv_heads
    t0 = time.time()
    model = L.random_model(cfg, seed=0, dtype="bfloat16", on_device=True)
    weight_bytes = model.weight_bytes()

    if args.only == "prefill":
        T = args.prefill_tokens
        pre_ms = prefill_run(model, T, iters=3)
        frac = prefill_flops(cfg, args.layers, T) / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)
        print(json.dumps({"only": "prefill", "ms": round(pre_ms, 3), "tokens": T, "layers": args.layers,
                          "tokens_per_s": round(T * 1000.0 / pre_ms, 1), "frac_of_bf16_peak": round(frac, 4), "peaks": pk_kind}))
        return 0
    if args.only == "decode":
        ms, launches, _, _, cache_bytes = decode_run(model, args.batch, args.context, steps, warmup)
        gbs = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9
        print(json.dumps({"only": "decode", "ms_per_step": round(ms, 4), "batch": args.batch, "context": args.context,
                          "layers": args.layers, "kv_heads": cfg["num_key_value_heads"], "gpu_launches": launches,
                          "tokens_per_s": round(args.batch * 1000.0 / ms, 1), "gb_per_s": round(gbs, 1),
                          "frac_of_hbm_peak": round(gbs / pk["hbm_gbs"], 4), "peaks": pk_kind}))
        return 0

    clocks = ClockSampler()
    clocks.start()
    ms, launches, _, _, cache_bytes = decode_run(model, args.batch, args.context, steps, warmup, clocks=clocks)
    clock_info = clocks.stop()
    value = args.batch * 1000.0 / ms
    ms_e2e, _, h2d, d2h, _ = decode_run(model, args.batch, args.context, steps, warmup, e2e=True)
    step_bytes = weight_bytes + cache_bytes
    achieved = step_bytes / (ms * 1e-3) / 1e9

    pre_ms = prefill_run(model, PREFILL_TOKENS)
    pre_flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            pms, *_ = decode_run(model, b, args.context, min(steps, 32), warmup)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)

    out = {
        "metric": "decode tok/s at batch 8, context 4096 (SmolLM2-1.7B shape)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids, random cache contents)",
        "impl": "ours",
        "config": {"model": "SmolLM2-1.7B shape", "layers": args.layers, "layers_full": FULL_LAYERS, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "rope_theta": cfg["rope_theta"],
                   "rms_norm_eps": cfg["rms_norm_eps"], "tied": True, "global_batch": args.batch, "seq_len": args.context,
                   "prefill_tokens": PREFILL_TOKENS, "parallelism": "1 GPU", "weights": "random bf16",
                   "l2": "inputs larger than L2 (a step reads %.1f GB)" % (step_bytes / 1e9), "peaks": pk_kind},
        "e2e": {"value": round(args.batch * 1000.0 / ms_e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": round(ms_e2e, 4)},
        "gpu_launches": int(launches),
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_info,
        "setup_seconds": round(time.time() - t0, 1),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
