"""Decode and prefill throughput of Qwen3 layer sizes with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--size 4b|8b|14b] [--batch 8] [--layers N]
                    [--impl ours|reference]

Prints ONE JSON line. ``value`` is decoded tokens per second at the default batch of 8: K decode
steps of the generation loop's own decode state (CUDA-graph replay), timed with CUDA events after W
warm-up steps (at least 32 untimed steps in both arms, see MIN_UNTIMED_STEPS; the count is named in
``config.untimed_steps``), every sequence at the midpoint of the size's workload: for ``4b`` a 2,048-token
prompt (ragged 1,024..2,048 above batch 1) plus 1,024 tokens decoded so far of a 4,096-token
context; ``8b`` 1,024 + 512 of 1,024; ``14b`` 2,048 + 256 of 512. ``e2e`` is the same measured
through ``Engine.generate`` (host token lists in, host tokens out). ``prefill`` is one 2,048-token
prompt; ``roofline`` relates the decode step to the bytes it must read; ``points`` hold the size's
other two batch sizes, each with its own step time, roofline fraction and clocks. The weights (8 to
28 GB) are far larger than L2, so no flush is needed between steps. For more than one GPU it says
so and exits with 2: this library runs on one.

``--impl reference`` times the unmodified reference engine (a copy of its folder under
``baseline/_ref``) through its own ``Engine(model_path)`` and ``Engine.generate`` on a model folder
of the same sizes written here with plain torch; nothing of this library is imported on that arm.
"""
import argparse
import contextlib
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

_COMMON = dict(architectures=["Qwen3ForCausalLM"], vocab_size=151936, num_key_value_heads=8, head_dim=128,
               rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960)
# layer sizes, and the workload each is quoted on: prompt length (ragged from half of it above batch 1 where
# `ragged`), decode steps of the whole run (timed at their midpoint), batch sizes
SIZES = {
    "4b": dict(config=dict(_COMMON, hidden_size=2560, intermediate_size=9728, num_hidden_layers=36,
                           num_attention_heads=32, tie_word_embeddings=True),
               name="Qwen3-4B", prompt=2048, ragged=True, decode=2048, batches=(1, 8, 64)),
    "8b": dict(config=dict(_COMMON, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                           num_attention_heads=32, tie_word_embeddings=False),
               name="Qwen3-8B", prompt=1024, ragged=False, decode=1024, batches=(1, 8, 64)),
    "14b": dict(config=dict(_COMMON, hidden_size=5120, intermediate_size=17408, num_hidden_layers=40,
                            num_attention_heads=40, tie_word_embeddings=False),
                name="Qwen3-14B", prompt=2048, ragged=False, decode=512, batches=(1, 8, 32)),
}
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]), source="measured")
    except Exception:
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.lines, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.proc.wait()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6 or not parts[0].isdigit():
                continue
            sm.append(int(parts[0]))
            mx.append(int(parts[1]))
            reasons.update(n for n, v in zip(names, parts[2:]) if v == "Active")
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": int(statistics.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def prompt_lengths(size, batch, seed):
    """Context each sequence holds when the timed steps begin: its prompt plus half of the run's decode steps."""
    import numpy as np
    w = SIZES[size]
    so_far = w["decode"] // 2
    if batch == 1 or not w["ragged"]:
        return [w["prompt"] + so_far] * batch
    r = np.random.RandomState(seed)
    return [int(x) + so_far for x in r.randint(w["prompt"] // 2, w["prompt"] + 1, batch)]


def random_prompts(vocab, lens, seed):
    import numpy as np
    rs = np.random.RandomState(seed + 1)
    return [rs.randint(0, vocab, n).tolist() for n in lens]


def kv_bytes_per_token(cfg):
    return cfg["num_hidden_layers"] * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def weight_bytes(cfg):
    """Bytes of bfloat16 weights a decode step reads: every matrix once, the head once (the embedding is
    read by row only, so it counts only where it is also the head)."""
    H, hd = cfg["hidden_size"], cfg["head_dim"]
    per_layer = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * hd * H + H * cfg["num_attention_heads"] * hd \
        + 3 * cfg["intermediate_size"] * H
    return 2 * (per_layer * cfg["num_hidden_layers"] + cfg["vocab_size"] * H)


def prefill_flops(cfg, tokens):
    H, hd, nh = cfg["hidden_size"], cfg["head_dim"], cfg["num_attention_heads"]
    per_layer = (nh + 2 * cfg["num_key_value_heads"]) * hd * H + H * nh * hd + 3 * cfg["intermediate_size"] * H
    L = cfg["num_hidden_layers"]
    return 2 * per_layer * L * tokens + 4 * nh * hd * tokens * (tokens + 1) / 2 * L + 2 * cfg["vocab_size"] * H


# ------------------------------------------------------------------------------------ this library
# Untimed steps before the timed ones: the W asked for, and at least this many, in both arms (after a
# prefill under the power cap the SM clock needs some tens of steps to settle; with five untimed steps
# the same step measured 5 % slower than with fifty). The count used is named in config.untimed_steps.
MIN_UNTIMED_STEPS = 32


def time_decode(torch, dk, model, cfg, size, batch, steps, warmup, seed):
    """K decode steps of the generation loop's own decode state (graph replay), timed on the device
    after ``warmup`` untimed ones."""
    from dryft_challenge_htn_2026_b200.csrc import api
    from dryft_challenge_htn_2026_b200.engine.generate import GpuBackend
    from dryft_challenge_htn_2026_b200.sampling import SamplingParams

    lens = prompt_lengths(size, batch, seed)
    total_new = warmup + steps + 8
    need = sum((n + total_new + 63) // 64 * 64 for n in lens)
    runner = dk.Runner(model, need, max_slots=max(batch, 1))
    backend = GpuBackend(runner, use_graph=True)
    prompts = random_prompts(model.spec.vocab_size, lens, seed)
    backend.start(prompts, SamplingParams(total_new), [0] * batch).wait()    # prefill (steps of at most 32k tokens), first token
    st = backend.state
    count0 = api.launch_count()
    st.body(advance=False, out_tok=torch.empty_like(st.ctx.tok))
    launches_per_step = api.launch_count() - count0
    st.capture()
    for _ in range(warmup):
        st.run()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    with ClockSampler() as cs:
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(steps):
            st.run()
        ev[1].record()
        torch.cuda.synchronize()
    ms = ev[0].elapsed_time(ev[1]) / steps
    ctx_mean = sum(lens) / batch + warmup + steps / 2
    step_bytes = model.weight_bytes_per_step() + batch * ctx_mean * kv_bytes_per_token(cfg)
    backend.finish()
    del st, backend, runner
    torch.cuda.empty_cache()
    return dict(ms=ms, tok_s=batch / ms * 1e3, bytes=step_bytes, ctx_mean=ctx_mean, launches=launches_per_step,
                clocks=cs.summary())


def time_prefill(torch, dk, model, cfg, tokens, iters=3):
    """One prompt of ``tokens`` tokens through the step function as generation calls it (a step shape
    that repeats is replayed as a CUDA graph): two untimed runs (plain, then the capture), then the
    median of ``iters`` runs, each between synchronisations, timed with CUDA events."""
    import numpy as np
    runner = dk.Runner(model, tokens + 64, max_slots=2)
    prompt = np.random.RandomState(7).randint(0, model.spec.vocab_size, tokens).tolist()
    times = []
    for i in range(iters + 2):
        slot = runner.begin()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([(slot, prompt, [tokens - 1])], graph=True)
        e1.record()
        torch.cuda.synchronize()
        runner.end(slot)
        if i >= 2:
            times.append(e0.elapsed_time(e1))
    del runner
    torch.cuda.empty_cache()
    return statistics.median(times), prefill_flops(cfg, tokens)


def time_e2e(torch, dk, model, size, batch, steps, warmup, seed):
    """Decode tokens per second through Engine.generate: host lists in, host tokens out; wall clock at
    each yield, the timed steps those between yield number ``warmup`` and yield ``warmup + steps`` of
    one call (what the reference arm's number is, see ref_decode)."""
    lens = prompt_lengths(size, batch, seed)
    prompts = random_prompts(model.spec.vocab_size, lens, seed)
    eng = dk.Engine(model=model)
    list(eng.generate(prompts, 4))          # first call: allocations and the graph of this batch shape (kept by the engine)
    stamps = [time.perf_counter() for _ in eng.generate(prompts, warmup + steps + 1)]
    assert len(stamps) == warmup + steps + 1
    h2d = sum(len(p) for p in prompts) * 3 * 4 / (warmup + steps + 1)     # token ids, row->sequence, positions, once
    del eng
    torch.cuda.empty_cache()
    return batch * steps / (stamps[warmup + steps] - stamps[warmup]), h2d, 4 * batch


def point(run, pk):
    achieved = run["bytes"] / (run["ms"] * 1e-3) / 1e9
    return {"value": round(run["tok_s"], 1), "ms_per_step": round(run["ms"], 4), "ctx_mean": round(run["ctx_mean"]),
            "roofline_frac": round(achieved / pk["hbm_gbs"], 4), "clocks": run["clocks"]}


def config_record(size, cfg, layers_full, batch, pk, **more):
    w = SIZES[size]
    rec = {"model": f"{w['name']} layer sizes", "global_batch": batch, "seq_len": w["prompt"] + w["decode"],
           "parallelism": "1gpu", "layers": cfg["num_hidden_layers"], "layers_full": layers_full,
           "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
           "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
           "tied_head": bool(cfg["tie_word_embeddings"]),
           "prompt_len": f"{w['prompt']}" + (f" ({w['prompt'] // 2}..{w['prompt']} ragged above batch 1)" if w["ragged"] else ""),
           "l2": "inputs larger than L2 (GBs of weights per step)", "peaks": pk["source"]}
    rec.update(more)
    return rec


def run_ours(args):
    import torch

    import dryft_challenge_htn_2026_b200 as dk
    from dryft_challenge_htn_2026_b200.csrc import api

    size = args.size
    cfg_d = dict(SIZES[size]["config"])
    full_layers = cfg_d["num_hidden_layers"]
    if args.layers:
        cfg_d["num_hidden_layers"] = args.layers
    cfg = dk.config_from_dict(cfg_d)
    api.set_pdl(bool(args.pdl))
    model = dk.random_model(cfg, seed=0, dtype=torch.bfloat16)
    pk = peaks()
    warmup = max(3, args.warmup)

    if args.prefill_only:
        ms, flops = time_prefill(torch, dk, model, cfg_d, args.prefill_tokens)
        print(json.dumps({"prefill": {"value": round(args.prefill_tokens / ms * 1e3, 1), "tokens": args.prefill_tokens,
                                      "ms": round(ms, 3), "layers": cfg.num_hidden_layers,
                                      "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}}))
        return 0
    untimed = max(warmup, MIN_UNTIMED_STEPS)
    main_run = time_decode(torch, dk, model, cfg_d, size, args.batch, args.steps, untimed, seed=0)
    e2e_val, h2d, d2h = time_e2e(torch, dk, model, size, args.batch, args.steps, untimed, seed=0)
    points, detail, prefill = {}, {}, None
    if not args.no_points:
        for b in SIZES[size]["batches"]:
            if b != args.batch:
                detail[f"decode_b{b}"] = point(time_decode(torch, dk, model, cfg_d, size, b, max(64, args.steps), untimed, seed=b), pk)
                points[f"decode_b{b}"] = detail[f"decode_b{b}"]["value"]
        ms, flops = time_prefill(torch, dk, model, cfg_d, PREFILL_TOKENS)
        prefill = {"value": round(PREFILL_TOKENS / ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
                   "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                   "short_ms": {str(n): round(time_prefill(torch, dk, model, cfg_d, n)[0], 3) for n in (128, 512)}}
    achieved = main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({SIZES[size]['name']}, bf16)", "value": round(main_run["tok_s"], 1),
        "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(main_run["ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": config_record(size, cfg_d, full_layers, args.batch, pk, ctx_mean_timed=round(main_run["ctx_mean"]),
                                pdl=bool(args.pdl), untimed_steps=untimed),
        "clocks": main_run["clocks"],
        "e2e": {"value": round(e2e_val, 1), "unit": "tok/s", "h2d_bytes_per_step": round(h2d), "d2h_bytes_per_step": d2h},
        "gpu_launches": main_run["launches"] * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if prefill is not None:
        out["prefill"] = prefill
        out["points"] = points
        out["points_detail"] = detail
    print(json.dumps(out))
    return 0


# --------------------------------------------------------------- another design beside Qwen3 at equal size
def nilivik_config(width, heads, kv_heads, ff_qwen, layers, vocab, chunk):
    """A Nilivik model of Qwen3's width, head size 128 and layer count, with as many parameters a layer:
    chunked attention of Qwen3's head counts, linear attention of half as many heads, and a feed-forward
    sized so that the layer's matrices add up to Qwen3's."""
    hd, rh = 128, heads // 2
    qwen = (heads + 2 * kv_heads) * hd + heads * hd + 3 * ff_qwen            # matrix columns of a Qwen3 layer, per width
    mix = (2 * heads + 2 * kv_heads) * hd + heads * hd + 4 * rh * hd + rh * hd
    ff = max(256, (qwen - mix) // 2 // 64 * 64)
    layer = {"type": "parallel",
             "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": hd, "vdim": hd, "mask": {"size": chunk},
                                "scale": hd ** -0.5},
                       "right": {"heads": rh, "dim": hd, "vdim": hd, "decay": [1.0 - 2.0 ** -(3 + 5 * i / max(1, rh - 1)) for i in range(rh)]},
                       "left_scale": 0.7, "right_scale": 0.7},
             "mlp": {"kind": "dense", "ff": ff}}
    return dict(architecture="Nilivik", vocab=vocab, width=width, embedding={"scale": 1.0}, norm={"eps": 1e-6},
                logit_softcap=30.0, layers=[layer] * layers)


def time_step_prefill(torch, dk, model, tokens, iters=3):
    import numpy as np
    runner = dk.Runner(model, tokens + 64, max_slots=2)
    prompt = np.random.RandomState(7).randint(0, model.spec.vocab_size, tokens).tolist()
    times = []
    for i in range(iters + 2):
        slot = runner.begin()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([(slot, prompt, [tokens - 1])], graph=True)
        e1.record()
        torch.cuda.synchronize()
        runner.end(slot)
        if i >= 2:
            times.append(e0.elapsed_time(e1))
    del runner
    torch.cuda.empty_cache()
    return statistics.median(times)


def time_step_decode(torch, dk, model, batch, context, steps, warmup):
    """Decode steps of the generation loop's decode state (graph replay) for ``batch`` sequences that hold
    ``context`` tokens each; returns (ms a step, kernels a step)."""
    from dryft_challenge_htn_2026_b200.csrc import api
    from dryft_challenge_htn_2026_b200.engine.generate import GpuBackend
    from dryft_challenge_htn_2026_b200.sampling import SamplingParams
    total_new = warmup + steps + 8
    runner = dk.Runner(model, batch * ((context + total_new + 63) // 64 * 64), max_slots=batch)
    backend = GpuBackend(runner, use_graph=True)
    prompts = random_prompts(model.spec.vocab_size, [context] * batch, 3)
    backend.start(prompts, SamplingParams(total_new), [0] * batch).wait()
    st = backend.state
    saved = runner.cache.state_snapshot([slot for slot, _ in st.filled])
    count0 = api.launch_count()
    st.body(advance=False, out_tok=torch.empty_like(st.ctx.tok))
    launches = api.launch_count() - count0
    runner.cache.state_restore(saved)
    st.capture()
    for _ in range(warmup):
        st.run()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record()
    for _ in range(steps):
        st.run()
    ev[1].record()
    torch.cuda.synchronize()
    ms = ev[0].elapsed_time(ev[1]) / steps
    backend.finish()
    del st, backend, runner
    torch.cuda.empty_cache()
    return ms, launches


def kernel_times(torch, dk, pk, heads, kv_heads, rh, chunk):
    """The new design's mixer kernels alone, beside the attention kernels of Qwen3 at the same head counts:
    CUDA events around one launch, L2 flushed before each (a 256 MB write), median of 5 after 2 untimed."""
    from dryft_challenge_htn_2026_b200.cache import Cache, KVRequest, StateRequest
    from dryft_challenge_htn_2026_b200.csrc import api
    from dryft_challenge_htn_2026_b200.engine.batch import build_context
    from dryft_challenge_htn_2026_b200.parts.attention import QueryTiles
    dev, bf = torch.device("cuda"), torch.bfloat16
    hd = 128
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)

    def timed(fn):
        ts = []
        for i in range(7):
            flush.fill_(float(i))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts[2:]) * 1e3        # microseconds

    out = {}
    r1 = torch.full((heads,), 0.3, device=dev)
    r2 = torch.full((heads,), 0.1, device=dev)
    sink = torch.zeros(heads, device=dev)
    decay = torch.tensor([1.0 - 2.0 ** -(3 + 5 * i / max(1, rh - 1)) for i in range(rh)], dtype=torch.float32, device=dev)
    for tokens in (2048, 8192):
        # ---- prompts: masked attention (this design) and Qwen3's attention, one sequence of ``tokens``
        plans = [QueryTiles(api.MASKED_TILE_ROWS), QueryTiles(api.TC_TILE_ROWS)]
        cache = Cache([[KVRequest(kv_heads, hd, None, bf, hd, chunk)], [KVRequest(kv_heads, hd, None, bf)],
                       [StateRequest((rh, hd, hd), torch.float32)]], tokens + 64, 2, dev)
        slot = cache.begin()
        ctx = build_context(cache, [(slot, [0] * tokens, [])], dev, plans=plans)
        q = torch.randn(tokens, heads * hd, device=dev).to(bf)
        g = torch.randn(tokens, heads * hd, device=dev).to(bf)
        o = torch.empty_like(q)
        for e in (0, 1):
            v = cache.views(e)[0]
            v.k.normal_(), v.v.normal_()
        m, f, stt = cache.views(0)[0], cache.views(1)[0], cache.views(2)[0].state
        seen = sum(min(i % chunk, i) + 1 for i in range(tokens))
        us = timed(lambda: api.attention_masked_prefill_bf16(q, o, g, 0.7, m.k, m.v, ctx.plans[plans[0].key], ctx.cu_q, ctx.seq_pos0,
                                                             ctx.tables[m.group], heads, kv_heads, hd, hd, None, chunk, hd ** -0.5, r1, r2, sink))
        out[f"masked_attention_prefill_mma_sync_{tokens}"] = {"us": round(us, 1), "tflops": round(4 * heads * hd * seen / us / 1e6, 1),
                                                              "frac_bf16": round(4 * heads * hd * seen / us / 1e6 / pk["bf16_tflops"], 4)}
        us = timed(lambda: api.attention_masked_prefill_tc(q, o, g, 0.7, m.k, m.v, ctx.plans[plans[1].key], ctx.cu_q, ctx.seq_pos0,
                                                           ctx.tables[m.group], heads, kv_heads, hd, None, chunk, hd ** -0.5, r1, r2, sink))
        out[f"masked_attention_prefill_{tokens}"] = {"us": round(us, 1), "tflops": round(4 * heads * hd * seen / us / 1e6, 1),
                                                     "frac_bf16": round(4 * heads * hd * seen / us / 1e6 / pk["bf16_tflops"], 4)}
        full = tokens * (tokens + 1) // 2
        us = timed(lambda: api.attention_prefill_tc(q, o, f.k, f.v, ctx.plans[plans[1].key], ctx.cu_q, ctx.seq_pos0, ctx.tables[f.group],
                                                    heads, kv_heads, hd, None, hd ** -0.5))
        out[f"qwen3_attention_prefill_{tokens}"] = {"us": round(us, 1), "tflops": round(4 * heads * hd * full / us / 1e6, 1),
                                                    "frac_bf16": round(4 * heads * hd * full / us / 1e6 / pk["bf16_tflops"], 4)}
        # ---- prompts: linear attention in blocks of 64 tokens; what it must move: q, k, v in, float32 o out
        x = torch.randn(tokens, 3 * rh * hd, device=dev).to(bf)
        lo = torch.empty(tokens, rh * hd, dtype=torch.float32, device=dev)
        us = timed(lambda: api.linear_attention(x[:, :rh * hd], x[:, rh * hd:2 * rh * hd], x[:, 2 * rh * hd:], lo, stt, ctx.cu_q, ctx.seq_pos0,
                                                ctx.seq_slot, decay, 1, rh, hd, hd, tokens))
        moved = tokens * rh * hd * (3 * 2 + 4)
        flops = tokens * rh * (2 * 64 * 2 * hd + 4 * hd * hd)
        out[f"linear_attention_prefill_{tokens}"] = {"us": round(us, 1), "gbs": round(moved / us / 1e3, 1),
                                                     "frac_hbm": round(moved / us / 1e3 / pk["hbm_gbs"], 4),
                                                     "tflops": round(flops / us / 1e6, 2)}
        cache.end(slot)
        del cache, q, g, o, x, lo
    for batch in (8, 64):
        # ---- single tokens: every sequence holds 3,000 tokens (952 of them in the newest chunk of 2,048)
        context = 3000
        cache = Cache([[KVRequest(kv_heads, hd, None, bf, hd, chunk)], [KVRequest(kv_heads, hd, None, bf)],
                       [StateRequest((rh, hd, hd), torch.float32)]], batch * (context + 64), batch, dev)
        slots = [cache.begin() for _ in range(batch)]
        for sl in slots:
            cache.reserve(sl, context)
            cache.length[sl] = context
        ctx = build_context(cache, [(sl, [0], []) for sl in slots], dev)
        for e in (0, 1):
            v = cache.views(e)[0]
            v.k.normal_(), v.v.normal_()
        m, f, stt = cache.views(0)[0], cache.views(1)[0], cache.views(2)[0].state
        q = torch.randn(batch, heads * hd, device=dev).to(bf)
        g = torch.randn(batch, heads * hd, device=dev).to(bf)
        o = torch.empty_like(q)
        keys = context - context // chunk * chunk + 1
        table = ctx.tables[m.group]
        span = api.masked_decode_span(heads, kv_heads, hd, None, chunk, table.shape[1], batch)
        mws = api.masked_decode_ws(batch, heads, hd, span[1], dev)
        us = timed(lambda: api.attention_masked_decode_bf16(q, o, g, 0.7, m.k, m.v, ctx.row_pos, table, heads, kv_heads, hd, hd, None,
                                                            chunk, hd ** -0.5, span, r1, r2, sink, None, None, mws))
        moved = batch * kv_heads * keys * 2 * hd * 2
        out[f"masked_attention_decode_block_kernel_b{batch}"] = {"us": round(us, 1), "keys": keys, "gbs": round(moved / us / 1e3, 1),
                                                                 "frac_hbm": round(moved / us / 1e3 / pk["hbm_gbs"], 4)}
        ns = api.masked_decode_splits(batch, kv_heads, heads // kv_heads, table.shape[1], None, chunk)
        mws2 = api.attention_decode_ws(batch, heads, hd, ns, dev)
        us = timed(lambda: api.attention_decode_masked_bf16(q, o, g, 0.7, m.k, m.v, ctx.row_pos, table, heads, kv_heads, hd, None, chunk,
                                                            hd ** -0.5, ns, mws2[0], mws2[1], r1, r2, sink))
        out[f"masked_attention_decode_b{batch}"] = {"us": round(us, 1), "keys": keys, "gbs": round(moved / us / 1e3, 1),
                                                    "frac_hbm": round(moved / us / 1e3 / pk["hbm_gbs"], 4)}
        nsplit = api.decode_splits(batch, kv_heads, heads // kv_heads, ctx.tables[f.group].shape[1])
        ws = api.attention_decode_ws(batch, heads, hd, nsplit, dev)
        us = timed(lambda: api.attention_decode_bf16(q, o, f.k, f.v, ctx.row_pos, ctx.tables[f.group], heads, kv_heads, hd, None,
                                                     hd ** -0.5, nsplit, *ws))
        moved = batch * kv_heads * (context + 1) * 2 * hd * 2
        out[f"qwen3_attention_decode_b{batch}"] = {"us": round(us, 1), "keys": context + 1, "gbs": round(moved / us / 1e3, 1),
                                                   "frac_hbm": round(moved / us / 1e3 / pk["hbm_gbs"], 4)}
        x = torch.randn(batch, 3 * rh * hd, device=dev).to(bf)
        lo = torch.empty(batch, rh * hd, dtype=torch.float32, device=dev)
        us = timed(lambda: api.linear_attention(x[:, :rh * hd], x[:, rh * hd:2 * rh * hd], x[:, 2 * rh * hd:], lo, stt, None, ctx.row_pos,
                                                ctx.seq_slot, decay, batch, rh, hd, hd, 1))
        moved = batch * rh * hd * hd * 4 * 2
        out[f"linear_attention_decode_b{batch}"] = {"us": round(us, 1), "gbs": round(moved / us / 1e3, 1),
                                                    "frac_hbm": round(moved / us / 1e3 / pk["hbm_gbs"], 4)}
        del cache, q, g, o, x, lo
    torch.cuda.empty_cache()
    return out


def pibulix_config(width, heads, kv_heads, ff_qwen, layers, vocab, window):
    """A Pibulix model of Qwen3's width, head size 128 and layer count: attention layers of Qwen3's head counts (4 taps,
    half the head rotated, a window that keeps 4 tokens, capped scores) with a dense feed-forward of Qwen3's size, in
    turn with gated-linear-attention layers of half as many heads whose mixture of 32 experts uses 4 a token, each a
    quarter of Qwen3's feed-forward (so that a token's feed-forward arithmetic is Qwen3's), plus a shared expert."""
    hd, gh = 128, heads // 2
    eff = max(64, ff_qwen // 4 // 64 * 64)
    att = {"type": "attention",
           "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": hd, "vdim": hd, "conv": 4, "scale": hd ** -0.5, "softcap": 50.0,
                     "rot": {"dims": hd // 2, "base": 1e6}, "mask": {"size": window, "keep_first": 4}},
           "mlp": {"kind": "dense", "ff": ff_qwen}}
    gla = {"type": "gla", "mixer": {"heads": gh, "dim": hd, "vdim": hd, "tau": 16.0},
           "mlp": {"kind": "moe", "expert": {"ff": eff}, "shared": {"ff": eff},
                   "router": {"experts": 32, "top": 4, "scale": 2.5, "groups": {"count": 4, "keep": 2}}}}
    return dict(architecture="Pibulix", vocab=vocab, width=width, norm={"eps": 1e-6}, postln_alpha=2.0,
                layers=[att if i % 2 == 0 else gla for i in range(layers)])


def pibulix_kernel_times(torch, dk, pk, width, heads, kv_heads, ff_qwen, window):
    """The design's own kernels alone, beside Qwen3's like kernels at the same head counts: CUDA events around one launch
    (or one part's forward), L2 flushed before each (a 256 MB write), median of 5 after 2 untimed."""
    from dryft_challenge_htn_2026_b200.cache import Cache, KVRequest, StateRequest
    from dryft_challenge_htn_2026_b200.config.specs import GatedMLPSpec, RoutedMLPSpec
    from dryft_challenge_htn_2026_b200.csrc import api
    from dryft_challenge_htn_2026_b200.engine.batch import build_context
    from dryft_challenge_htn_2026_b200.parts import Runtime, build_part
    from dryft_challenge_htn_2026_b200.parts.attention import QueryTiles
    dev, bf = torch.device("cuda"), torch.bfloat16
    hd, gh, keep, cap = 128, heads // 2, 4, 50.0
    eff = max(64, ff_qwen // 4 // 64 * 64)
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)

    def timed(fn):
        ts = []
        for i in range(7):
            flush.fill_(float(i))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts[2:]) * 1e3        # microseconds

    def flops_rec(us, flops):
        return {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1), "frac_bf16": round(flops / us / 1e6 / pk["bf16_tflops"], 4)}

    def bytes_rec(us, moved):
        return {"us": round(us, 1), "gbs": round(moved / us / 1e3, 1), "frac_hbm": round(moved / us / 1e3 / pk["hbm_gbs"], 4)}

    out = {}
    sink = torch.zeros(heads, device=dev)
    rt = Runtime(dev, bf)
    moe = build_part(RoutedMLPSpec(width, eff, 32, 4, 4, 2, 2.5, eff), rt)
    dense = build_part(GatedMLPSpec(width, ff_qwen), rt)
    g = torch.Generator(device=dev).manual_seed(1)
    for part in (moe, dense):
        part.bind({d.name: (torch.randn(d.shape, generator=g, device=dev) * (0.2 if d.init == "wide" else 0.02)).to(
            torch.float32 if d.keep_float32 else bf) for d in part.param_decls()})
    scratch = {}

    class Ctx:
        def scratch(self, key, make):
            if key not in scratch:
                scratch[key] = make()
            return scratch[key]
    for tokens in (2048, 8192):
        plans = [QueryTiles(api.TC_TILE_ROWS)]
        cache = Cache([[KVRequest(kv_heads, hd, window, bf, hd, None, keep)], [KVRequest(kv_heads, hd, None, bf)],
                       [StateRequest((gh, hd, hd), torch.float32)]], tokens + 64, 2, dev)
        slot = cache.begin()
        ctx = build_context(cache, [(slot, [0] * tokens, [])], dev, plans=plans)
        q = torch.randn(tokens, heads * hd, device=dev).to(bf)
        o = torch.empty_like(q)
        for e in (0, 1):
            v = cache.views(e)[0]
            v.k.normal_(), v.v.normal_()
        m, f, stt = cache.views(0)[0], cache.views(1)[0], cache.views(2)[0].state
        seen = sum(min(i + 1, window) + min(keep, max(0, i + 1 - window)) for i in range(tokens))
        us = timed(lambda: api.attention_masked_prefill_tc(q, o, None, 1.0, m.k, m.v, ctx.plans[plans[0].key], ctx.cu_q, ctx.seq_pos0,
                                                           ctx.tables[m.group], heads, kv_heads, hd, window, None, hd ** -0.5, None, None,
                                                           sink, cap, keep))
        out[f"window_attention_prefill_{tokens}"] = flops_rec(us, 4 * heads * hd * seen)
        us = timed(lambda: api.attention_masked_prefill_tc(q, o, None, 1.0, m.k, m.v, ctx.plans[plans[0].key], ctx.cu_q, ctx.seq_pos0,
                                                           ctx.tables[m.group], heads, kv_heads, hd, window, None, hd ** -0.5, None, None,
                                                           sink, None, keep))
        out[f"window_attention_prefill_without_cap_{tokens}"] = flops_rec(us, 4 * heads * hd * seen)
        full = tokens * (tokens + 1) // 2
        us = timed(lambda: api.attention_prefill_tc(q, o, f.k, f.v, ctx.plans[plans[0].key], ctx.cu_q, ctx.seq_pos0, ctx.tables[f.group],
                                                    heads, kv_heads, hd, None, hd ** -0.5))
        out[f"qwen3_attention_prefill_{tokens}"] = flops_rec(us, 4 * heads * hd * full)
        # ---- prompts: gated linear attention; what it must move: q, k, v in, the decay's float32 rows in, float32 o out
        x = torch.randn(tokens, 3 * gh * hd, device=dev).to(bf)
        z = torch.randn(tokens, gh * hd, device=dev)
        zb = torch.zeros(gh * hd, device=dev)
        lo = torch.empty(tokens, gh * hd, dtype=torch.float32, device=dev)
        us = timed(lambda: api.gated_linear_attention(x[:, :gh * hd], x[:, gh * hd:2 * gh * hd], x[:, 2 * gh * hd:], lo, stt, ctx.cu_q,
                                                           ctx.seq_pos0, ctx.seq_slot, z, zb, 16.0, hd ** -0.5, 1, gh, hd, hd))
        out[f"gated_linear_attention_prefill_{tokens}"] = bytes_rec(us, tokens * gh * hd * (3 * 2 + 4 + 4))
        # ---- prompts: the routed feed-forward beside Qwen3's dense one (a token's arithmetic is the same but for the shared expert)
        a = torch.randn(tokens, width, device=dev).to(bf)
        us = timed(lambda: moe.forward(Ctx(), a))
        out[f"routed_feed_forward_prefill_{tokens}"] = flops_rec(us, tokens * 5 * 6 * eff * width)
        us = timed(lambda: dense.forward(None, a))
        out[f"qwen3_feed_forward_prefill_{tokens}"] = flops_rec(us, tokens * 6 * ff_qwen * width)
        cache.end(slot)
        del cache, q, o, x, z, lo, a
    for batch in (8, 64):
        # ---- single tokens: every sequence holds 3,000 tokens, of which the window and the kept ones are read
        context = 3000
        cache = Cache([[KVRequest(kv_heads, hd, None, bf, hd, None, keep)], [KVRequest(kv_heads, hd, None, bf)],
                       [StateRequest((gh, hd, hd), torch.float32)]], batch * (context + 64), batch, dev)
        slots = [cache.begin() for _ in range(batch)]
        for sl in slots:
            cache.reserve(sl, context)
            cache.length[sl] = context
        ctx = build_context(cache, [(sl, [0], []) for sl in slots], dev)
        for e in (0, 1):
            v = cache.views(e)[0]
            v.k.normal_(), v.v.normal_()
        m, f, stt = cache.views(0)[0], cache.views(1)[0], cache.views(2)[0].state
        q = torch.randn(batch, heads * hd, device=dev).to(bf)
        o = torch.empty_like(q)
        table = ctx.tables[m.group]
        keys = min(window, context + 1) + keep
        ns = api.masked_decode_splits(batch, kv_heads, heads // kv_heads, table.shape[1], window, None)
        ws = api.attention_decode_ws(batch, heads, hd, ns, dev)
        us = timed(lambda: api.attention_decode_masked_bf16(q, o, None, 1.0, m.k, m.v, ctx.row_pos, table, heads, kv_heads, hd, window, None,
                                                            hd ** -0.5, ns, ws[0], ws[1], None, None, sink, cap, keep))
        out[f"window_attention_decode_b{batch}"] = dict(bytes_rec(us, batch * kv_heads * keys * 2 * hd * 2), keys=keys)
        nsplit = api.decode_splits(batch, kv_heads, heads // kv_heads, ctx.tables[f.group].shape[1])
        ws2 = api.attention_decode_ws(batch, heads, hd, nsplit, dev)
        us = timed(lambda: api.attention_decode_bf16(q, o, f.k, f.v, ctx.row_pos, ctx.tables[f.group], heads, kv_heads, hd, None,
                                                     hd ** -0.5, nsplit, *ws2))
        out[f"qwen3_attention_decode_b{batch}"] = dict(bytes_rec(us, batch * kv_heads * (context + 1) * 2 * hd * 2), keys=context + 1)
        x = torch.randn(batch, 3 * gh * hd, device=dev).to(bf)
        z = torch.randn(batch, gh * hd, device=dev)
        zb = torch.zeros(gh * hd, device=dev)
        lo = torch.empty(batch, gh * hd, dtype=torch.float32, device=dev)
        us = timed(lambda: api.gated_linear_attention(x[:, :gh * hd], x[:, gh * hd:2 * gh * hd], x[:, 2 * gh * hd:], lo, stt, None,
                                                           ctx.row_pos, ctx.seq_slot, z, zb, 16.0, hd ** -0.5, batch, gh, hd, hd))
        out[f"gated_linear_attention_decode_b{batch}"] = bytes_rec(us, batch * gh * hd * hd * 4 * 2)
        a = torch.randn(batch, width, device=dev).to(bf)
        us = timed(lambda: moe.forward(Ctx(), a))
        experts_read = min(32, batch * 4) + 1              # at most: every pair another expert, and the shared one
        out[f"routed_feed_forward_decode_b{batch}"] = bytes_rec(us, experts_read * 3 * eff * width * 2)
        us = timed(lambda: dense.forward(None, a))
        out[f"qwen3_feed_forward_decode_b{batch}"] = bytes_rec(us, 3 * ff_qwen * width * 2)
        del cache, q, o, x, z, lo, a
    torch.cuda.empty_cache()
    return out


PIBULIX_WINDOW = 1024
VENIDRA_WINDOW = 1024
VENIDRA_CHUNK = 2048


def venidra_config(width, heads, kv_heads, ff_qwen, layers, vocab):
    """A Venidra model of Qwen3's width, head counts, head size 128, layer count and feed-forward size: attention layers
    (half the head rotated, unit RMS of q and k, chunks of 2,048, values blended with the first layer's) in turn with
    layers of attention through latents (a query latent of 0.3 of the width, a key/value latent of 512 and a shared rotated
    key part of 64, as published models of that kind have them, plain key and value heads of 128, a window of 1,024)."""
    hd = 128
    att = {"type": "attention",
           "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "v_mix": True,
                     "rot": {"dims": hd // 2, "base": 1e6}, "mask": {"size": VENIDRA_CHUNK}},
           "mlp": {"kind": "dense", "ff": ff_qwen}}
    lat = {"type": "latent_attention",
           "mixer": {"heads": heads, "dim": hd, "rot_dim": 64, "vdim": hd, "q_rank": width * 3 // 10 // 64 * 64, "kv_rank": 512,
                     "scale": (hd + 64) ** -0.5, "rot": {"base": 1e4, "dims": 64}, "mask": {"size": VENIDRA_WINDOW}},
           "mlp": {"kind": "dense", "ff": ff_qwen}}
    return dict(architecture="Venidra", vocab=vocab, width=width, norm={"eps": 1e-6}, embedding={"scale": 1.0}, logit_scale=1.0,
                logit_softcap=30.0, layers=[att if i % 2 == 0 else lat for i in range(layers)])


def venidra_kernel_times(torch, dk, pk, cfg_d, heads, kv_heads):
    """The design's own mixer steps alone (the parts of a model of ``cfg_d``, so each step runs whichever kernel the part
    picks), beside Qwen3's attention kernels at the same head counts: CUDA events around one step, L2 flushed before
    each (a 256 MB write), median of 5 after 2 untimed."""
    from dryft_challenge_htn_2026_b200.cache import Cache, KVRequest
    from dryft_challenge_htn_2026_b200.csrc import api
    from dryft_challenge_htn_2026_b200.engine.batch import build_context
    from dryft_challenge_htn_2026_b200.parts import Runtime, build_part
    from dryft_challenge_htn_2026_b200.parts.attention import QueryTiles
    dev, bf = torch.device("cuda"), torch.bfloat16
    hd = 128
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)

    def timed(fn):
        ts = []
        for i in range(7):
            flush.fill_(float(i))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts[2:]) * 1e3        # microseconds

    def flops_rec(us, flops):
        return {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1), "frac_bf16": round(flops / us / 1e6 / pk["bf16_tflops"], 4)}

    def bytes_rec(us, moved):
        return {"us": round(us, 1), "gbs": round(moved / us / 1e3, 1), "frac_hbm": round(moved / us / 1e3 / pk["hbm_gbs"], 4)}

    spec = dk.config_from_dict(cfg_d).to_spec()
    rt = Runtime(dev, bf)
    g = torch.Generator(device=dev).manual_seed(1)
    att, lat = build_part(spec.layers[0].mixer, rt), build_part(spec.layers[1].mixer, rt)
    for part in (att, lat):
        part.bind({d.name: (torch.rand(d.shape, generator=g, device=dev) * 0.5 if d.init == "fraction" else
                            torch.randn(d.shape, generator=g, device=dev) * 0.02 + (1.0 if d.init == "norm" else 0.0)).to(
            torch.float32 if d.keep_float32 else bf) for d in part.param_decls()})
        part.prepare(16384)
    ls = lat.spec
    H, L, R, D, Dv, Qr = ls.num_heads, ls.kv_rank, ls.rot_dim, ls.head_dim, ls.v_head_dim, ls.q_rank
    chunk, window = att.spec.chunk, ls.window
    out = {}

    def fill(cache, n):
        for e in range(n):
            v = cache.views(e)[0]
            v.k.normal_()
            if v.v is not None:
                v.v.normal_()

    def steps(ctx, cache, rows, tag, keys_att, keys_lat, pairs_att, pairs_lat, pairs_full):
        """One record per step of the two mixers; ``pairs_*``: (query, key) pairs in sight, ``keys_*``: keys a row reads."""
        a_views, l_views, f = cache.views(0), cache.views(1), cache.views(2)[0]
        proj = torch.randn(rows, att.n_in, device=dev).to(bf)
        ctx.carry = {("value_mix", att.n_v): torch.randn(rows, att.n_v, device=dev).to(bf)}
        mid = torch.empty(rows, att.n_mid, dtype=bf, device=dev)
        prepared = att.prepared_rows(ctx, a_views, proj)
        us = timed(lambda: att.prepared_rows(ctx, a_views, proj))
        out[f"rotation_unit_rms_blend_cache_write_{tag}"] = bytes_rec(us, rows * (2 * att.n_qkv + att.n_k + 2 * att.n_v) * 2)
        q, k, v = prepared[:, :att.n_q], prepared[:, att.n_q:att.n_q + att.n_k], prepared[:, att.n_q + att.n_k:]
        us = timed(lambda: att.attend(ctx, a_views[0], q, k, v, None, mid, 1.0, writes=False))
        out[f"chunk_attention_{tag}"] = flops_rec(us, 4 * heads * hd * pairs_att) if pairs_att else \
            dict(bytes_rec(us, rows * kv_heads * keys_att * 2 * hd * 2), keys=keys_att)
        down = torch.randn(rows, lat.n_down, device=dev).to(bf)
        cq = torch.empty(rows, Qr, dtype=bf, device=dev)
        cos, sin, rot = lat._tables(ctx)
        table = ctx.tables[l_views[0].group]
        us = timed(lambda: api.latent_norm_rope_write(down, cq, lat.q_norm_w, lat.kv_norm_w, ls.norm_eps, cos, sin, rot, ctx.row_pos,
                                                      ctx.row_seq, Qr, L, R, l_views[0].k, l_views[0].v, table))
        out[f"latent_norms_rotation_cache_write_{tag}"] = bytes_rec(us, rows * (lat.n_down + Qr + L + R) * 2)
        qu = torch.randn(rows, lat.n_q, device=dev).to(bf)
        ql = lat.queries(ctx, qu)
        us = timed(lambda: lat.queries(ctx, qu))
        out[f"latent_query_heads_{tag}"] = flops_rec(us, 2 * rows * H * D * L) if pairs_lat else \
            bytes_rec(us, H * D * L * 2 + rows * (lat.n_q + H * lat.lat) * 2)
        o_lat = torch.empty(rows, H * L, dtype=bf, device=dev)
        us = timed(lambda: lat.core.attend(ctx, l_views[0], ql, None, None, None, o_lat, 1.0, writes=False))
        out[f"latent_attention_{tag}"] = flops_rec(us, 2 * H * (lat.lat + L) * pairs_lat) if pairs_lat else \
            dict(bytes_rec(us, rows * keys_lat * lat.lat * 2), keys=keys_lat)
        us = timed(lambda: lat.values(o_lat))
        out[f"latent_value_heads_{tag}"] = flops_rec(us, 2 * rows * H * Dv * L) if pairs_lat else \
            bytes_rec(us, H * Dv * L * 2 + rows * (H * L + lat.n_mid) * 2)
        return f

    for tokens in (2048, 8192):
        plans = att.step_plans() + lat.step_plans() + [QueryTiles(api.TC_TILE_ROWS)]
        cache = Cache([att.cache_requests(), lat.cache_requests(), [KVRequest(kv_heads, hd, None, bf)]], tokens + 64, 2, dev)
        slot = cache.begin()
        ctx = build_context(cache, [(slot, [0] * tokens, [])], dev, plans=plans)
        fill(cache, 3)
        pairs_att = sum(i % chunk + 1 for i in range(tokens))
        pairs_lat = sum(min(i + 1, window) for i in range(tokens))
        full = tokens * (tokens + 1) // 2
        f = steps(ctx, cache, tokens, str(tokens), None, None, pairs_att, pairs_lat, full)
        q = torch.randn(tokens, heads * hd, device=dev).to(bf)
        o = torch.empty_like(q)
        us = timed(lambda: api.attention_prefill_tc(q, o, f.k, f.v, ctx.plans[plans[-1].key], ctx.cu_q, ctx.seq_pos0, ctx.tables[f.group],
                                                    heads, kv_heads, hd, None, hd ** -0.5))
        out[f"qwen3_attention_prefill_{tokens}"] = flops_rec(us, 4 * heads * hd * full)
        cache.end(slot)
        del cache, q, o
    for batch in (8, 64):
        context = 3000       # 952 keys of the newest chunk and the window's 1,024 in sight
        cache = Cache([att.cache_requests(), lat.cache_requests(), [KVRequest(kv_heads, hd, None, bf)]], batch * (context + 64), batch, dev)
        slots = [cache.begin() for _ in range(batch)]
        for sl in slots:
            cache.reserve(sl, context + 1)
            cache.length[sl] = context
        ctx = build_context(cache, [(sl, [0], []) for sl in slots], dev, plans=att.step_plans() + lat.step_plans())
        fill(cache, 3)
        f = steps(ctx, cache, batch, f"decode_b{batch}", context % chunk + 1, min(window, context + 1), 0, 0, 0)
        q = torch.randn(batch, heads * hd, device=dev).to(bf)
        o = torch.empty_like(q)
        nsplit = api.decode_splits(batch, kv_heads, heads // kv_heads, ctx.tables[f.group].shape[1])
        ws = api.attention_decode_ws(batch, heads, hd, nsplit, dev)
        us = timed(lambda: api.attention_decode_bf16(q, o, f.k, f.v, ctx.row_pos, ctx.tables[f.group], heads, kv_heads, hd, None,
                                                     hd ** -0.5, nsplit, *ws))
        out[f"qwen3_attention_decode_b{batch}"] = dict(bytes_rec(us, batch * kv_heads * (context + 1) * 2 * hd * 2), keys=context + 1)
        del cache, q, o
    torch.cuda.empty_cache()
    return out


NEVOTAR_WINDOW = 1024


def nevotar_config(width, heads, kv_heads, ff_qwen, layers, vocab):
    """A Nevotar model of Qwen3's width, layer count and feed-forward arithmetic: differential attention of half Qwen3's
    head counts (two maps of 64 side by side, values of 128, a temperature every 128 positions), an HGRN2 layer of as many
    heads of 128, and layers that run attention with mixed head scores (heads of 128, half the head rotated, a window of
    1,024) beside a state-space mixer as wide as the model (heads of 128, states of 128, 4 groups, 4 taps); every layer
    with a mixture of 32 clamped experts of which a token uses 4, each a quarter of Qwen3's feed-forward, and a shared one."""
    h2, g2 = heads // 2, max(1, kv_heads // 2)
    eff = max(64, ff_qwen // 4 // 64 * 64)
    mlp = {"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "router": {"experts": 32, "top": 4}, "shared": {"ff": eff, "limit": 7.0}}
    att = {"type": "attention", "mixer": {"heads": h2, "kv_heads": g2, "dim": 64, "vdim": 128, "scale": 0.125, "diff": 0.5,
                                          "q_temp": {"coef": 0.25, "every": 128}}, "mlp": mlp}
    hg = {"type": "hgrn2", "mixer": {"heads": h2, "dim": 128, "vdim": 128}, "mlp": mlp}
    par = {"type": "parallel",
           "mixer": {"left": {"heads": h2, "kv_heads": g2, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "rot": {"dims": 64, "base": 5e5},
                              "mask": {"size": NEVOTAR_WINDOW}},
                     "right": {"heads": width // 128, "vdim": 128, "state": 128, "groups": 4, "conv": 4, "norm_groups": 4},
                     "left_scale": 0.7, "right_scale": 0.8}, "mlp": mlp}
    return dict(architecture="Nevotar", vocab=vocab, width=width, norm={"eps": 1e-6, "groups": 2},
                layers=[(att, hg, par, par)[i % 4] for i in range(layers)])


def nevotar_kernel_times(torch, dk, pk, cfg_d, p_cfg):
    """The design's mixer and feed-forward steps alone (the parts of a model of ``cfg_d``, so each step runs whichever kernel
    the part picks), beside the like steps of the Pibulix model ``p_cfg`` of the same width: CUDA events around one step, L2
    flushed before each (a 256 MB write), median of 5 after 2 untimed."""
    from dryft_challenge_htn_2026_b200.cache import Cache
    from dryft_challenge_htn_2026_b200.engine.batch import build_context
    from dryft_challenge_htn_2026_b200.parts import Runtime, build_part
    dev, bf = torch.device("cuda"), torch.bfloat16
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)

    def timed(fn):
        ts = []
        for i in range(7):
            flush.fill_(float(i))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts[2:]) * 1e3        # microseconds

    def flops_rec(us, flops):
        return {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1), "frac_bf16": round(flops / us / 1e6 / pk["bf16_tflops"], 4)}

    def bytes_rec(us, moved):
        return {"us": round(us, 1), "gbs": round(moved / us / 1e3, 1), "frac_hbm": round(moved / us / 1e3 / pk["hbm_gbs"], 4)}

    rt = Runtime(dev, bf)
    g = torch.Generator(device=dev).manual_seed(1)
    spec, pspec = dk.config_from_dict(cfg_d).to_spec(), dk.config_from_dict(p_cfg).to_spec()
    W = spec.hidden_size

    def bound(part_spec):
        part = build_part(part_spec, rt)
        part.bind({d.name: (torch.rand(d.shape, generator=g, device=dev) * 0.5 if d.init == "fraction" else
                            torch.eye(d.shape[-1], device=dev) + 0.1 * torch.randn(d.shape, generator=g, device=dev) if d.init == "near_identity" else
                            torch.randn(d.shape, generator=g, device=dev) * (0.2 if d.init == "wide" else 0.02) + (1.0 if d.init == "norm" else 0.0)).to(
            torch.float32 if d.keep_float32 else bf) for d in part.param_decls()})
        part.prepare(16384)
        return part

    diff, hg, par = bound(spec.layers[0].mixer), bound(spec.layers[1].mixer), bound(spec.layers[2].mixer)
    talk, ssd = par.branches[0][1], par.branches[1][1]
    moe, norm = bound(spec.layers[0].feed_forward), bound(spec.layers[0].norm_in)
    p_att, p_gla = bound(pspec.layers[0].mixer), bound(pspec.layers[1].mixer)
    p_moe, p_norm = bound(pspec.layers[1].feed_forward), bound(pspec.layers[0].norm_mix)
    ds, ts_, ss, hs, ps = diff.spec, talk.spec, ssd.spec, hg.spec, p_att.spec
    window = ts_.window
    out = {}
    scratch = {}

    class Ctx:
        def scratch(self, key, make):
            if key not in scratch:
                scratch[key] = make()
            return scratch[key]

    def fill(cache, n):
        for e in range(n):
            for v in cache.views(e):
                if hasattr(v, "k"):
                    v.k.normal_()
                    if v.v is not None:
                        v.v.normal_()

    def steps(ctx, cache, rows, tag, pairs_full, pairs_win, keys_full, keys_win, keys_p):
        """One record per step; ``pairs_*``: (query, key) pairs in sight in a prompt, ``keys_*``: keys a single token reads."""
        mids = {n: torch.empty(rows, part.n_mid, dtype=bf, device=dev) for n, part in (("d", diff), ("t", talk), ("s", ssd), ("h", hg), ("pa", p_att), ("pg", p_gla))}
        projs = {n: (torch.randn(rows, part.n_in, device=dev) * 0.5).to(bf) for n, part in (("d", diff), ("t", talk), ("s", ssd), ("h", hg), ("pa", p_att), ("pg", p_gla))}
        ctx.carry = {}
        H, D, V = ds.num_heads, ds.head_dim, ds.v_head_dim
        us = timed(lambda: diff.mix(ctx, cache.views(0), projs["d"], mids["d"], 1.0))
        out[f"differential_attention_{tag}"] = flops_rec(us, 4 * H * (D + V) * pairs_full) if pairs_full else \
            dict(bytes_rec(us, rows * ds.num_kv_heads * keys_full * (2 * D + V) * 2), keys=keys_full)
        H, D, V = ts_.num_heads, ts_.head_dim, ts_.v_head_dim
        us = timed(lambda: talk.mix(ctx, cache.views(1)[:1], projs["t"], mids["t"], 1.0))
        out[f"mixed_scores_attention_{tag}"] = flops_rec(us, 2 * H * (D + V) * pairs_win) if pairs_win else \
            dict(bytes_rec(us, rows * ts_.num_kv_heads * keys_win * (D + V) * 2), keys=keys_win)
        us = timed(lambda: p_att.mix(ctx, cache.views(3), projs["pa"], mids["pa"], 1.0))
        out[f"pibulix_window_attention_{tag}"] = flops_rec(us, 4 * ps.num_heads * ps.head_dim * pairs_win) if pairs_win else \
            dict(bytes_rec(us, rows * ps.num_kv_heads * keys_p * 2 * ps.head_dim * 2), keys=keys_p)
        # the recurrences: what a prompt must move (operands in float32 in, outputs out), what a single token must (the state, twice)
        us = timed(lambda: hg.mix(ctx, cache.views(2), projs["h"], mids["h"], 1.0))
        out[f"lower_bound_recurrence_{tag}"] = bytes_rec(us, rows * hs.num_heads * (3 * hs.head_dim + 2 * hs.v_head_dim) * 4 if pairs_full else
                                                         rows * hs.num_heads * hs.head_dim * hs.v_head_dim * 4 * 2)
        us = timed(lambda: ssd.mix(ctx, cache.views(1)[1:], projs["s"], mids["s"], 1.0))
        out[f"state_space_mixer_{tag}"] = bytes_rec(us, rows * (ss.num_heads * 2 * ss.v_head_dim + 2 * ss.groups * ss.state_dim) * 4 if pairs_full else
                                                    rows * ss.num_heads * ss.state_dim * ss.v_head_dim * 4 * 2)
        gs = p_gla.spec
        us = timed(lambda: p_gla.mix(ctx, cache.views(4), projs["pg"], mids["pg"], 1.0))
        out[f"pibulix_gated_linear_attention_{tag}"] = bytes_rec(us, rows * gs.num_heads * (3 * gs.head_dim + 2 * gs.v_head_dim) * 4 if pairs_full else
                                                                 rows * gs.num_heads * gs.head_dim * gs.v_head_dim * 4 * 2)
        a = torch.randn(rows, W, device=dev).to(bf)
        ms, pm = moe.spec, p_moe.spec
        us = timed(lambda: moe.forward(Ctx(), a))
        pairs = rows * (ms.top + 1)
        read = (min(ms.num_experts, rows * ms.top) + 1) * 3 * ms.expert_ff * W * 2
        out[f"clamped_experts_{tag}"] = flops_rec(us, pairs * 6 * ms.expert_ff * W) if pairs_full else bytes_rec(us, read)
        us = timed(lambda: p_moe.forward(Ctx(), a))
        read = (min(pm.num_experts, rows * pm.top) + 1) * 3 * pm.expert_ff * W * 2
        out[f"pibulix_experts_{tag}"] = flops_rec(us, rows * (pm.top + 1) * 6 * pm.expert_ff * W) if pairs_full else bytes_rec(us, read)
        h = torch.randn(rows, W, device=dev)
        o = torch.empty(rows, W, dtype=bf, device=dev)
        us = timed(lambda: norm.add_forward(h, a, o))
        out[f"norm_in_groups_{tag}"] = bytes_rec(us, rows * W * (4 + 4 + 2 + 2))
        us = timed(lambda: p_norm.scale_add_forward(h, 1.0, a, o))
        out[f"pibulix_norm_{tag}"] = bytes_rec(us, rows * W * (4 + 4 + 2 + 2))

    entries = [diff.cache_requests(), par.cache_requests(), hg.cache_requests(), p_att.cache_requests(), p_gla.cache_requests()]
    plans = list({p.key: p for part in (diff, par, p_att) for p in part.step_plans()}.values())
    for tokens in (2048, 8192):
        cache = Cache(entries, tokens + 64, 2, dev)
        slot = cache.begin()
        ctx = build_context(cache, [(slot, [0] * tokens, [])], dev, plans=plans)
        fill(cache, 5)
        steps(ctx, cache, tokens, str(tokens), tokens * (tokens + 1) // 2, sum(min(i + 1, window) for i in range(tokens)), 0, 0, 0)
        cache.end(slot)
        del cache
    for batch in (8, 64):
        context = 3000
        cache = Cache(entries, batch * (context + 64), batch, dev)
        slots = [cache.begin() for _ in range(batch)]
        for sl in slots:
            cache.reserve(sl, context + 1)
            cache.length[sl] = context
        ctx = build_context(cache, [(sl, [0], []) for sl in slots], dev, plans=plans)
        fill(cache, 5)
        steps(ctx, cache, batch, f"decode_b{batch}", 0, 0, context + 1, min(window, context + 1), min(ps.window, context + 1) + ps.keep_first)
        del cache
    torch.cuda.empty_cache()
    return out


def run_design(args):
    """``--design nilivik`` / ``--design pibulix`` / ``--design venidra`` / ``--design nevotar``: prefill and decode of that decoder at Qwen3 layer sizes (random weights,
    ``--layers`` layers, default 4) beside Qwen3 itself at the same width, layer count and parameters a
    layer, and the design's mixer kernels alone beside Qwen3's attention kernels. One JSON line."""
    import torch

    import dryft_challenge_htn_2026_b200 as dk
    from dryft_challenge_htn_2026_b200.csrc import api

    api.set_pdl(bool(args.pdl))
    pk = peaks()
    layers = args.layers or 4
    chunk = 2048
    vocab = 32768
    out = {"design": args.design, "beside": "Pibulix" if args.design == "nevotar" else "Qwen3ForCausalLM", "layers": layers, "chunk": chunk, "vocab": vocab, "dtype": "bf16",
           "data": "synthetic: random weights, uniform random token ids", "peaks": pk, "sizes": {}}
    for size in args.design_sizes.split(","):
        q = dict(SIZES[size]["config"], num_hidden_layers=layers, vocab_size=vocab, tie_word_embeddings=True)
        beside = ("qwen3", q)
        if args.design == "nevotar":
            n = nevotar_config(q["hidden_size"], q["num_attention_heads"], q["num_key_value_heads"], q["intermediate_size"], layers, vocab)
            beside = ("pibulix", pibulix_config(q["hidden_size"], q["num_attention_heads"], q["num_key_value_heads"], q["intermediate_size"],
                                                layers, vocab, PIBULIX_WINDOW))
            rec = {"width": q["hidden_size"], "window": NEVOTAR_WINDOW, "expert_ff": n["layers"][0]["mlp"]["expert"]["ff"],
                   "beside": "Pibulix of the same width, layer count and feed-forward arithmetic (the closest of the library's designs)"}
        elif args.design == "venidra":
            n = venidra_config(q["hidden_size"], q["num_attention_heads"], q["num_key_value_heads"], q["intermediate_size"], layers, vocab)
            rec = {"width": q["hidden_size"], "chunk": VENIDRA_CHUNK, "window": VENIDRA_WINDOW, "q_rank": n["layers"][1]["mixer"]["q_rank"],
                   "kv_rank": 512, "rot_dim": 64}
        elif args.design == "pibulix":
            n = pibulix_config(q["hidden_size"], q["num_attention_heads"], q["num_key_value_heads"], q["intermediate_size"], layers,
                               vocab, PIBULIX_WINDOW)
            rec = {"width": q["hidden_size"], "window": PIBULIX_WINDOW, "expert_ff": n["layers"][1]["mlp"]["expert"]["ff"]}
        else:
            n = nilivik_config(q["hidden_size"], q["num_attention_heads"], q["num_key_value_heads"], q["intermediate_size"], layers,
                               vocab, chunk)
            rec = {"width": q["hidden_size"], "nilivik_ff": n["layers"][0]["mlp"]["ff"]}
        for name, cfg_d in ((args.design, n), beside):
            model = dk.random_model(dk.config_from_dict(cfg_d), seed=0, dtype=torch.bfloat16)
            r = {"weight_mb_per_step": round(model.weight_bytes_per_step() / 1e6, 1), "prefill": {}, "decode": {}}
            for tokens in (2048, 8192):
                ms = time_step_prefill(torch, dk, model, tokens)
                r["prefill"][str(tokens)] = {"ms": round(ms, 3), "tok_s": round(tokens / ms * 1e3)}
            for batch in (1, 8, 64):
                # 3,072 tokens of context: in the middle of a chunk of 2,048 for the chunked design (half a chunk of keys in sight)
                ms, launches = time_step_decode(torch, dk, model, batch, 3072, max(16, args.steps // 2), 24)
                r["decode"][f"b{batch}"] = {"ms": round(ms, 4), "tok_s": round(batch / ms * 1e3, 1), "kernels_per_step": launches,
                                            "weights_frac_hbm": round(model.weight_bytes_per_step() / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}
            rec[name] = r
            del model
            torch.cuda.empty_cache()
        if args.design == "nevotar":
            rec["kernels"] = nevotar_kernel_times(torch, dk, pk, n, beside[1])
        elif args.design == "venidra":
            rec["kernels"] = venidra_kernel_times(torch, dk, pk, n, q["num_attention_heads"], q["num_key_value_heads"])
        elif args.design == "pibulix":
            rec["kernels"] = pibulix_kernel_times(torch, dk, pk, q["hidden_size"], q["num_attention_heads"], q["num_key_value_heads"],
                                                  q["intermediate_size"], PIBULIX_WINDOW)
        else:
            rec["kernels"] = kernel_times(torch, dk, pk, q["num_attention_heads"], q["num_key_value_heads"],
                                          q["num_attention_heads"] // 2, chunk)
        out["sizes"][size] = rec
    api.gemm_tc_check()
    print(json.dumps(out))
    return 0


# ------------------------------------------------------------------------------ the reference arm
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
# The reference's own switches (engine/engine.py:31,98; engine/fused.py:19), set in the environment before it
# is imported. Speculative decoding and fp8 prefill products are not part of the metric (plain bf16 decoding).
# ENGINE_PDL=0: the reference patches the C launcher that Triton 3.1 generates; with the Triton of this image
# the patched text is not found, every fused kernel then fails to compile (AssertionError) and its self-test
# falls back to its torch ops, 5 times slower. Without the patch its fused Triton ops pass their self-test.
REF_ENV = {"ENGINE_SPEC": "0", "ENGINE_FP8": "0", "ENGINE_PDL": "0"}


def reference_source():
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            return json.load(f).get("reference_path") or ""
    except Exception:
        return ""


def install_reference():
    """baseline/_ref: an unmodified copy of the reference's folder (it has no setup.py or pyproject.toml
    for pip to install). Returns None, or the reason it is not there."""
    if os.path.isfile(os.path.join(REF_DIR, "engine", "engine.py")):
        return None
    src = os.environ.get("DRYFT_REFERENCE") or reference_source()
    if not src or not os.path.isfile(os.path.join(src, "engine", "engine.py")):
        return f"no copy of the reference under baseline/_ref and no source folder to copy it from ({src or 'none named'})"
    os.makedirs(os.path.dirname(REF_DIR), exist_ok=True)
    shutil.copytree(src, REF_DIR, ignore=shutil.ignore_patterns(".git", "__pycache__"))
    return None


def write_model_folder(torch, cfg, folder, seed=0, dev="cuda"):
    """config.json (rope_theta at the top level, as the reference reads it) and one safetensors file per
    layer with the checkpoint names of Qwen3ForCausalLM; matrices N(0, 0.02), norm weights 1 + N(0, 0.1)."""
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(cfg, model_type="qwen3", hidden_act="silu", attention_bias=False), f)
    gen = torch.Generator(device=dev).manual_seed(seed)
    H, hd, I, V = cfg["hidden_size"], cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    mat = lambda *s: (0.02 * torch.randn(s, generator=gen, device=dev, dtype=torch.float32)).to(torch.bfloat16).cpu()
    nrm = lambda n: (1.0 + 0.1 * torch.randn(n, generator=gen, device=dev, dtype=torch.float32)).to(torch.bfloat16).cpu()
    top = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": nrm(H)}
    if not cfg["tie_word_embeddings"]:
        top["lm_head.weight"] = mat(V, H)
    save_file(top, os.path.join(folder, "model-top.safetensors"))
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        save_file({p + "input_layernorm.weight": nrm(H), p + "post_attention_layernorm.weight": nrm(H),
                   p + "self_attn.q_norm.weight": nrm(hd), p + "self_attn.k_norm.weight": nrm(hd),
                   p + "self_attn.q_proj.weight": mat(nh * hd, H), p + "self_attn.k_proj.weight": mat(nkv * hd, H),
                   p + "self_attn.v_proj.weight": mat(nkv * hd, H), p + "self_attn.o_proj.weight": mat(H, nh * hd),
                   p + "mlp.gate_proj.weight": mat(I, H), p + "mlp.up_proj.weight": mat(I, H),
                   p + "mlp.down_proj.weight": mat(H, I)}, os.path.join(folder, f"model-layer{i:03d}.safetensors"))


def ref_decode(torch, eng, prompts, steps, warmup, sample_clocks=False):
    """Decode steps of the reference's generator, as its tests/bench.py:104-111 times a run: wall clock at
    each yield; the timed steps are those between yield number ``warmup`` and yield ``warmup + steps``."""
    stamps = []
    gen = eng.generate(prompts, warmup + steps + 1)
    cs = ClockSampler() if sample_clocks else contextlib.nullcontext()
    with cs:
        for _ in gen:
            stamps.append(time.perf_counter())
    assert len(stamps) == warmup + steps + 1
    ms = (stamps[warmup + steps] - stamps[warmup]) / steps * 1e3
    return ms, (cs.summary() if sample_clocks else None)


def run_reference(args):
    why = install_reference()
    if why:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    os.environ.update({k: os.environ.get(k, v) for k, v in REF_ENV.items()})
    real_stdout = sys.stdout
    sys.stdout = sys.stderr                       # the reference prints its self-test results; the JSON line stays alone
    try:
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        sys.path.insert(0, os.path.join(REF_DIR, "engine"))
        from engine import Engine                 # the reference's engine/engine.py, unmodified

        size = args.size
        w = SIZES[size]
        cfg = dict(w["config"])
        full_layers = cfg["num_hidden_layers"]
        if args.layers:
            cfg["num_hidden_layers"] = args.layers
        pk = peaks()
        warmup = max(3, args.warmup)
        untimed = max(warmup, MIN_UNTIMED_STEPS)
        folder = tempfile.mkdtemp(prefix="dryft_ref_model_")
        try:
            t0 = time.time()
            write_model_folder(torch, cfg, folder)
            print(f"[bench] model folder written in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
            t0 = time.time()
            eng = Engine(folder)                  # loads, self-tests its fused ops against its torch ops, picks a back end
            print(f"[bench] reference engine ready in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
        finally:
            shutil.rmtree(folder, ignore_errors=True)
        backend = type(eng.ops).__name__
        import fused
        backend += f" (PDL {'on' if getattr(fused, 'PDL', False) else 'off'})"
        V = cfg["vocab_size"]

        def decode_point(batch, equal, steps, seed, clocks=False):
            lens = prompt_lengths(size, batch, seed)
            if equal:
                lens = [max(lens)] * batch
            ms, c = ref_decode(torch, eng, random_prompts(V, lens, seed), steps, untimed, clocks)
            ctx_mean = sum(lens) / batch + untimed + steps / 2
            nbytes = weight_bytes(cfg) + batch * ctx_mean * kv_bytes_per_token(cfg)
            return dict(ms=ms, tok_s=batch / ms * 1e3, bytes=nbytes, ctx_mean=ctx_mean, clocks=c)

        decode_point(args.batch, False, 4, seed=0)                      # compiles what this shape needs
        main_run = decode_point(args.batch, False, args.steps, seed=0, clocks=True)
        points, detail, prefill = {}, {}, None
        if not args.no_points:
            psteps = max(16, min(64, args.steps))
            if w["ragged"] and args.batch > 1:
                # the reference runs a ragged batch as one stream per prompt length (engine/engine.py:1093-1105);
                # with equal lengths the same batch is one stream
                detail[f"decode_b{args.batch}_equal_lengths"] = point(decode_point(args.batch, True, psteps, seed=0, clocks=True), pk)
            for b in w["batches"]:
                if b != args.batch:
                    equal = b > 8                  # 64 streams of one sequence each would only measure batch 1 again
                    key = f"decode_b{b}" + ("_equal_lengths" if equal and w["ragged"] else "")
                    detail[key] = point(decode_point(b, equal, psteps, seed=b, clocks=True), pk)
            points = {k: v["value"] for k, v in detail.items()}
            prompt = random_prompts(V, [PREFILL_TOKENS], 6)
            times = []
            for i in range(4):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in eng.generate(prompt, 1):
                    pass
                torch.cuda.synchronize()
                if i:
                    times.append((time.perf_counter() - t0) * 1e3)
            ms = statistics.median(times)
            prefill = {"value": round(PREFILL_TOKENS / ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
                       "frac": round(prefill_flops(cfg, PREFILL_TOKENS) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                       "how": "wall clock of generate(prompt, 1), the reference's TTFT"}
        achieved = main_run["bytes"] / (main_run["ms"] * 1e-3) / 1e9
        lens = prompt_lengths(size, args.batch, 0)
        out = {
            "impl": "reference",
            "metric": f"decode tok/s at batch {args.batch} ({w['name']}, bf16)", "value": round(main_run["tok_s"], 1),
            "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(main_run["ms"], 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: random weights N(0,0.02), uniform random token ids",
            "config": config_record(size, cfg, full_layers, args.batch, pk, ctx_mean_timed=round(main_run["ctx_mean"]),
                                    reference_backend=f"{backend}, {len(set(lens))} streams",
                                    reference_env=" ".join(f"{k}={os.environ[k]}" for k in sorted(REF_ENV)),
                                    untimed_steps=untimed),
            "clocks": main_run["clocks"],
            # the reference's only interface is the host-side generator: host token lists in, host tokens out;
            # value and e2e are the same measurement (wall clock between yields)
            "e2e": {"value": round(main_run["tok_s"], 1), "unit": "tok/s",
                    "h2d_bytes_per_step": round(sum(lens) * 8 / (untimed + args.steps + 1)), "d2h_bytes_per_step": 8 * args.batch},
            "gpu_launches": None,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4)},
        }
        if prefill is not None:
            out["prefill"] = prefill
            out["points"] = points
            out["points_detail"] = detail
    except Exception as e:                         # the arm reports, it does not fail the round
        import traceback
        traceback.print_exc(file=sys.stderr)
        out = {"impl": "reference", "unavailable": f"the reference engine did not run here: {type(e).__name__}: {str(e)[:300]}"}
    finally:
        sys.stdout = real_stdout
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=48,
                    help="untimed steps before the timed ones; the default outlasts the tens of milliseconds the SM clock "
                         "takes to come back after the power-capped prefill")
    ap.add_argument("--size", default="4b", choices=sorted(SIZES), help="layer sizes and workload (default: Qwen3-4B)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the other batch sizes and the prefill")
    ap.add_argument("--prefill-only", action="store_true", help="only the 2,048-token prefill (for profiling its kernels)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="with --prefill-only: a prompt of another length")
    ap.add_argument("--pdl", type=int, default=1, help="programmatic dependent launch on (1) or off (0)")
    ap.add_argument("--design", default=None, choices=["nilivik", "pibulix", "venidra", "nevotar"],
                    help="instead of the default workload: prefill and decode of this design at Qwen3 layer sizes beside Qwen3 "
                         "itself at equal size (nevotar: beside Pibulix, the closest of the library's designs), and its mixer "
                         "kernels alone (one JSON line of its own)")
    ap.add_argument("--design-sizes", default="4b,8b", help="with --design: which of the layer sizes")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this library runs one model on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    if args.design:
        return run_design(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
