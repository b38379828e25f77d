#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-0.5B sizes with random
weights on one B200.  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]
                    [--config 0.5b|1.5b-mixed|7b|pufuzen|katopel|vizonex|zobelorn]

A "step" is one decode step of the whole batch.  `value` is decoded tokens a
second timed on the device over K steps that never return to the host
(`Engine.decode_steps`); `e2e` is the same through the scheduler that the Python
entry point (`generate_batch`) runs: prompts come from the host, every step's
positions, slots and block tables are copied from pinned host memory and its
sampled ids are read back by the host, which judges the ends one step behind.  The line also carries the prefill of 2,048 tokens, the decode
roofline and decode at batch 1 and 64.

`--config 7b` prints the same line at Qwen2.5-7B sizes (prefill of 2,048 tokens, decoding at batch
1/8/64 with 8,192-token contexts); `--config 1.5b-mixed` runs 32 requests of random prompt lengths
in [64, 2048] with 128 new tokens each through the scheduler under a budget of 512 tokens a step,
half of them beginning with one of four shared 256-token beginnings, at Qwen2.5-1.5B sizes.  Both
first compare a few logits rows of a 2-layer model of the same layer sizes with the plain
implementation under tests/, and refuse to time an engine that fails that.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: Qwen2.5-0.5B sizes
SIZES = dict(num_hidden_layers=24, hidden_size=896, num_attention_heads=14, num_key_value_heads=2,
             head_dim=64, intermediate_size=4864, vocab_size=151936, rope_theta=1000000.0,
             rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=32768,
             use_sliding_window=False, sliding_window=32768, max_window_layers=24)
# BASELINE.json configs[3] and configs[4]: Qwen2.5-1.5B and Qwen2.5-7B sizes
SIZES_1_5B = dict(num_hidden_layers=28, hidden_size=1536, num_attention_heads=12, num_key_value_heads=2,
                  head_dim=128, intermediate_size=8960, vocab_size=151936, rope_theta=1000000.0,
                  rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=32768,
                  use_sliding_window=False, sliding_window=32768, max_window_layers=28)
SIZES_7B = dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
                head_dim=128, intermediate_size=18944, vocab_size=152064, rope_theta=1000000.0,
                rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=32768,
                use_sliding_window=False, sliding_window=32768, max_window_layers=28)
PROMPT_LEN, NEW_TOKENS, PREFILL_TOKENS, PAGE = 512, 256, 2048, 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            raw = json.load(open(path))
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in raw.items() if k in out and v})
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def weight_bytes(cfg, layers):
    """Bytes of weights one decode step reads: every matrix once (bfloat16),
    gains and biases in float32."""
    h, d = cfg["hidden_size"], cfg["head_dim"]
    q, kv, inner = cfg["num_attention_heads"] * d, cfg["num_key_value_heads"] * d, cfg["intermediate_size"]
    per_layer = 2 * ((q + 2 * kv) * h + h * q + 3 * inner * h) + 4 * ((q + 2 * kv) + 2 * h)
    head = 2 * cfg["vocab_size"] * h
    return layers * per_layer + head + 4 * h


def kv_bytes_per_token(cfg, layers):
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, layers, tokens):
    h, d = cfg["hidden_size"], cfg["head_dim"]
    q, kv, inner = cfg["num_attention_heads"] * d, cfg["num_key_value_heads"] * d, cfg["intermediate_size"]
    linear = 2 * tokens * ((q + 2 * kv) * h + h * q + 3 * inner * h)
    attention = 2 * 2 * cfg["num_attention_heads"] * d * tokens * (tokens + 1) / 2
    return layers * (linear + attention) + 2 * h * cfg["vocab_size"]


def products_note():
    """Where a prompt step's plain matrix products run (the decoding steps that `value` times use
    the framework's own kernels only)."""
    choice = os.environ.get("TOKB200_GEMM", "")
    return "own tcgen05 kernel" if choice == "own" else "vendor library (torch.mm); TOKB200_GEMM=own for the own kernel"


def full_config(sizes, layers=None):
    layers = layers or sizes["num_hidden_layers"]
    return dict(sizes, num_hidden_layers=layers, max_window_layers=layers,
                architectures=["Qwen2ForCausalLM"], hidden_act="silu")


def gate_on_logits(sizes, what):
    """Before a configuration is timed: a 2-layer model of its layer sizes (random weights
    through a model folder) must give, in bfloat16, the plain implementation's logits for a
    prompt step, a portion that continues it and decoding steps of three requests together.
    Returns the largest error as a fraction of the largest logit; raises if it passes 2 %."""
    import torch
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_qwen2 as plain
    config = tb.Qwen2Config.from_dict(dict(full_config(sizes, 2), max_position_embeddings=1024))
    gen = torch.Generator().manual_seed(99)
    ids = torch.randint(0, config.vocab_size, (150,), generator=gen).tolist()
    rows = [16, 63, 99, 139, 140, 141, 142]
    with tempfile.TemporaryDirectory() as folder:
        tb.write_random_model(folder, config, seed=3)
        cfg, w = plain.load_folder(folder)
        want = plain.all_logits(cfg, w, ids[:143], rows=rows)
        del w
        model = tb.load_model(folder, dtype="bfloat16", device="cuda:0")
    at = {r: i for i, r in enumerate(rows)}
    engine = tb.engine_for(model, 3 * 160, PAGE, max_requests=3, share_prefixes=False)
    caches = [engine.cache.open(("gate", i)) for i in range(3)]
    lengths = [140, 100, 17]                         # each a beginning of the same sequence
    worst = 0.0
    scale = float(want.abs().max())

    def check(logits, positions):
        nonlocal worst
        got = logits.float().cpu()
        for row, position in zip(got, positions):
            worst = max(worst, float((row - want[at[position]]).abs().max()) / scale)

    engine.cache.reserve(caches[0], 100)
    check(engine.step([StepEntry(caches[0], ids[:100], [63, 99])]), [63, 99])
    engine.cache.reserve(caches[0], 40)
    for c, n in zip(caches[1:], lengths[1:]):
        engine.cache.reserve(c, n)
    check(engine.step([StepEntry(caches[0], ids[100:140], [39]), StepEntry(caches[1], ids[:100], [99]),
                       StepEntry(caches[2], ids[:17], [16])]), [139, 99, 16])
    for step in range(3):
        engine.cache.reserve(caches[0], 1)
        check(engine.step([StepEntry(caches[0], [ids[140 + step]], [0])]), [140 + step])
    engine.check()
    del engine, model
    torch.cuda.empty_cache()
    if not worst <= 0.02:
        raise SystemExit(f"bench.py: {what}: the engine's logits are off by {worst:.3%} of the largest logit "
                         f"against the plain implementation; nothing is timed")
    return worst


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=SIZES["num_hidden_layers"])
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--config", default="0.5b", choices=["0.5b", "1.5b-mixed", "7b", "pufuzen", "katopel", "vizonex", "zobelorn"],
                        help="0.5b: the headline line; 7b: the same at Qwen2.5-7B sizes with 8,192-token "
                             "contexts; 1.5b-mixed: 32 requests through the scheduler at Qwen2.5-1.5B sizes; "
                             "pufuzen: prefill and decoding of the Pufuzen design at two widths beside Qwen2 at "
                             "equal width, depth and parameters, and its kernels alone; katopel: the same for the Katopel design; "
                             "vizonex: the Vizonex design beside the Katopel design at equal width, depth and parameters; "
                             "zobelorn: the Zobelorn design beside Qwen2 at equal width, depth, heads and parameters")
    parser.add_argument("--context", type=int, default=8192, help="--config 7b: tokens held before decoding")
    parser.add_argument("--layer-phases", action="store_true",
                        help="print where the time of the whole-layer kernel (TOKB200_LAYER=fused) goes, phase by "
                             "phase, from the kernel's own time stamps, beside the time of the four kernels it replaces")
    parser.add_argument("--stream-probe", action="store_true",
                        help="read a 1 GB matrix once in each of the access patterns the decoding kernels choose "
                             "between (plain loads by whole and by half lines, bulk copies of several sizes) and "
                             "print the bytes a second each reaches")
    parser.add_argument("--skip-gate", action="store_true",
                        help="do not compare with the plain implementation first (profiling runs)")
    parser.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    parser.add_argument("--only-decode", action="store_true",
                        help="time the decode steps only and print a short line (for profiling)")
    parser.add_argument("--only-kernels", action="store_true",
                        help="--config katopel, vizonex, zobelorn: the kernels alone, without the models")
    parser.add_argument("--only-prefill", action="store_true",
                        help="time the 2,048-token prefill only and print a short line (for profiling)")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (candle, CPU); no cargo/rustc or maturin "
                          "offline, and its Python package binds only the cl100k tokenizer"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    args.warmup = max(args.warmup, 3)
    if args.layer_phases:
        return run_layer_phases(args)
    if args.stream_probe:
        return run_stream_probe(args)
    if args.config == "7b":
        return run_7b(args)
    if args.config == "1.5b-mixed":
        return run_mixed(args)
    if args.config == "pufuzen":
        return run_pufuzen(args)
    if args.config == "katopel":
        return run_katopel(args)
    if args.config == "vizonex":
        return run_vizonex(args)
    if args.config == "zobelorn":
        return run_zobelorn(args)
    args.steps = max(1, min(args.steps, NEW_TOKENS - args.warmup - 1))

    import torch
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    from tokenizer_b200.kernels.ops import counter

    torch.cuda.set_device(0)
    cfg = dict(SIZES, num_hidden_layers=args.layers, max_window_layers=args.layers,
               architectures=["Qwen2ForCausalLM"], hidden_act="silu")
    config = tb.Qwen2Config.from_dict(cfg)
    pk = peaks()
    gen = torch.Generator().manual_seed(1234)

    def random_prompt(n):
        return torch.randint(0, config.vocab_size, (n,), generator=gen).tolist()

    with tempfile.TemporaryDirectory() as folder:
        tb.write_random_model(folder, config, seed=2)
        model = tb.load_model(folder, dtype="bfloat16", device="cuda:0")
    biggest = max(args.batch, 1 if (args.no_points or args.only_prefill) else 64)
    pool_tokens = max(biggest * (PROMPT_LEN + NEW_TOKENS + PAGE), PREFILL_TOKENS + PAGE)
    engine = tb.engine_for(model, pool_tokens, PAGE, max_requests=max(biggest, 1), share_prefixes=False)

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    # ---- prefill of 2,048 tokens in one step ------------------------------------
    prefill_ms = []
    for rep in range(0 if args.only_decode else 3 + 5):
        cache = engine.cache.open(("prefill", rep))
        engine.cache.reserve(cache, PREFILL_TOKENS)
        entry = StepEntry(cache, random_prompt(PREFILL_TOKENS), [PREFILL_TOKENS - 1])
        torch.cuda.synchronize()
        start, stop = events()
        start.record()
        engine.step([entry])
        stop.record()
        torch.cuda.synchronize()
        if rep >= 3:
            prefill_ms.append(start.elapsed_time(stop))
        engine.cache.close(cache)
    prefill_best = sorted(prefill_ms)[len(prefill_ms) // 2] if prefill_ms else float("nan")
    # a portion of 512 tokens (the budget of the 1.5B configuration's scheduler), as a step of its own
    portion_ms = []
    for rep in range(0 if (args.only_decode or args.only_prefill) else 3 + 5):
        cache = engine.cache.open(("portion", rep))
        engine.cache.reserve(cache, 512)
        entry = StepEntry(cache, random_prompt(512), [511])
        torch.cuda.synchronize()
        start, stop = events()
        start.record()
        engine.step([entry])
        stop.record()
        torch.cuda.synchronize()
        if rep >= 3:
            portion_ms.append(start.elapsed_time(stop))
        engine.cache.close(cache)
    if args.only_prefill:
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "layers": args.layers,
                          "ms": prefill_best, "tok_s": PREFILL_TOKENS / (prefill_best / 1e3)}))
        return 0
    prefill = {"value": PREFILL_TOKENS / (prefill_best / 1e3), "tokens": PREFILL_TOKENS,
               "ms": prefill_best,
               "frac": prefill_flops(cfg, args.layers, PREFILL_TOKENS) / (prefill_best / 1e3)
               / (pk["bf16_tflops"] * 1e12)}

    # ---- decode -----------------------------------------------------------------
    def decode_run(batch, steps, warmup, sample_clocks):
        caches = [engine.cache.open(("decode", batch, i)) for i in range(batch)]
        for lo in range(0, batch, 8):          # prompts in steps of up to 4,096 tokens
            group = caches[lo:lo + 8]
            for c in group:
                engine.cache.reserve(c, PROMPT_LEN)
            logits = engine.step([StepEntry(c, random_prompt(PROMPT_LEN), [PROMPT_LEN - 1])
                                  for c in group])
            first = engine.sampler.greedy(logits).tolist()
            for c, t in zip(group, first):
                c.next_token = t
        ids = engine.decode_steps([StepEntry(c, [c.next_token]) for c in caches], warmup)
        clocks = ClockSampler() if sample_clocks else None
        if clocks:
            clocks.start()
            time.sleep(0.25)
        torch.cuda.synchronize()
        launches = counter.launches
        start, stop = events()
        start.record()
        ids = engine.decode_steps([StepEntry(c, [t]) for c, t in zip(caches, ids[-1])], steps)
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop)
        launches = counter.launches - launches
        clock_record = clocks.stop() if clocks else None
        context = caches[0].length
        for c in caches:
            engine.cache.close(c)
        return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3),
                "launches": launches, "clocks": clock_record, "context_end": context}

    main_run = decode_run(args.batch, args.steps, args.warmup, not args.only_decode)
    if args.only_decode:
        print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": main_run["ms_per_step"],
                          "tok_s": main_run["tok_s"], "gpu_launches": main_run["launches"]}))
        return 0
    points = {}
    if portion_ms:
        points["prefill_512"] = 512 / (sorted(portion_ms)[len(portion_ms) // 2] / 1e3)
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = decode_run(b, min(args.steps, 64), 4, False)["tok_s"]

    mean_context = main_run["context_end"] - args.steps / 2
    step_bytes = weight_bytes(cfg, args.layers) + args.batch * mean_context * kv_bytes_per_token(cfg, args.layers)
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9

    # ---- the same through the Python entry point ----------------------------------
    from tokenizer_b200.engine.scheduler import Scheduler

    def through_scheduler(burst):
        """Decoding through the scheduler: host ids in, host ids out.  With burst 1
        every step copies its inputs to the device and its ids back."""
        prompts = [random_prompt(PROMPT_LEN) for _ in range(args.batch)]
        tokens = min(args.steps + args.warmup + burst, NEW_TOKENS)
        scheduler = Scheduler(engine, max_batch_size=args.batch, token_budget=8 * PROMPT_LEN,
                              decode_burst=burst)
        for p in prompts:
            scheduler.add_request(p, tb.GenerateParams(max_tokens=tokens))
        while any(len(r.context) == len(r.prompt) for r in scheduler.running) or scheduler.waiting:
            scheduler.step()                      # prompts, not timed
        while scheduler.stats.steps < args.warmup + 1:
            scheduler.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        sampled0, steps0 = scheduler.stats.tokens_sampled, scheduler.stats.steps
        while scheduler.has_work() and scheduler.stats.steps - steps0 + burst <= args.steps - 1:
            scheduler.step()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        steps = max(1, scheduler.stats.steps - steps0)
        value = (scheduler.stats.tokens_sampled - sampled0) / seconds
        scheduler.run()
        return value, steps

    e2e_value, e2e_steps = through_scheduler(1)
    h2d = engine.builder.last_bytes
    burst_value, burst_steps = through_scheduler(8)

    line = {
        "metric": "decode tok/s (Qwen2.5-0.5B sizes, batch %d, 512-token prompts)" % args.batch,
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": main_run["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": main_run["tok_s"] / 34.382, "dtype": "bf16",
        "data": "synthetic: random weights (seed 2), uniform random token ids",
        "config": {"model": "Qwen2.5-0.5B sizes", "layers": args.layers,
                   "layers_of_config": SIZES["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                   "vocab": cfg["vocab_size"], "global_batch": args.batch, "seq_len": PROMPT_LEN,
                   "new_tokens": NEW_TOKENS, "context_at_timing": int(mean_context),
                   "page_size": PAGE, "parallelism": "single GPU",
                   "l2": "each step reads > 126 MB of weights (inputs larger than L2)",
                   "peaks": pk["source"], "plain_products_of_65_rows_and_more": products_note()},
        "clocks": main_run["clocks"],
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4 * args.batch, "steps": e2e_steps,
                "note": "every step: its positions, slots and block tables from pinned host memory, its drawn "
                        "ids back to the host; a step's token ids reach it on the device, so the host reads "
                        "a draw while the next step runs"},
        "e2e_burst": {"value": burst_value, "unit": "tokens/s", "steps": burst_steps, "burst": 8,
                      "note": "8 greedy steps on the device between visits to the host: "
                              "one input copy and one read of 8 steps' ids per burst"},
        "gpu_launches": main_run["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
    }
    engine.check()                 # a bounded wait that ran out inside a kernel invalidates the numbers
    print(json.dumps(line))
    return 0


def run_stream_probe(args):
    """What a read-only stream reaches on this device in the access patterns of the decoding
    kernels: a [151552, 3584] bfloat16 matrix (1.09 GB, larger than L2) read once per launch,
    five launches after two of warm-up, CUDA events around them.  One JSON line."""
    import torch
    from tokenizer_b200.kernels import ops

    torch.cuda.set_device(0)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    N, K = 151552, 3584
    w = torch.ones((N, K), dtype=torch.bfloat16, device="cuda:0")
    sink = torch.zeros(16, dtype=torch.int32, device="cuda:0")
    nbytes = N * K * 2

    def rate(fn):
        fn(); fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(5):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return round(nbytes / (start.elapsed_time(stop) / 5 / 1e3) / 1e12, 2)

    out = {}
    for pattern in ("coalesced", "fragment", "fragment_wide"):
        for in_flight in (2, 4, 8):
            for per_sm in (2, 4, 8):
                if pattern == "coalesced" and in_flight == 2:
                    continue
                key = f"{pattern}, {in_flight} steps in flight, {per_sm} blocks an SM"
                out[key] = rate(lambda: ops.stream_probe_loads(w, pattern, in_flight, per_sm * sms, sink))
    for depth in (4, 6, 8):
        for per_sm in (1, 2, 3):
            if per_sm * 8 * depth * 16 * 144 > 220 * 1024:
                continue
            key = f"async ring of {depth} stages a warp, {per_sm} blocks an SM ({per_sm * 8 * (depth - 1) * 2} KB in flight)"
            out[key] = rate(lambda: ops.stream_probe_async_ring(w, depth, per_sm * sms, sink))
    for piece in (512, 1024, 1792, 3584, 7168):
        for rows in (16, 32):
            for kb in (64, 192):
                stages = min(16, kb * 1024 // (rows * piece))
                if stages < 2:
                    continue
                key = f"bulk copies of {piece} bytes, {rows} a stage, {stages} stages ({stages * rows * piece // 1024} KB)"
                out[key] = rate(lambda: ops.stream_probe_bulk(w, piece, rows, stages, sms, sink))
    print(json.dumps({"stream_probe_TB_per_s": out, "bytes": nbytes}))
    return 0


def run_layer_phases(args):
    """The whole-layer kernel for few rows at Qwen2.5-0.5B layer sizes: 24 launches with 24 sets of
    weights (a step's worth, so nothing stays in L2), the median over the later layers of the time at
    which the last block passes each phase (from the kernel's own stamps of %globaltimer), and the
    time per layer of the captured chain."""
    import math
    import torch
    from tokenizer_b200.kernels import ops as o

    torch.cuda.set_device(0)
    dev = "cuda:0"
    M, ctx = args.batch, PROMPT_LEN + 88
    H, I, nh, nkv, d = (SIZES[k] for k in ("hidden_size", "intermediate_size", "num_attention_heads",
                                           "num_key_value_heads", "head_dim"))
    L = SIZES["num_hidden_layers"]
    g = torch.Generator(device=dev).manual_seed(1)

    def rnd(*shape, dtype=torch.bfloat16, scale=0.05):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(dtype)

    layers = [dict(w_qkv=rnd((nh + 2 * nkv) * d, H), b=rnd((nh + 2 * nkv) * d, dtype=torch.float32),
                   w_o=rnd(H, nh * d), g1=1 + rnd(H, dtype=torch.float32), g2=1 + rnd(H, dtype=torch.float32),
                   w_gu=rnd(2 * I, H), w_d=rnd(H, I), k=rnd(M * 1024, nkv, d, scale=1.0),
                   v=rnd(M * 1024, nkv, d, scale=1.0)) for _ in range(L)]
    tables = torch.arange(M * 1024 // PAGE, dtype=torch.int32, device=dev).view(M, 1024 // PAGE)
    pos = torch.full((M,), ctx - 1, dtype=torch.int32, device=dev)
    slot = (tables[:, (ctx - 1) // PAGE] * PAGE + (ctx - 1) % PAGE).to(torch.int32)
    row_req = torch.arange(M, dtype=torch.int32, device=dev)
    inv = torch.tensor([1.0 / (1e6 ** (i / d)) for i in range(0, d, 2)], dtype=torch.float64).float().to(dev)
    cos, sin = o.rope_table(inv, 2048)
    down_splits, _ = o.layer_small_m_splits(M, H, I, nh, nkv, d)
    if down_splits == 0:
        print(json.dumps({"layer_phases": None, "why": "the layer kernel does not take %d rows" % M}))
        return 0
    x = rnd(M, H, dtype=torch.float32, scale=1.0)
    blocks = torch.cuda.get_device_properties(0).multi_processor_count
    stamps = torch.zeros(L, blocks, 32, dtype=torch.int64, device=dev)

    def chain(with_stamps):
        xin, delta = x, None
        for at, w in enumerate(layers):
            x_mid, x_out = torch.empty_like(x), torch.empty_like(x)
            out = torch.empty(down_splits, M, H, dtype=torch.float32, device=dev)
            nxt = layers[at + 1] if at + 1 < L else None
            o.layer_small_m(xin, delta, x_mid, x_out, out, w["g1"], 1e-6, w["w_qkv"], w["b"], pos, slot, row_req,
                            tables, cos, sin, w["k"], w["v"], True, w["w_o"], w["g2"], 1e-6, w["w_gu"], w["w_d"],
                            nh, nkv, d, PAGE, None, 1 / math.sqrt(d), "silu", stamps[at] if with_stamps else None,
                            (nxt["w_qkv"], nxt["g1"], nxt["b"]) if nxt else None)
            xin, delta = x_out, out

    for _ in range(3):
        chain(False)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        chain(False)
    for _ in range(3):
        graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(20):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    per_layer_us = start.elapsed_time(stop) / 20 / L * 1e3
    chain(True)
    torch.cuda.synchronize()
    o.raise_if_error()
    st = stamps[4:].double().cpu()
    base = st[:, :, 0].min(dim=1, keepdim=True).values
    names = ["start", "predecessor done", "first norm", "q/k/v", "barrier 1", "attention", "barrier 2",
             "output projection", "barrier 3", "second norm", "gate/up", "barrier 4", "down"]
    phases = {n: round(float(((st[:, :, i] - base) / 1e3).max(dim=1).values.median()), 2)
              for i, n in enumerate(names)}
    print(json.dumps({"layer_phases_us_since_start_last_block": phases, "rows": M, "context": ctx,
                      "us_per_layer_in_a_captured_chain": round(per_layer_us, 2), "layers": L,
                      "model": "Qwen2.5-0.5B layer sizes"}))
    return 0


def run_7b(args):
    """Qwen2.5-7B sizes: a prefill of 2,048 tokens, decoding at batch 1/8/64 with `--context`
    (8,192) tokens held by every request.  Weights are drawn on the device (15.2 GB in
    bfloat16 would be a long file); the cache holds the live requests of the largest batch."""
    import torch
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    from tokenizer_b200.kernels.ops import counter

    torch.cuda.set_device(0)
    layers = args.layers if args.layers != SIZES["num_hidden_layers"] else SIZES_7B["num_hidden_layers"]
    gate = None if args.skip_gate else gate_on_logits(SIZES_7B, "7B layer sizes")
    cfg = full_config(SIZES_7B, layers)
    config = tb.Qwen2Config.from_dict(cfg)
    pk = peaks()
    gen = torch.Generator().manual_seed(1234)
    model = tb.random_model(config, seed=2, dtype="bfloat16", device="cuda:0")
    context, steps = args.context, max(4, min(args.steps, 64))
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    per_request = context + steps + args.warmup + 2 * PAGE
    engine = tb.engine_for(model, max(batches) * per_request, PAGE, max_requests=max(batches),
                           share_prefixes=False)

    def random_ids(n):
        return torch.randint(0, config.vocab_size, (n,), generator=gen).tolist()

    def timed(fn):
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop), out

    prefill_ms = []
    for rep in range(3 + 3):
        cache = engine.cache.open(("prefill", rep))
        engine.cache.reserve(cache, PREFILL_TOKENS)
        entry = StepEntry(cache, random_ids(PREFILL_TOKENS), [PREFILL_TOKENS - 1])
        ms, _ = timed(lambda: engine.step([entry]))
        if rep >= 3:
            prefill_ms.append(ms)
        engine.cache.close(cache)
    prefill_best = sorted(prefill_ms)[len(prefill_ms) // 2]

    results = {}
    clocks_main = None
    for batch in batches:
        caches = [engine.cache.open(("decode", batch, i)) for i in range(batch)]
        nexts = []
        # contexts in steps of 2,048 tokens a request, four requests a step
        for lo in range(0, batch, 4):
            group = caches[lo:lo + 4]
            prompts = [random_ids(context) for _ in group]
            for done in range(0, context, 2048):
                take = min(2048, context - done)
                for c in group:
                    engine.cache.reserve(c, take)
                last = done + take == context
                logits = engine.step([StepEntry(c, p[done:done + take], [take - 1] if last else [])
                                      for c, p in zip(group, prompts)])
            nexts += engine.sampler.greedy(logits).tolist()
        ids = engine.decode_steps([StepEntry(c, [t]) for c, t in zip(caches, nexts)], args.warmup)
        clocks = ClockSampler() if batch == args.batch else None
        if clocks:
            clocks.start()
            time.sleep(0.25)
        launches = counter.launches
        ms, ids = timed(lambda: engine.decode_steps([StepEntry(c, [t]) for c, t in zip(caches, ids[-1])], steps))
        launches = counter.launches - launches
        if clocks:
            clocks_main = clocks.stop()
        mean_context = caches[0].length - steps / 2
        step_bytes = weight_bytes(cfg, layers) + batch * mean_context * kv_bytes_per_token(cfg, layers)
        results[batch] = {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
                          "frac": step_bytes / (ms / steps / 1e3) / 1e9 / pk["hbm_gbs"],
                          "gbs": step_bytes / (ms / steps / 1e3) / 1e9, "context": int(mean_context)}
        for c in caches:
            engine.cache.close(c)
    engine.check()
    main_run = results[args.batch]
    line = {
        "metric": "decode tok/s (Qwen2.5-7B sizes, batch %d, %d-token context)" % (args.batch, context),
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights drawn on the device (seed 2), uniform random token ids",
        "config": {"model": "Qwen2.5-7B sizes", "layers": layers, "layers_of_config": SIZES_7B["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": context, "context_at_timing": main_run["context"],
                   "page_size": PAGE, "parallelism": "single GPU",
                   "l2": "each step reads > 126 MB of weights (inputs larger than L2)", "peaks": pk["source"],
                   "logits_gate": gate, "plain_products_of_65_rows_and_more": products_note()},
        "clocks": clocks_main, "gpu_launches": main_run["launches"],
        "prefill": {"value": PREFILL_TOKENS / (prefill_best / 1e3), "tokens": PREFILL_TOKENS, "ms": prefill_best,
                    "frac": prefill_flops(cfg, layers, PREFILL_TOKENS) / (prefill_best / 1e3)
                    / (pk["bf16_tflops"] * 1e12)},
        "roofline": {"bound": "hbm", "achieved": main_run["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": main_run["frac"]},
        "points": {f"decode_b{b}": r["tok_s"] for b, r in results.items()},
        "points_frac": {f"decode_b{b}": r["frac"] for b, r in results.items()},
        "points_ms": {f"decode_b{b}": r["ms_per_step"] for b, r in results.items()},
    }
    print(json.dumps(line))
    return 0


# ---- a design's prefill and decoding, timed on the device ----
def device_timed(fn, reps=1):
    import torch
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        out = fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / reps, out

def measure_design(config, vocab, args, gen, context, steps):
    """Prefill of PREFILL_TOKENS tokens (one step, median of five) and decoding at batch 1 and `--batch` with
    `context`-token contexts, `steps` steps on the device, of a model of `config` with random weights."""
    import torch
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    from tokenizer_b200.kernels import ops
    from tokenizer_b200.parts.model import declared_tensors
    timed = device_timed
    model = tb.random_model(config, seed=3, dtype="bfloat16", device="cuda:0")
    params = sum(int(torch.tensor(t.shape).prod()) for t in declared_tensors(config.model_spec()))
    batches = sorted({1, args.batch})
    engine = tb.engine_for(model, max(batches) * (context + steps + args.warmup + 4 * PAGE), PAGE,
                           max_requests=max(batches), share_prefixes=False)
    ids = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
    prefill = []
    for rep in range(3 + 5):
        cache = engine.cache.open(("prefill", rep))
        engine.cache.reserve(cache, PREFILL_TOKENS)
        entry = StepEntry(cache, ids(PREFILL_TOKENS), [PREFILL_TOKENS - 1])
        ms, _ = timed(lambda: engine.step([entry]))
        if rep >= 3:
            prefill.append(ms)
        engine.cache.close(cache)
    out = {"parameters_m": round(params / 1e6, 1), "prefill_ms": sorted(prefill)[len(prefill) // 2]}
    out["prefill_tok_s"] = PREFILL_TOKENS / (out["prefill_ms"] / 1e3)
    for batch in batches:
        caches = [engine.cache.open(("decode", batch, i)) for i in range(batch)]
        nexts = []
        for lo in range(0, batch, 4):
            group = caches[lo:lo + 4]
            for c in group:
                engine.cache.reserve(c, context)
            logits = engine.step([StepEntry(c, ids(context), [context - 1]) for c in group])
            nexts += engine.sampler.greedy(logits).tolist()
        drawn = engine.decode_steps([StepEntry(c, [t]) for c, t in zip(caches, nexts)], args.warmup)
        launches = ops.counter.launches
        ms, _ = timed(lambda: engine.decode_steps([StepEntry(c, [t]) for c, t in zip(caches, drawn[-1])], steps))
        out[f"decode_b{batch}_ms"] = ms / steps
        out[f"decode_b{batch}_tok_s"] = batch * steps / (ms / 1e3)
        out[f"decode_b{batch}_launches_a_step"] = (ops.counter.launches - launches) // steps
        for c in caches:
            engine.cache.close(c)
    engine.check()
    del engine, model
    torch.cuda.empty_cache()
    return out


# ---- the Pufuzen design beside the Qwen2 decoder at equal width, depth and parameter count ----
PUFUZEN_SIZES = {
    # width, heads, dim / vdim of a head, query and key/value latents, positional lanes, recurrence width,
    # feed-forward width; `qwen_inner`: the gated feed-forward width that gives the Qwen2 model of the same
    # width, depth and heads about the same parameters a layer
    "1k": dict(width=1024, heads=16, dim=64, vdim=64, q_rank=384, kv_rank=128, kv_rank_rot=96, rot_dim=32,
               gru=2048, ff=2816, vocab=32000, layers=8, window=1024, qwen_head_dim=64, qwen_inner=2432),
    "2k": dict(width=2048, heads=16, dim=128, vdim=128, q_rank=768, kv_rank=128, kv_rank_rot=96, rot_dim=32,
               gru=4096, ff=5632, vocab=32000, layers=8, window=1024, qwen_head_dim=128, qwen_inner=4864),
}


def pufuzen_config(z):
    """Layers in the pattern recurrence, windowed latent attention, rotary latent attention with a
    sink, recurrence; the attention layers carry the feed-forward."""
    import tokenizer_b200 as tb
    dense = {"kind": "dense", "ff": z["ff"]}
    gru = {"type": "mingru", "mixer": {"width": z["gru"]}, "mlp": None}
    common = {"heads": z["heads"], "dim": z["dim"], "vdim": z["vdim"], "q_rank": z["q_rank"]}
    windowed = {"type": "latent_attention", "mlp": dense,
                "mixer": dict(common, kv_rank=z["kv_rank"], scale=z["dim"] ** -0.5, mask={"size": z["window"]})}
    rotary = {"type": "latent_attention_2", "mlp": dense,
              "mixer": dict(common, kv_rank=z["kv_rank_rot"], rot_dim=z["rot_dim"], scale=(z["dim"] + z["rot_dim"]) ** -0.5,
                            rot={"base": 500000.0, "dims": z["rot_dim"]})}
    pattern = [gru, windowed, rotary, gru]
    return tb.config.PufuzenConfig.from_dict({
        "architecture": "Pufuzen", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5},
        "logit_scale": 1.0, "layers": [pattern[i % 4] for i in range(z["layers"])]})


def run_pufuzen(args):
    """Prefill (one step of 2,048 tokens) and decoding (batch 1 and `--batch`, 2,048-token contexts) of
    the Pufuzen design at two widths, beside the Qwen2 decoder of the same width, depth, heads and
    about the same parameters a layer; then the design's own kernels alone beside the like kernels
    of the Qwen2 path, each on inputs larger than L2, as bytes a second of the measured copy peak."""
    import torch
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    from tokenizer_b200.kernels import ops
    from tokenizer_b200.parts.model import declared_tensors

    torch.cuda.set_device(0)
    pk = peaks()
    gen = torch.Generator().manual_seed(99)
    context, steps = 2048, max(8, min(args.steps, 64))

    timed = device_timed

    def measure(config, vocab):
        return measure_design(config, vocab, args, gen, context, steps)

    models = {}
    for name, z in PUFUZEN_SIZES.items():
        models[name] = {"pufuzen": measure(pufuzen_config(z), z["vocab"])}
        qwen = tb.Qwen2Config.from_dict(dict(
            architectures=["Qwen2ForCausalLM"], hidden_act="silu", num_hidden_layers=z["layers"],
            hidden_size=z["width"], num_attention_heads=z["heads"], num_key_value_heads=2, head_dim=z["qwen_head_dim"],
            intermediate_size=z["qwen_inner"], vocab_size=z["vocab"], rope_theta=1000000.0, rms_norm_eps=1e-6,
            tie_word_embeddings=False, max_position_embeddings=32768, use_sliding_window=False,
            sliding_window=32768, max_window_layers=z["layers"]))
        models[name]["qwen2"] = measure(qwen, z["vocab"])

    # ---- kernels alone: inputs larger than L2, a 256 MB write between the timed launches ----
    dev = "cuda:0"
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)

    def kernel_time(fn, reps=7):
        times = []
        for _ in range(3 + reps):
            flush.zero_()
            ms, _ = timed(fn)
            times.append(ms)
        return sorted(times[3:])[reps // 2]

    kernels = {}

    def record(name, ms, nbytes, like):
        kernels[name] = {"us": round(ms * 1e3, 1), "gb_s": round(nbytes / (ms / 1e3) / 1e9), "like": like,
                         "of_measured_copy_peak": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 2)}

    T, W, H, I = 8192, 4096, 2048, 5632
    rnd = lambda *shape, dtype=torch.float32: torch.randn(*shape, device=dev, dtype=torch.float32).to(dtype)
    proj = rnd(T, 3 * W)
    state = torch.zeros(4, W, device=dev)
    out16 = torch.empty(T, W, dtype=torch.bfloat16, device=dev)
    for requests in (1, 4):
        spans = torch.tensor([T * r // requests for r in range(requests + 1)], dtype=torch.int32, device=dev)
        slots = torch.arange(requests, dtype=torch.int32, device=dev)
        record(f"min_gru_scan, {T} tokens of {requests} request(s), width {W}",
               kernel_time(lambda: ops.min_gru_scan(proj, 0, W, 2 * W, W, state, spans, slots, T // requests, out16)),
               T * W * (3 * 4 + 2), "silu_gate")
    z = rnd(T, I + H)
    act = torch.empty(T, I, dtype=torch.bfloat16, device=dev)
    coeff = torch.tensor([0.5, 0.3, 0.2, 0.1], device=dev)
    record(f"poly_norm, {T} x {I}", kernel_time(lambda: ops.poly_norm(z[:, :I], coeff, 1e-5, act)), T * I * (4 + 2),
           "silu_gate")
    y = rnd(T, H, dtype=torch.bfloat16)
    delta = torch.empty(T, H, device=dev)
    record(f"gated_delta, {T} x {H}", kernel_time(lambda: ops.gated_delta(y, None, z[:, I:], delta)), T * H * (2 + 4 + 4),
           "rms_norm")
    q_rank, kv_rank, rot = 768, 96, 32
    wide = rnd(T, q_rank + kv_rank + rot + H)
    pool = torch.zeros(T + 64, 1, 128, dtype=torch.bfloat16, device=dev)
    cq = torch.empty(T, q_rank, dtype=torch.bfloat16, device=dev)
    ones_q, ones_c = torch.ones(q_rank, device=dev), torch.ones(kv_rank, device=dev)
    freq = torch.tensor([500000.0 ** (-2.0 * i / rot) for i in range(rot // 2)], device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    req = torch.zeros(T, dtype=torch.int32, device=dev)
    record(f"latent_prepare, {T} tokens", kernel_time(lambda: ops.latent_prepare(
        wide, 0, q_rank, q_rank, kv_rank, rot, rot, ones_q, ones_c, 1e-5, freq, pos, req, pos, cq, pool)),
        T * ((q_rank + kv_rank + rot) * 4 + (q_rank + 128) * 2), "rope_store")
    q = rnd(T, 16 * 128, dtype=torch.bfloat16)
    record(f"rotate_interleaved, {T} tokens x 16 heads, 32 of 128 lanes",
           kernel_time(lambda: ops.rotate_interleaved(q, 16, kv_rank, rot, freq, pos, req)), T * 16 * 128 * 2 * 2 // 2,
           "rope_store")
    # the like kernels of the Qwen2 path
    gu = rnd(T, 2 * I, dtype=torch.bfloat16)
    record(f"silu_gate, {T} x {I} (Qwen2 path)", kernel_time(lambda: ops.silu_gate(gu, act)), T * I * 6, None)
    x = rnd(T, H)
    gain = torch.ones(H, device=dev)
    h16 = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    record(f"rms_norm with pending add, {T} x {H} (Qwen2 path)",
           kernel_time(lambda: ops.rms_norm(x, gain, 1e-6, h16, delta=y)), T * H * (4 + 4 + 2 + 2), None)
    nh, nkv, d = 16, 2, 128
    qkv = rnd(T, (nh + 2 * nkv) * d, dtype=torch.bfloat16)
    cos, sin = ops.rope_table(torch.tensor([1e6 ** (-2.0 * i / d) for i in range(d // 2)], device=dev), T)
    q_out = torch.empty(T, nh * d, dtype=torch.bfloat16, device=dev)
    k_pool = torch.zeros(T + 64, nkv, d, dtype=torch.bfloat16, device=dev)
    v_pool = torch.zeros_like(k_pool)
    record(f"rope_store, {T} tokens (Qwen2 path)", kernel_time(lambda: ops.rope_store(
        qkv, None, pos, pos, cos, sin, q_out, k_pool, v_pool, nh, nkv, d, d)), T * (nh + 2 * nkv) * d * 2 * 2, None)
    # decoding attention: 64 rows of 8,192 keys; the latent's row is read as keys and as values
    rows, keys = 64, 8192
    pages = rows * keys // PAGE
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(rows, keys // PAGE)
    row_req = torch.arange(rows, dtype=torch.int32, device=dev)
    last = torch.full((rows,), keys - 1, dtype=torch.int32, device=dev)
    lat = rnd(rows * keys, 1, 128, dtype=torch.bfloat16)
    ql = rnd(rows, 16 * 128, dtype=torch.bfloat16)
    ol = torch.empty_like(ql)
    sink = torch.zeros(16, device=dev)
    record("decode attention over a cached latent, 64 rows x 8,192 keys, 16 heads, rows of 128 lanes",
           kernel_time(lambda: ops.decode_attention(ql, lat, lat, ol, table, row_req, last, 16, 1, 128, PAGE, None, 0.09,
                                                    sink=sink)), rows * keys * 128 * 2, "decode attention (Qwen2 path)")
    kq, vq = rnd(rows * keys, 2, 128, dtype=torch.bfloat16), rnd(rows * keys, 2, 128, dtype=torch.bfloat16)
    record("decode attention, 64 rows x 8,192 keys, 16 heads over 2 of 128 lanes (Qwen2 path)",
           kernel_time(lambda: ops.decode_attention(ql, kq, vq, ol, table, row_req, last, 16, 2, 128, PAGE, None, 0.09)),
           rows * keys * 2 * 2 * 128 * 2, None)
    ops.raise_if_error()
    print(json.dumps({
        "metric": "prefill and decode tok/s of the Pufuzen design beside Qwen2 at equal width, depth and parameters",
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup, "dtype": "bf16",
        "data": "synthetic: random weights drawn on the device, uniform random token ids",
        "config": {"sizes": PUFUZEN_SIZES, "prefill_tokens": PREFILL_TOKENS, "decode_context": context,
                   "peaks": pk["source"], "hbm_gbs": pk["hbm_gbs"],
                   "l2": "kernels alone: inputs larger than L2 and a 256 MB write between timed launches"},
        "models": models, "kernels": kernels}))
    return 0


# ---- the Katopel design beside the Qwen2 decoder at equal width, depth and parameter count ----
KATOPEL_SIZES = {
    # width; the attention beside the delta rule (heads over kv heads of dim / vdim lanes, chunks of `chunk`
    # positions, `rot` rotated lanes); the delta rule (heads over kv heads, dim x vdim matrices, taps); dense and
    # expert feed-forward widths (experts, of which a token uses `top`, and a shared one)
    "1k": dict(width=1024, heads=16, kv_heads=4, dim=64, vdim=64, chunk=1024, rot=32, d_heads=8, d_kv=4, d_dim=128,
               d_vdim=128, taps=4, ff=2816, experts=8, top=2, expert_ff=704, shared_ff=1408, vocab=32000, layers=8,
               qwen_head_dim=64),
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, chunk=1024, rot=64, d_heads=16, d_kv=8, d_dim=128,
               d_vdim=128, taps=4, ff=5632, experts=8, top=2, expert_ff=1408, shared_ff=2816, vocab=32000, layers=8,
               qwen_head_dim=128),
}


def katopel_config(z):
    """Layers in the pattern delta rule + dense, two mixers side by side + experts, two mixers side by side +
    dense, delta rule + experts; no loop, so that every layer has weights of its own as in the model beside it."""
    import tokenizer_b200 as tb
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["shared_ff"]}}
    delta = {"heads": z["d_heads"], "kv_heads": z["d_kv"], "dim": z["d_dim"], "vdim": z["d_vdim"], "conv": z["taps"]}
    left = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
            "mask": {"size": z["chunk"]}, "rot": {"base": 1000000.0, "dims": z["rot"]}}
    side = {"left": left, "right": delta, "left_scale": 0.5, "right_scale": 1.25}
    pattern = [{"type": "delta", "mixer": delta, "mlp": dense}, {"type": "parallel", "mixer": side, "mlp": moe},
               {"type": "parallel", "mixer": side, "mlp": dense}, {"type": "delta", "mixer": delta, "mlp": moe}]
    return tb.config.KatopelConfig.from_dict({
        "architecture": "Katopel", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6},
        "embedding": {"scale": 2.0}, "layers": [pattern[i % 4] for i in range(z["layers"])]})


def run_katopel(args):
    """Prefill (one step of 2,048 tokens) and decoding (batch 1 and `--batch`, 2,048-token contexts) of the
    Katopel design at two widths, beside the Qwen2 decoder of the same width, depth and heads with the
    feed-forward width that gives it the same parameters; then the design's own kernels alone beside the like
    kernels of the paths that were there before, each on inputs larger than L2, against the measured copy peak."""
    import torch
    import tokenizer_b200 as tb
    from tokenizer_b200.kernels import ops
    from tokenizer_b200.parts.model import declared_tensors

    torch.cuda.set_device(0)
    pk = peaks()
    gen = torch.Generator().manual_seed(99)
    context, steps = 2048, max(8, min(args.steps, 64))
    timed = device_timed
    count = lambda config: sum(int(torch.tensor(t.shape).prod()) for t in declared_tensors(config.model_spec()))

    def qwen_config(z, inner):
        return tb.Qwen2Config.from_dict(dict(
            architectures=["Qwen2ForCausalLM"], hidden_act="silu", num_hidden_layers=z["layers"],
            hidden_size=z["width"], num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"],
            head_dim=z["qwen_head_dim"], intermediate_size=inner, vocab_size=z["vocab"], rope_theta=1000000.0,
            rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=32768, use_sliding_window=False,
            sliding_window=32768, max_window_layers=z["layers"]))

    models = {}
    for name, z in KATOPEL_SIZES.items():
        if args.only_kernels:
            break
        config = katopel_config(z)
        models[name] = {"katopel": measure_design(config, z["vocab"], args, gen, context, steps)}
        # the gated feed-forward width (whole 128s) that brings Qwen2 to the same parameters
        base, step = count(qwen_config(z, 128)), count(qwen_config(z, 256)) - count(qwen_config(z, 128))
        inner = max(1, round((count(config) - base) / step) + 1) * 128
        models[name]["qwen2"] = dict(measure_design(qwen_config(z, inner), z["vocab"], args, gen, context, steps),
                                     intermediate_size=inner)

    # ---- kernels alone: inputs larger than L2, a 256 MB write between the timed launches ----
    dev = "cuda:0"
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)

    def kernel_time(fn, reps=7):
        times = []
        for _ in range(3 + reps):
            flush.zero_()
            ms, _ = timed(fn)
            times.append(ms)
        return sorted(times[3:])[reps // 2]

    kernels = {}

    def record(name, ms, nbytes, like, flops=None):
        kernels[name] = {"us": round(ms * 1e3, 1), "gb_s": round(nbytes / (ms / 1e3) / 1e9), "like": like,
                         "of_measured_copy_peak": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 2)}
        if flops is not None:
            kernels[name]["fp32_tflops"] = round(flops / (ms / 1e3) / 1e12, 1)

    ints = lambda values: torch.tensor(list(values), dtype=torch.int32, device=dev)
    rnd = lambda *shape, dtype=torch.float32: torch.randn(*shape, device=dev, dtype=torch.float32).to(dtype)
    T, H, I = 8192, 2048, 5632
    heads, groups, dim, vdim, taps = 16, 8, 128, 128, 4
    channels = 2 * groups * dim + heads * vdim
    padded = ops.gdn_padded_dim(dim)
    conv_off = heads * vdim * padded
    slot_floats = -(-(conv_off + (taps - 1) * channels) // 4) * 4
    proj = rnd(T, channels + 2 * heads + heads * vdim)
    conv, a_log, dt_bias = rnd(channels, taps), rnd(heads), rnd(heads)
    qkv, bg = torch.empty(T, channels, device=dev), torch.empty(T, 2 * heads + groups, device=dev)
    o = torch.empty(T, heads * vdim, device=dev)
    y16 = torch.empty(T, heads * vdim, dtype=torch.bfloat16, device=dev)
    gain_v = torch.ones(vdim, device=dev)
    for requests in (1, 4):
        state = torch.zeros(requests, slot_floats, device=dev)
        spans, slots = ints(T * r // requests for r in range(requests + 1)), ints(range(requests))
        row_req = ints(r for r in range(requests) for _ in range(T // requests))
        record(f"gdn_prepare, {T} tokens of {requests} request(s), {channels} channels of {taps} taps",
               kernel_time(lambda: ops.gdn_prepare(proj, 0, channels, channels + heads, groups, heads, dim, vdim, taps, conv,
                                                   a_log, dt_bias, state, conv_off, row_req, spans, slots, qkv, bg)),
               T * (channels + 2 * heads) * 8, "rope_store")
        record(f"gdn_scan, {T} tokens of {requests} request(s), {heads} heads of {dim} x {vdim}",
               kernel_time(lambda: ops.gdn_scan(qkv, bg, groups, heads, dim, vdim, state, spans, slots, o, longest=T // requests)),
               T * (channels + 2 * heads + heads * vdim) * 4, "min_gru_scan", flops=T * heads * dim * vdim * 8)
    record(f"gdn_out_norm, {T} tokens x {heads} heads of {vdim}",
           kernel_time(lambda: ops.gdn_out_norm(o, proj, channels + 2 * heads, gain_v, 1.0, 1e-6, y16, heads, vdim, row_req)),
           T * heads * vdim * (4 + 4 + 2), "silu_gate")
    # decoding: 64 requests of one token each; the matrices are read and written once a token
    rows = 64
    state = torch.zeros(rows, slot_floats, device=dev)
    spans, slots = ints(range(rows + 1)), ints(range(rows))
    record(f"gdn_scan, {rows} requests of one token, {heads} heads of {dim} x {vdim}",
           kernel_time(lambda: ops.gdn_scan(qkv[:rows], bg[:rows], groups, heads, dim, vdim, state, spans, slots, o[:rows])),
           rows * conv_off * 8, "decode attention")
    x, y = rnd(T, H), rnd(T, H, dtype=torch.bfloat16)
    g1, b1 = torch.ones(H, device=dev), torch.zeros(H, device=dev)
    h16 = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    record(f"post_norm_add with the next norm, {T} x {H}",
           kernel_time(lambda: ops.post_norm_add(x, [(y, 1.0)], g1, b1, 1e-6, g1, b1, 1e-6, h16)), T * H * (2 + 4 + 4 + 2),
           "rms_norm")
    two = rnd(2, T, H)
    record(f"post_norm_add of two scaled terms (float32 partial sums and bfloat16) with the next norm, {T} x {H}",
           kernel_time(lambda: ops.post_norm_add(x, [(two, 0.5), (y, 1.25)], g1, b1, 1e-6, g1, b1, 1e-6, h16)),
           T * H * (8 + 2 + 4 + 4 + 2), "rms_norm")
    nh, nkv, d = 16, 4, 128
    wide = rnd(T, (nh + 2 * nkv) * d + 64)
    bias = torch.zeros((nh + 2 * nkv) * d, device=dev)
    freq = torch.tensor([1e6 ** (-2.0 * i / 64) for i in range(32)], device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    req = torch.zeros(T, dtype=torch.int32, device=dev)
    q_out = torch.empty(T, nh * d, dtype=torch.bfloat16, device=dev)
    k_pool = torch.zeros(T + 64, nkv, d, dtype=torch.bfloat16, device=dev)
    v_pool = torch.zeros_like(k_pool)
    record(f"qkv_rotate_store, {T} tokens, {nh} heads over {nkv} of {d} lanes, 64 rotated",
           kernel_time(lambda: ops.qkv_rotate_store(wide, 64, bias, freq, 64, pos, pos, req, q_out, k_pool, v_pool, nh, nkv, d, d, d)),
           T * (nh + 2 * nkv) * d * (4 + 2), "rope_store")
    experts, ff, shared_ff = 8, 512, 1536
    gu = rnd(T, 2 * I, dtype=torch.bfloat16)
    share = torch.rand(T, experts + 1, device=dev)
    act = torch.empty(T, I, dtype=torch.bfloat16, device=dev)
    record(f"moe_gate, {T} x {I} lanes of {experts} experts and a shared one",
           kernel_time(lambda: ops.moe_gate(gu, share, act, experts, ff, True)), T * I * 6, "silu_gate")
    h_in = rnd(T, H, dtype=torch.bfloat16)
    router = rnd(experts + 1, H)
    record(f"moe_route, {T} tokens, {experts} experts of which 2, width {H}",
           kernel_time(lambda: ops.moe_route(h_in, router, experts, 2, True, share)), T * H * 2, "rms_norm")
    # the like kernels of the paths that were there before
    record(f"silu_gate, {T} x {I}", kernel_time(lambda: ops.silu_gate(gu, act)), T * I * 6, None)
    gain = torch.ones(H, device=dev)
    record(f"rms_norm with pending add, {T} x {H}", kernel_time(lambda: ops.rms_norm(x, gain, 1e-6, h16, delta=y)),
           T * H * (4 + 4 + 2 + 2), None)
    qkv16 = rnd(T, (nh + 2 * nkv) * d, dtype=torch.bfloat16)
    cos, sin = ops.rope_table(torch.tensor([1e6 ** (-2.0 * i / d) for i in range(d // 2)], device=dev), T)
    record(f"rope_store, {T} tokens", kernel_time(lambda: ops.rope_store(
        qkv16, None, pos, pos, cos, sin, q_out, k_pool, v_pool, nh, nkv, d, d)), T * (nh + 2 * nkv) * d * 2 * 2, None)
    W = 4096
    gru = rnd(T, 3 * W)
    gru_state = torch.zeros(4, W, device=dev)
    out16 = torch.empty(T, W, dtype=torch.bfloat16, device=dev)
    record(f"min_gru_scan, {T} tokens of one request, width {W}",
           kernel_time(lambda: ops.min_gru_scan(gru, 0, W, 2 * W, W, gru_state, ints([0, T]), ints([0]), T, out16)),
           T * W * (3 * 4 + 2), None)
    keys = 8192
    table = torch.arange(rows * keys // PAGE, dtype=torch.int32, device=dev).view(rows, keys // PAGE)
    last = torch.full((rows,), keys - 1, dtype=torch.int32, device=dev)
    kq, vq = rnd(rows * keys, 2, 128, dtype=torch.bfloat16), rnd(rows * keys, 2, 128, dtype=torch.bfloat16)
    ql = rnd(rows, 16 * 128, dtype=torch.bfloat16)
    ol = torch.empty_like(ql)
    record("decode attention, 64 rows x 8,192 keys, 16 heads over 2 of 128 lanes",
           kernel_time(lambda: ops.decode_attention(ql, kq, vq, ol, table, ints(range(rows)), last, 16, 2, 128, PAGE, None, 0.09)),
           rows * keys * 2 * 2 * 128 * 2, None)
    ops.raise_if_error()
    print(json.dumps({
        "metric": "prefill and decode tok/s of the Katopel design beside Qwen2 at equal width, depth and parameters",
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup, "dtype": "bf16",
        "data": "synthetic: random weights drawn on the device, uniform random token ids",
        "config": {"sizes": KATOPEL_SIZES, "prefill_tokens": PREFILL_TOKENS, "decode_context": context,
                   "peaks": pk["source"], "hbm_gbs": pk["hbm_gbs"],
                   "l2": "kernels alone: inputs larger than L2 and a 256 MB write between timed launches"},
        "models": models, "kernels": kernels}))
    return 0


# ---- the Vizonex design beside the Katopel design at equal width, depth and parameter count ----
VIZONEX_SIZES = {
    # width; the attention (heads over kv heads of dim / vdim lanes, chunks of `chunk` positions); the state-space
    # mixer (heads of vdim lanes, `state` lanes in `groups` groups, taps, parts of the output norm); experts (of
    # which a token uses `top`, inside the best `keep` of `egroups` groups) and a shared one; taps in front of every
    # mixer.  The dense feed-forward's width is chosen so that the model has the parameters of the Katopel model
    # of the same name.
    "1k": dict(width=1024, heads=16, kv_heads=4, dim=64, vdim=64, chunk=1024, s_heads=16, s_vdim=64, state=128, groups=1,
               conv=4, norm_groups=1, experts=8, top=2, egroups=2, keep=1, expert_ff=704, shared_ff=1408, taps=4,
               vocab=32000, layers=8, positions=4096),
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, chunk=1024, s_heads=64, s_vdim=64, state=128, groups=8,
               conv=4, norm_groups=8, experts=8, top=2, egroups=4, keep=2, expert_ff=1408, shared_ff=2816, taps=4,
               vocab=32000, layers=8, positions=4096),
}


def vizonex_config(z, ff):
    """Layers in the pattern state space + dense, attention + experts, state space + experts, attention + dense."""
    import tokenizer_b200 as tb
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"], "limit": 7.0},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 2.5, "groups": {"count": z["egroups"], "keep": z["keep"]}},
           "shared": {"ff": z["shared_ff"], "limit": 7.0}}
    ssm = {"heads": z["s_heads"], "vdim": z["s_vdim"], "state": z["state"], "groups": z["groups"], "conv": z["conv"],
           "norm_groups": z["norm_groups"]}
    attn = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
            "mask": {"size": z["chunk"]}}
    pattern = [{"type": "mamba2", "mixer": ssm, "mlp": dense}, {"type": "attention", "mixer": attn, "mlp": moe},
               {"type": "mamba2", "mixer": ssm, "mlp": moe}, {"type": "attention", "mixer": attn, "mlp": dense}]
    return tb.config.VizonexConfig.from_dict({
        "architecture": "Vizonex", "vocab": z["vocab"], "width": z["width"], "max_positions": z["positions"],
        "norm": {"eps": 1e-6}, "canon": {"taps": z["taps"]}, "layers": [pattern[i % 4] for i in range(z["layers"])]})


def run_vizonex(args):
    """Prefill (one step of 2,048 tokens) and decoding (batch 1 and `--batch`, 2,048-token contexts) of the
    Vizonex design at two widths, beside the closest design that was there, Katopel (a recurrence with a matrix
    state a head, attention inside chunks, routed experts), at the same width and depth with the dense
    feed-forward width that gives both the same parameters; then the design's own kernels alone beside the like
    kernels of the other paths, each on inputs larger than L2, against the measured copy peak."""
    import torch
    import tokenizer_b200 as tb
    from tokenizer_b200.kernels import ops
    from tokenizer_b200.parts.model import declared_tensors

    torch.cuda.set_device(0)
    pk = peaks()
    gen = torch.Generator().manual_seed(99)
    context, steps = 2048, max(8, min(args.steps, 64))
    timed = device_timed
    count = lambda config: sum(int(torch.tensor(t.shape).prod()) for t in declared_tensors(config.model_spec()))

    models = {}
    for name, z in VIZONEX_SIZES.items():
        if args.only_kernels:
            break
        beside = katopel_config(KATOPEL_SIZES[name])
        base, step = count(vizonex_config(z, 128)), count(vizonex_config(z, 256)) - count(vizonex_config(z, 128))
        ff = max(1, round((count(beside) - base) / step) + 1) * 128
        models[name] = {"vizonex": dict(measure_design(vizonex_config(z, ff), z["vocab"], args, gen, context, steps), ff=ff),
                        "katopel": measure_design(beside, z["vocab"], args, gen, context, steps)}

    # ---- kernels alone: inputs larger than L2, a 256 MB write between the timed launches ----
    dev = "cuda:0"
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)

    def kernel_time(fn, reps=7):
        times = []
        for _ in range(3 + reps):
            flush.zero_()
            ms, _ = timed(fn)
            times.append(ms)
        return sorted(times[3:])[reps // 2]

    kernels = {}

    def record(name, ms, nbytes, like, flops=None):
        kernels[name] = {"us": round(ms * 1e3, 1), "gb_s": round(nbytes / (ms / 1e3) / 1e9), "like": like,
                         "of_measured_copy_peak": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 2)}
        if flops is not None:
            kernels[name]["fp32_tflops"] = round(flops / (ms / 1e3) / 1e12, 1)

    ints = lambda values: torch.tensor(list(values), dtype=torch.int32, device=dev)
    rnd = lambda *shape, dtype=torch.float32: torch.randn(*shape, device=dev, dtype=torch.float32).to(dtype)
    T, H, I = 8192, 2048, 5632
    # the state-space mixer at the 2k size: 64 heads of 64 lanes, 128 state lanes in 8 groups, 4 taps
    heads, groups, vdim, n_state, taps, parts = 64, 8, 64, 128, 4, 8
    inner, channels = heads * vdim, heads * vdim + 2 * groups * n_state
    conv_off = heads * vdim * n_state
    slot_floats = -(-(conv_off + (taps - 1) * channels) // 4) * 4
    proj = rnd(T, inner + channels + heads)
    conv_w, conv_b = rnd(channels, taps), rnd(channels)
    a_log, dt_bias, skip = rnd(heads), rnd(heads), rnd(heads)
    xbc = torch.empty(T, channels, device=dev)
    y = torch.empty(T, inner, device=dev)
    y16 = torch.empty(T, inner, dtype=torch.bfloat16, device=dev)
    gain_i = torch.ones(inner, device=dev)
    for requests in (1, 4):
        state = torch.zeros(requests, slot_floats, device=dev)
        spans, slots = ints(T * r // requests for r in range(requests + 1)), ints(range(requests))
        row_req = ints(r for r in range(requests) for _ in range(T // requests))
        record(f"short_conv with silu, {T} tokens of {requests} request(s), {channels} channels of {taps} taps",
               kernel_time(lambda: ops.short_conv(proj, inner, channels, conv_w, conv_b, state, conv_off, row_req, spans, slots,
                                                  xbc, activation="silu")), T * channels * 8, "gdn_prepare")
        record(f"mamba2_scan, {T} tokens of {requests} request(s), {heads} heads of {n_state} x {vdim}",
               kernel_time(lambda: ops.mamba2_scan(xbc, proj, inner + channels, dt_bias, a_log, skip, heads, groups, vdim,
                                                   n_state, state, spans, slots, y)),
               T * (channels + heads + inner) * 4, "gdn_scan", flops=T * heads * n_state * vdim * 4)
    record(f"mamba2_out_norm, {T} tokens x {inner} lanes in {parts} parts",
           kernel_time(lambda: ops.mamba2_out_norm(y, proj, 0, gain_i, 1e-6, parts, row_req, y16)), T * inner * (4 + 4 + 2),
           "gdn_out_norm")
    rows = 64
    state = torch.zeros(rows, slot_floats, device=dev)
    spans, slots = ints(range(rows + 1)), ints(range(rows))
    record(f"mamba2_scan, {rows} requests of one token, {heads} heads of {n_state} x {vdim}",
           kernel_time(lambda: ops.mamba2_scan(xbc[:rows], proj[:rows], inner + channels, dt_bias, a_log, skip, heads, groups,
                                               vdim, n_state, state, spans, slots, y[:rows])),
           rows * conv_off * 8, "gdn_scan, one token")
    # the layer's own kernels: the convolution in front of the mixer (on four times the rows: bfloat16 in and out, and
    # the rows of T alone would fit L2), the scaled add with the next norm
    T4 = 4 * T
    h16 = rnd(T4, H, dtype=torch.bfloat16)
    canon = rnd(H, taps)
    side = torch.zeros(4, (taps - 1) * H, device=dev)
    read16 = torch.empty(T4, H, dtype=torch.bfloat16, device=dev)
    spans4, slots4 = ints(T4 * r // 4 for r in range(5)), ints(range(4))
    row_req4 = ints(r for r in range(4) for _ in range(T4 // 4))
    record(f"short_conv added to its input, {T4} x {H}, {taps} taps",
           kernel_time(lambda: ops.short_conv(h16, 0, H, canon, None, side, 0, row_req4, spans4, slots4, read16, residual=True)),
           T4 * H * 4, "silu_gate")
    del h16, read16
    x, a16, b16 = rnd(T, H), rnd(T, H, dtype=torch.bfloat16), rnd(T, H, dtype=torch.bfloat16)
    v1, v2, g1 = torch.ones(H, device=dev), torch.ones(H, device=dev), torch.ones(H, device=dev)
    out16 = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    record(f"scaled_add_norm, two scaled outputs and the next norm, {T} x {H}",
           kernel_time(lambda: ops.scaled_add_norm(x, [(a16, v1), (b16, v2)], g1, 1e-6, out16)), T * H * (2 + 2 + 4 + 4 + 2),
           "rms_norm")
    nh, nkv, d = 16, 4, 128
    wide = rnd(T, (nh + 2 * nkv) * d)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    req = torch.zeros(T, dtype=torch.int32, device=dev)
    q_out = torch.empty(T, nh * d, dtype=torch.bfloat16, device=dev)
    k_pool = torch.zeros(T + 64, nkv, d, dtype=torch.bfloat16, device=dev)
    v_pool = torch.zeros_like(k_pool)
    qg, kg, temp = torch.ones(nh * d, device=dev), torch.ones(nkv * d, device=dev), torch.ones(nh, device=dev)
    record(f"qkv_rotate_store with whole-projection norms and temperatures, {T} tokens, {nh} heads over {nkv} of {d} lanes",
           kernel_time(lambda: ops.qkv_rotate_store(wide, 0, None, None, 0, pos, pos, req, q_out, k_pool, v_pool, nh, nkv, d, d, d,
                                                    q_gain=qg, k_gain=kg, eps=1e-6, temp=temp)),
           T * (nh + 2 * nkv) * d * (4 + 2), "qkv_rotate_store")
    freq = torch.tensor([1e6 ** (-2.0 * i / 64) for i in range(32)], device=dev)
    bias = torch.zeros((nh + 2 * nkv) * d, device=dev)
    record(f"qkv_rotate_store, biases and 64 rotated lanes (Katopel path), {T} tokens",
           kernel_time(lambda: ops.qkv_rotate_store(wide, 0, bias, freq, 64, pos, pos, req, q_out, k_pool, v_pool, nh, nkv, d, d, d)),
           T * (nh + 2 * nkv) * d * (4 + 2), None)
    experts, ff, shared_ff = 8, 512, 1536
    gu = rnd(T, 2 * I, dtype=torch.bfloat16)
    share = torch.rand(T, experts + 1, device=dev)
    act = torch.empty(T, I, dtype=torch.bfloat16, device=dev)
    record(f"moe_gate, clamped activation, {T} x {I} lanes of {experts} experts and a shared one",
           kernel_time(lambda: ops.moe_gate(gu, share, act, experts, ff, True, activation="clamped_swish", limit=7.0,
                                            shared_limit=7.0, alpha=1.702)), T * I * 6, "moe_gate")
    record(f"moe_gate, silu (Katopel path), {T} x {I}", kernel_time(lambda: ops.moe_gate(gu, share, act, experts, ff, True)),
           T * I * 6, None)
    h_in = rnd(T, H, dtype=torch.bfloat16)
    router, correction = rnd(experts, H), rnd(experts)
    record(f"moe_route, sigmoid scores, 2 of {experts} experts inside 2 of 4 groups, width {H}",
           kernel_time(lambda: ops.moe_route(h_in, router, experts, 2, "one", share, score="sigmoid", correction=correction,
                                             groups=4, keep=2, scale=2.5)), T * H * 2, "moe_route")
    router9 = rnd(experts + 1, H)
    record(f"moe_route, softmax of the chosen (Katopel path), width {H}",
           kernel_time(lambda: ops.moe_route(h_in, router9, experts, 2, True, share)), T * H * 2, None)
    table16, ptable16 = rnd(32000, H, dtype=torch.bfloat16), rnd(T, H, dtype=torch.bfloat16)
    ids = torch.randint(0, 32000, (T,), device=dev, dtype=torch.int32)
    record(f"embed_positions, {T} x {H}", kernel_time(lambda: ops.embed_positions(ids, pos, req, table16, ptable16, x)),
           T * H * (2 + 2 + 4), "embed")
    record(f"embed, {T} x {H}", kernel_time(lambda: ops.embed(ids, table16, x)), T * H * (2 + 4), None)
    # the like kernels of the paths that were there before
    record(f"silu_gate, {T} x {I}", kernel_time(lambda: ops.silu_gate(gu, act)), T * I * 6, None)
    record(f"rms_norm with pending add, {T} x {H}", kernel_time(lambda: ops.rms_norm(x, g1, 1e-6, out16, delta=a16)),
           T * H * (4 + 4 + 2 + 2), None)
    b1 = torch.zeros(H, device=dev)
    record(f"post_norm_add with the next norm (Katopel path), {T} x {H}",
           kernel_time(lambda: ops.post_norm_add(x, [(a16, 1.0)], g1, b1, 1e-6, g1, b1, 1e-6, out16)), T * H * (2 + 4 + 4 + 2), None)
    # the delta rule at the Katopel 2k size: its prepare, scan and output norm
    d_heads, d_groups, d_dim, d_vdim = 16, 8, 128, 128
    d_channels = 2 * d_groups * d_dim + d_heads * d_vdim
    padded = ops.gdn_padded_dim(d_dim)
    d_off = d_heads * d_vdim * padded
    d_slot = -(-(d_off + (taps - 1) * d_channels) // 4) * 4
    d_proj = rnd(T, d_channels + 2 * d_heads + d_heads * d_vdim)
    d_conv = rnd(d_channels, taps)
    qkv, bg = torch.empty(T, d_channels, device=dev), torch.empty(T, 2 * d_heads + d_groups, device=dev)
    o = torch.empty(T, d_heads * d_vdim, device=dev)
    o16 = torch.empty(T, d_heads * d_vdim, dtype=torch.bfloat16, device=dev)
    d_a, d_b = rnd(d_heads), rnd(d_heads)
    for requests in (1, 4):
        state = torch.zeros(requests, d_slot, device=dev)
        spans, slots = ints(T * r // requests for r in range(requests + 1)), ints(range(requests))
        row_req = ints(r for r in range(requests) for _ in range(T // requests))
        record(f"gdn_prepare (Katopel path), {T} tokens of {requests} request(s), {d_channels} channels of {taps} taps",
               kernel_time(lambda: ops.gdn_prepare(d_proj, 0, d_channels, d_channels + d_heads, d_groups, d_heads, d_dim, d_vdim,
                                                   taps, d_conv, d_a, d_b, state, d_off, row_req, spans, slots, qkv, bg)),
               T * (d_channels + 2 * d_heads) * 8, None)
        record(f"gdn_scan (Katopel path), {T} tokens of {requests} request(s), {d_heads} heads of {d_dim} x {d_vdim}",
               kernel_time(lambda: ops.gdn_scan(qkv, bg, d_groups, d_heads, d_dim, d_vdim, state, spans, slots, o,
                                                longest=T // requests)),
               T * (d_channels + 2 * d_heads + d_heads * d_vdim) * 4, None, flops=T * d_heads * d_dim * d_vdim * 8)
    record(f"gdn_out_norm (Katopel path), {T} tokens x {d_heads} heads of {d_vdim}",
           kernel_time(lambda: ops.gdn_out_norm(o, d_proj, d_channels + 2 * d_heads, torch.ones(d_vdim, device=dev), 1.0, 1e-6,
                                                o16, d_heads, d_vdim, row_req)), T * d_heads * d_vdim * (4 + 4 + 2), None)
    state = torch.zeros(rows, d_slot, device=dev)
    spans, slots = ints(range(rows + 1)), ints(range(rows))
    record(f"gdn_scan (Katopel path), {rows} requests of one token",
           kernel_time(lambda: ops.gdn_scan(qkv[:rows], bg[:rows], d_groups, d_heads, d_dim, d_vdim, state, spans, slots, o[:rows])),
           rows * d_off * 8, None)
    ops.raise_if_error()
    print(json.dumps({
        "metric": "prefill and decode tok/s of the Vizonex design beside Katopel at equal width, depth and parameters",
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup, "dtype": "bf16",
        "data": "synthetic: random weights drawn on the device, uniform random token ids",
        "config": {"sizes": VIZONEX_SIZES, "prefill_tokens": PREFILL_TOKENS, "decode_context": context,
                   "peaks": pk["source"], "hbm_gbs": pk["hbm_gbs"],
                   "l2": "kernels alone: inputs larger than L2 and a 256 MB write between timed launches"},
        "models": models, "kernels": kernels}))
    return 0


# ---- the Zobelorn design beside the Qwen2 decoder at equal width, depth, heads and parameter count ----
ZOBELORN_SIZES = {
    # width; attention of `heads` over `kv_heads` heads of dim / vdim lanes: the windowed kind (a window of `window`
    # keys, `rot` rotated lanes, a cap on the scores, a gate on the outputs) and the chunked kind (chunks of `chunk`
    # positions, whole heads rotated; every other one of them borrows the keys and values of the one before);
    # a dense feed-forward of `ff`; experts of which a token uses `top`, and a shared one
    "1k": dict(width=1024, heads=16, kv_heads=4, dim=64, vdim=64, window=1024, chunk=1024, rot=32, softcap=50.0,
               ff=2816, experts=8, top=2, expert_ff=704, shared_ff=1408, vocab=32000, layers=8),
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, chunk=1024, rot=64, softcap=50.0,
               ff=5632, experts=8, top=2, expert_ff=1408, shared_ff=2816, vocab=32000, layers=8),
}


def zobelorn_config(z):
    """Layers in the pattern chunked + dense, windowed + experts, chunked on the first layer's keys + experts,
    windowed + dense, twice."""
    import tokenizer_b200 as tb
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["shared_ff"]}}
    heads = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5}
    windowed = dict(heads, mask={"size": z["window"]}, softcap=z["softcap"],
                    rot={"base": 10000.0, "dims": z["rot"], "scaling": {"factor": 4.0}})
    chunked = dict(heads, mask={"size": z["chunk"]},
                   rot={"base": 500000.0, "dims": z["dim"], "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}})
    layers = []
    for i in range(z["layers"]):
        kind = i % 4
        if kind == 0:
            layers.append({"type": "attention_2", "mixer": chunked, "mlp": dense})
        elif kind == 2:
            layers.append({"type": "attention_2", "mixer": dict(chunked, kv_from=i - 2), "mlp": moe})
        else:
            layers.append({"type": "attention", "mixer": windowed, "mlp": moe if kind == 1 else dense})
    return tb.config.ZobelornConfig.from_dict({
        "architecture": "Zobelorn", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6},
        "embedding": {"scale": 32.0}, "residual_mult": 0.5, "layers": layers})


def run_zobelorn(args):
    """Prefill (one step of 2,048 tokens) and decoding (batch 1 and `--batch`, 2,048-token contexts) of the
    Zobelorn design at two widths, beside the closest model that was there, the Qwen2 decoder (attention in every
    layer, nothing recurrent), at the same width, depth and heads with the feed-forward width that gives it the
    same parameters.  Then the design's own kernels alone beside the like kernels
    of the paths that were there, each on inputs larger than L2, against the measured copy peak; the attention
    kernels with and without the cap on the scores, against one another."""
    import torch
    import tokenizer_b200 as tb
    from tokenizer_b200.kernels import ops
    from tokenizer_b200.parts.attention import RowTiles
    from tokenizer_b200.parts.model import declared_tensors

    torch.cuda.set_device(0)
    pk = peaks()
    gen = torch.Generator().manual_seed(99)
    context, steps = 2048, max(8, min(args.steps, 64))
    timed = device_timed
    count = lambda config: sum(int(torch.tensor(t.shape).prod()) for t in declared_tensors(config.model_spec()))

    def qwen_config(z, inner):
        return tb.Qwen2Config.from_dict(dict(
            architectures=["Qwen2ForCausalLM"], hidden_act="silu", num_hidden_layers=z["layers"],
            hidden_size=z["width"], num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"],
            head_dim=z["dim"], intermediate_size=inner, vocab_size=z["vocab"], rope_theta=1000000.0,
            rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=32768, use_sliding_window=False,
            sliding_window=32768, max_window_layers=z["layers"]))

    models = {}
    for name, z in ZOBELORN_SIZES.items():
        if args.only_kernels:
            break
        config = zobelorn_config(z)
        models[name] = {"zobelorn": measure_design(config, z["vocab"], args, gen, context, steps)}
        # the gated feed-forward width (whole 128s) that brings Qwen2 to the same parameters
        base, step = count(qwen_config(z, 128)), count(qwen_config(z, 256)) - count(qwen_config(z, 128))
        inner = max(1, round((count(config) - base) / step) + 1) * 128
        models[name]["qwen2"] = dict(measure_design(qwen_config(z, inner), z["vocab"], args, gen, context, steps),
                                     intermediate_size=inner)

    # ---- kernels alone: inputs larger than L2, a 256 MB write between the timed launches ----
    dev = "cuda:0"
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)

    def kernel_time(fn, reps=7):
        times = []
        for _ in range(3 + reps):
            flush.zero_()
            ms, _ = timed(fn)
            times.append(ms)
        return sorted(times[3:])[reps // 2]

    kernels = {}

    def record(name, ms, nbytes, like, flops=None):
        kernels[name] = {"us": round(ms * 1e3, 1), "gb_s": round(nbytes / (ms / 1e3) / 1e9), "like": like,
                         "of_measured_copy_peak": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 2)}
        if flops is not None:
            kernels[name]["bf16_tflops"] = round(flops / (ms / 1e3) / 1e12, 1)

    rnd = lambda *shape, dtype=torch.float32: torch.randn(*shape, device=dev, dtype=torch.float32).to(dtype)
    T, H, I = 8192, 2048, 5632
    # the norm behind a sublayer, the add and the next norm; beside it the pre-norm path's norm with its pending add
    x, a16 = rnd(T, H), rnd(T, H, dtype=torch.bfloat16)
    g1 = torch.ones(H, device=dev)
    out16 = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    record(f"post_norm_add, RMS form with the next norm, {T} x {H} (bfloat16 term)",
           kernel_time(lambda: ops.post_norm_add(x, [(a16, 1.0)], g1, None, 1e-6, g1, None, 1e-6, out16, rms=True, next_rms=True)),
           T * H * (2 + 4 + 4 + 2), "rms_norm with pending add")
    parts = rnd(2, T, H)
    record(f"post_norm_add, RMS form with the next norm, {T} x {H} (two float32 partial sums)",
           kernel_time(lambda: ops.post_norm_add(x, [(parts, 1.0)], g1, None, 1e-6, g1, None, 1e-6, out16, rms=True, next_rms=True)),
           T * H * (8 + 4 + 4 + 2), "rms_norm with pending add")
    record(f"rms_norm with pending add, {T} x {H}", kernel_time(lambda: ops.rms_norm(x, g1, 1e-6, out16, delta=a16)),
           T * H * (4 + 4 + 2 + 2), None)
    b1 = torch.zeros(H, device=dev)
    record(f"post_norm_add, layer-norm form with the next norm (Katopel path), {T} x {H}",
           kernel_time(lambda: ops.post_norm_add(x, [(a16, 1.0)], g1, b1, 1e-6, g1, b1, 1e-6, out16)), T * H * (2 + 4 + 4 + 2), None)
    del parts
    # queries, keys and values: both kinds of layer, a layer of queries alone, the Katopel path beside them
    nh, nkv, d = 16, 4, 128
    wide = rnd(T, (nh + 2 * nkv) * d + nh * d)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    req = torch.zeros(T, dtype=torch.int32, device=dev)
    q_out = torch.empty(T, nh * d, dtype=torch.bfloat16, device=dev)
    k_pool = torch.zeros(T + 64, nkv, d, dtype=torch.bfloat16, device=dev)
    v_pool = torch.zeros_like(k_pool)
    qg, kg = torch.ones(nh * d, device=dev), torch.ones(nkv * d, device=dev)
    # frequencies in 64-bit, as the position part hands them over (the angle is then formed in 64-bit)
    freq64 = torch.tensor([1e6 ** (-2.0 * i / 64) for i in range(32)], dtype=torch.float64, device=dev)
    freq128 = torch.tensor([5e5 ** (-2.0 * i / 128) for i in range(64)], dtype=torch.float64, device=dev)
    qkv_bytes = T * (nh + 2 * nkv) * d * (4 + 2)
    record(f"qkv_rotate_store, whole-projection norms and 64 lanes rotated by halves, {T} tokens, {nh} heads over {nkv} of {d}",
           kernel_time(lambda: ops.qkv_rotate_store(wide, 0, None, freq64, 64, pos, pos, req, q_out, k_pool, v_pool, nh, nkv, d, d, d,
                                                    q_gain=qg, k_gain=kg, eps=1e-6, layout="half")), qkv_bytes, "qkv_rotate_store")
    record(f"qkv_rotate_store, whole heads rotated in pairs and a norm a head, {T} tokens",
           kernel_time(lambda: ops.qkv_rotate_store(wide, 0, None, freq128, 128, pos, pos, req, q_out, k_pool, v_pool, nh, nkv, d, d,
                                                    d, head_norm_eps=1e-6)), qkv_bytes, "qkv_rotate_store")
    record(f"qkv_rotate_store, queries alone with a norm a head, {T} tokens",
           kernel_time(lambda: ops.qkv_rotate_store(wide, 0, None, freq128, 128, pos, None, req, q_out, None, None, nh, 0, d, d, d,
                                                    head_norm_eps=1e-6)), T * nh * d * (4 + 2), "qkv_rotate_store")
    bias = torch.zeros((nh + 2 * nkv) * d, device=dev)
    record(f"qkv_rotate_store, biases and 64 rotated lanes (Katopel path), {T} tokens",
           kernel_time(lambda: ops.qkv_rotate_store(wide, 0, bias, freq64, 64, pos, pos, req, q_out, k_pool, v_pool, nh, nkv, d, d, d)),
           qkv_bytes, None)
    mixed16 = rnd(T, nh * d, dtype=torch.bfloat16)
    record(f"attention_gate, {T} tokens x {nh} heads of {d}",
           kernel_time(lambda: ops.attention_gate(mixed16, wide, (nh + 2 * nkv) * d, nh, d, d)), T * nh * d * (4 + 2 + 2), "silu_gate")
    experts, ff, top = 8, 512, 2
    gu = rnd(T, 2 * I, dtype=torch.bfloat16)
    share = torch.zeros(T, experts + 1, device=dev)
    act = torch.empty(T, I, dtype=torch.bfloat16, device=dev)
    h_in = rnd(T, H, dtype=torch.bfloat16)
    router = rnd(experts, H)
    record(f"moe_route, sigmoid scores, {top} of {experts} experts, width {H}",
           kernel_time(lambda: ops.moe_route(h_in, router, experts, top, "one", share, score="sigmoid")), T * H * 2, "moe_route")
    router9 = rnd(experts + 1, H)
    share9 = torch.zeros(T, experts + 1, device=dev)
    record(f"moe_route, softmax of the chosen (Katopel path), width {H}",
           kernel_time(lambda: ops.moe_route(h_in, router9, experts, top, True, share9)), T * H * 2, None)
    record(f"moe_gate, weights on the experts' input, {T} x {I} lanes of {experts} experts and a shared one",
           kernel_time(lambda: ops.moe_gate(gu, share, act, experts, ff, True, on_input=True)), T * I * 6, "moe_gate")
    record(f"moe_gate, weights on the output (Katopel path), {T} x {I}",
           kernel_time(lambda: ops.moe_gate(gu, share, act, experts, ff, True)), T * I * 6, None)
    record(f"silu_gate, {T} x {I}", kernel_time(lambda: ops.silu_gate(gu, act)), T * I * 6, None)
    del gu, act, wide, mixed16
    # attention with and without the cap: 8,192-token prompt portions of four requests (the tcgen05 and the mma.sync
    # kernels), then 64 rows of one token over 8,192 keys (the split-key kernel), 16 heads over 4 of 128 lanes
    page, n_req, n_keys = 16, 4, 8192
    pages_each = n_keys // page
    k_pool = rnd(n_req * n_keys, nkv, d, dtype=torch.bfloat16)
    v_pool = rnd(n_req * n_keys, nkv, d, dtype=torch.bfloat16)
    table = torch.arange(n_req * pages_each, dtype=torch.int32, device=dev).view(n_req, pages_each)
    portion = 2048
    q = rnd(n_req * portion, nh * d, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    row_req = torch.arange(n_req, dtype=torch.int32, device=dev).repeat_interleave(portion)
    pos = (torch.arange(portion, dtype=torch.int32, device=dev) + (n_keys - portion)).repeat(n_req)
    import numpy as np
    for kernel, run, rows in (("attention_tcgen05", ops.attention_tcgen05, ops.WIDE_TILE_ROWS),
                              ("prefill_attention", ops.prefill_attention, ops.PREFILL_TILE_ROWS)):
        note = RowTiles(rows)
        words = np.zeros(note.capacity(n_req * portion, n_req), dtype=np.int32)
        n_tiles = note.fill(words, np.arange(n_req, dtype=np.int32) * portion, np.full(n_req, portion, dtype=np.int32),
                            np.full(n_req, n_keys - portion, dtype=np.int32), False)
        tiles = torch.tensor(words, device=dev).view(-1, 2)
        window = 1023
        # a row of the portion reads the 1,024 keys of its window: two products of 2 * d a key and head
        flops = n_req * portion * nh * 1024 * 4 * d
        for cap in (None, 50.0):
            record(f"{kernel}, {n_req} portions of {portion} rows, a window of 1,024 keys, " + ("capped" if cap else "no cap"),
                   kernel_time(lambda: run(q, k_pool, v_pool, out, table, row_req, pos, tiles, n_tiles, nh, nkv, d, page, window,
                                           d ** -0.5, softcap=cap)), 0, None if cap is None else kernel + ", no cap", flops=flops)
    rows = 64
    big_k = rnd(rows * n_keys, nkv, d, dtype=torch.bfloat16)
    big_v = rnd(rows * n_keys, nkv, d, dtype=torch.bfloat16)
    table = torch.arange(rows * pages_each, dtype=torch.int32, device=dev).view(rows, pages_each)
    q1 = rnd(rows, nh * d, dtype=torch.bfloat16)
    out1 = torch.empty_like(q1)
    req1 = torch.arange(rows, dtype=torch.int32, device=dev)
    pos1 = torch.full((rows,), n_keys - 1, dtype=torch.int32, device=dev)
    for cap in (None, 50.0):
        record(f"decode_attention, {rows} rows x {n_keys} keys, " + ("capped" if cap else "no cap"),
               kernel_time(lambda: ops.decode_attention(q1, big_k, big_v, out1, table, req1, pos1, nh, nkv, d, page, None,
                                                        d ** -0.5, softcap=cap)), rows * n_keys * nkv * d * 4,
               None if cap is None else "decode_attention, no cap")
    ops.raise_if_error()
    print(json.dumps({
        "metric": "prefill and decode tok/s of the Zobelorn design beside Qwen2 at equal width, depth, heads and parameters",
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup, "dtype": "bf16",
        "data": "synthetic: random weights drawn on the device, uniform random token ids",
        "config": {"sizes": ZOBELORN_SIZES, "prefill_tokens": PREFILL_TOKENS, "decode_context": context,
                   "peaks": pk["source"], "hbm_gbs": pk["hbm_gbs"],
                   "l2": "kernels alone: inputs larger than L2 and a 256 MB write between timed launches"},
        "models": models, "kernels": kernels}))
    return 0


def run_mixed(args):
    """BASELINE.json configs[3]: 32 requests at Qwen2.5-1.5B sizes, prompt lengths uniform in
    [64, 2048] from a fixed seed, 128 new tokens each, continuous batching under a budget of 512
    tokens a step, half of the prompts beginning with one of four shared beginnings of 256 tokens
    (whole pages, taken over from the first request that computed them).  Host tokens in, host
    ids out; the run is timed by the wall clock between two device synchronisations."""
    import torch
    import tokenizer_b200 as tb

    torch.cuda.set_device(0)
    layers = args.layers if args.layers != SIZES["num_hidden_layers"] else SIZES_1_5B["num_hidden_layers"]
    gate = None if args.skip_gate else gate_on_logits(SIZES_1_5B, "1.5B layer sizes")
    cfg = full_config(SIZES_1_5B, layers)
    config = tb.Qwen2Config.from_dict(cfg)
    pk = peaks()
    model = tb.random_model(config, seed=2, dtype="bfloat16", device="cuda:0")
    n_requests, new_tokens, budget, shared_len = 32, 128, 512, 256

    def workload(token_seed, seed=1234):
        """Lengths and the choice of beginnings from `seed`, every token from `token_seed`: runs on
        different tokens have the same shapes of steps and share nothing with each other."""
        gen = torch.Generator().manual_seed(seed)
        lengths = torch.randint(64, 2049, (n_requests,), generator=gen).tolist()
        gen = torch.Generator().manual_seed(token_seed)
        beginnings = [torch.randint(0, config.vocab_size, (shared_len,), generator=gen).tolist() for _ in range(4)]
        prompts = []
        for i, n in enumerate(lengths):
            ids = torch.randint(0, config.vocab_size, (n,), generator=gen).tolist()
            if i % 2 == 0:                         # every other request starts with a shared beginning
                ids = (beginnings[(i // 2) % 4] + ids)[:max(n, shared_len + 1)]
            prompts.append(ids)
        return prompts

    def serve(share):
        """An engine as a server keeps it (its captured steps live with it), and a function that
        runs a workload through a fresh scheduler on it."""
        pool = n_requests * (2048 + shared_len + new_tokens + PAGE)
        engine = tb.engine_for(model, pool, PAGE, max_requests=n_requests, share_prefixes=share)

        def run(prompts):
            scheduler = tb.Scheduler(engine, max_batch_size=n_requests, token_budget=budget)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ids = [scheduler.add_request(p, tb.GenerateParams.greedy(new_tokens)) for p in prompts]
            finished = scheduler.run()
            torch.cuda.synchronize()
            seconds = time.perf_counter() - t0
            engine.check()
            assert all(len(finished[i].tokens) == new_tokens for i in ids)
            return seconds, scheduler.stats, engine
        return run

    run = serve(True)
    run(workload(7))                                # warm-up on other tokens: compiles, captures the steps' shapes
    clocks = ClockSampler()
    clocks.start()
    time.sleep(0.25)
    # five runs, each on tokens of its own (nothing is shared between runs); the median stands: a
    # run is some 200 steps that the host packs, and a shared host disturbs some of them
    workloads = [workload(1234 + i) for i in range(5)]
    samples = sorted((run(w) + (w,) for w in workloads), key=lambda r: r[0])
    seconds, stats, engine, prompts = samples[len(samples) // 2]
    clock_record = clocks.stop()
    run_private = serve(False)
    run_private(workload(7))
    samples_private = sorted((run_private(w) for w in workloads), key=lambda r: r[0])
    seconds_private, stats_private, _ = samples_private[len(samples_private) // 2]
    prompt_tokens = sum(len(p) for p in prompts)
    # the least a device of the measured peaks would take: every step reads the weights once,
    # every decoded token its request's keys and values; every token run costs its products
    # and its attention over the keys before it
    h, d = cfg["hidden_size"], cfg["head_dim"]
    q, kv, inner = cfg["num_attention_heads"] * d, cfg["num_key_value_heads"] * d, cfg["intermediate_size"]
    per_token_linear = 2 * layers * ((q + 2 * kv) * h + h * q + 3 * inner * h)
    flops = stats.tokens_run * per_token_linear + n_requests * new_tokens * 2 * h * cfg["vocab_size"]
    kv_read = 0
    for p in prompts:
        flops += layers * 4 * q * (len(p) + new_tokens) ** 2 / 2
        kv_read += sum(len(p) + i for i in range(new_tokens)) * kv_bytes_per_token(cfg, layers)
    bytes_read = stats.steps * weight_bytes(cfg, layers) + kv_read
    bound_s = max(bytes_read / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops_sustained"] * 1e12))
    line = {
        "metric": "generated tok/s (Qwen2.5-1.5B sizes, 32 requests, prompts U[64,2048], 128 new tokens, "
                  "512-token budget, shared beginnings)",
        "value": n_requests * new_tokens / seconds, "unit": "tokens/s", "n_gpus": 1, "steps": stats.steps,
        "warmup": 1, "runs": 5, "ms_per_step": 1e3 * seconds / stats.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights drawn on the device (seed 2), uniform random token ids (seed 1234)",
        "config": {"model": "Qwen2.5-1.5B sizes", "layers": layers,
                   "layers_of_config": SIZES_1_5B["num_hidden_layers"], "hidden": h,
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": d,
                   "intermediate": inner, "vocab": cfg["vocab_size"], "requests": n_requests,
                   "prompt_tokens": prompt_tokens, "new_tokens": new_tokens, "token_budget": budget,
                   "page_size": PAGE, "parallelism": "single GPU", "peaks": pk["source"], "logits_gate": gate,
                   "plain_products_of_65_rows_and_more": products_note()},
        "clocks": clock_record,
        "mixed": {"seconds": seconds, "total_tok_s": (prompt_tokens + n_requests * new_tokens) / seconds,
                  "tokens_run": stats.tokens_run, "shared_prefix_tokens": stats.shared_prefix_tokens,
                  "preemptions": stats.preemptions, "max_running": stats.max_running,
                  "peak_pages": stats.peak_pages, "steps_fed_on_device": engine.steps_fed_on_device,
                  "seconds_of_5_runs": [round(r[0], 4) for r in samples],
                  "seconds_without_sharing": seconds_private,
                  "seconds_without_sharing_of_5_runs": [round(r[0], 4) for r in samples_private], "tokens_run_without_sharing": stats_private.tokens_run,
                  "bound_seconds": bound_s, "frac": bound_s / seconds},
        "e2e": {"value": n_requests * new_tokens / seconds, "unit": "tokens/s",
                "h2d_bytes_per_step": engine.builder.last_bytes, "d2h_bytes_per_step": 4 * n_requests,
                "note": "the run IS end to end: host prompts in, host ids out, through Scheduler"},
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
