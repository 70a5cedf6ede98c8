#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-MoE engine on ONE B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of the LLaMA-MoE-3.5B (4/16) shape (32 layers, width 4096,
32/32 heads of 128, 16 experts top-4 of width 688, vocabulary 32000, context 4096) with random
bfloat16 weights, a batch of 8 and prompt lengths uniform in [128, 2048].  A "step" is one decode
step.  It prints ONE JSON line:

  value      decoded tokens a second: regions of exactly K steps each, timed on the device with CUDA
             events, repeated until at least a second has been timed; the median region counts
             (ms_per_step, with the fastest and slowest region under "spread"); the sampled tokens
             stay on the device between steps
  e2e        the same through transformer_b200.generate (as many steps as all regions together): host
             token lists in and out, the step's index arrays copied from pinned memory and the
             sampled tokens read back at every step
  prefill    one sequence of 2,048 tokens; frac = flops / time / the measured bf16 peak
  roofline   bytes the decode step has to read (every weight it uses once, the cache of the live
             requests) / its time, against the measured copy bandwidth
  points     decode tokens a second at batch 1 (a prompt of 1,088 tokens, the mean of the range) and
             64, each with its mean context, distinct experts per layer, fraction of the copy
             bandwidth and end-to-end figure

Every timed step reads far more than the 126 MB of L2 (all weights), so no L2 flush is needed.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE = {   # BASELINE.json configs[2]
    "model_type": "llama", "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 32, "head_dim": 128, "intermediate_size": 688, "num_local_experts": 16,
    "num_experts_per_tok": 4, "max_position_embeddings": 4096, "vocab_size": 32000, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "tie_word_embeddings": False,
}
FULL_LAYERS = 32
PROMPT_MIN, PROMPT_MAX = 128, 2048
PREFILL_TOKENS = 2048
# The other shapes BASELINE.json names (configs[3], configs[4]); not the default and not the headline: further sizes
# for the same kernels.  name -> (config, layers of the full model, prompt length range)
OTHER_SHAPES = {
    "mixtral-8x7b": ({
        "model_type": "llama", "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "num_local_experts": 8,
        "num_experts_per_tok": 2, "max_position_embeddings": 32768, "vocab_size": 32000, "rms_norm_eps": 1e-5,
        "rope_theta": 1e6, "tie_word_embeddings": False}, 32, (512, 8192)),
    "mixtral-8x22b": ({
        "model_type": "llama", "num_hidden_layers": 16, "hidden_size": 6144, "num_attention_heads": 48,
        "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 16384, "num_local_experts": 8,
        "num_experts_per_tok": 2, "max_position_embeddings": 65536, "vocab_size": 32768, "rms_norm_eps": 1e-5,
        "rope_theta": 1e6, "tie_word_embeddings": False}, 56, (1, 16384)),
}
MIN_TIMED_SECONDS = 1.0     # the K-step region is repeated until this much has been timed
MAX_REGIONS = 40


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class Clocks:
    """nvidia-smi sampling in the background while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid=None):
        """uuid: of the device the process runs on (cuda:0 of this process is rarely index 0 of a shared box)."""
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        self.gpu = f"GPU-{uuid}" if uuid else "0"

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu, f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()     # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.file.close()
        os.unlink(self.file.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def prefill_flops(c, T):
    L, d, nh, nkvh, dh = c["num_hidden_layers"], c["hidden_size"], c["num_attention_heads"], \
        c["num_key_value_heads"], c["head_dim"]
    E, k, di, V = c["num_local_experts"], c["num_experts_per_tok"], c["intermediate_size"], c["vocab_size"]
    per_layer = 2 * T * d * (nh + 2 * nkvh) * dh + 2 * T * nh * dh * d + 2 * T * d * E + 2 * T * k * 3 * d * di \
        + 4 * nh * dh * T * (T + 1) // 2
    return L * per_layer + 2 * d * V


def decode_bytes(c, distinct_experts_per_layer, context_tokens, elem=2):
    """Bytes one decode step must read: every weight it uses once + the cache of the live requests."""
    L, d, nh, nkvh, dh = c["num_hidden_layers"], c["hidden_size"], c["num_attention_heads"], \
        c["num_key_value_heads"], c["head_dim"]
    E, di, V = c["num_local_experts"], c["intermediate_size"], c["vocab_size"]
    fixed = L * (d * (nh + 2 * nkvh) * dh + nh * dh * d + E * d) * elem + L * 2 * d * 4 + d * 4 + V * d * elem
    experts = sum(distinct_experts_per_layer) * 3 * d * di * elem
    cache = L * context_tokens * 2 * nkvh * dh * elem
    return fixed + experts + cache


def main():
    global PROMPT_MIN, PROMPT_MAX, PREFILL_TOKENS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers of the same sizes (named in config)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--skip-points", action="store_true", help="leave out the batch 1 / 64 points")
    ap.add_argument("--shape", default="llama-moe-3.5b", choices=["llama-moe-3.5b", *OTHER_SHAPES],
                    help="layer sizes: the benchmark's (default) or another shape BASELINE.json names")
    ap.add_argument("--prompt-max", type=int, default=0, help="longest prompt drawn (default: the shape's own)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS)
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "YdrMaster/transformer is a Rust workspace with git dependencies: no Rust toolchain, no "
                          "network and no Python package to install here (pip finds no setup.py or pyproject.toml)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this library does no work on several GPUs (asked for {args.gpus})")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import transformer_b200 as tb
    from transformer_b200.csrc import lib
    from transformer_b200.sampling import Sampler

    pk = peaks()
    shape, full_layers = SHAPE, FULL_LAYERS
    if args.shape != "llama-moe-3.5b":
        shape, full_layers, (PROMPT_MIN, PROMPT_MAX) = OTHER_SHAPES[args.shape]
        if args.layers == FULL_LAYERS:
            args.layers = shape["num_hidden_layers"]
    if args.prompt_max:
        PROMPT_MAX = max(PROMPT_MIN, args.prompt_max)
    PREFILL_TOKENS = args.prefill_tokens
    cfg = dict(shape, num_hidden_layers=args.layers)
    K, W, B = args.steps, args.warmup, args.batch
    gen = torch.Generator().manual_seed(1234)

    def lengths(n):
        return torch.randint(PROMPT_MIN, PROMPT_MAX + 1, (n,), generator=gen).tolist()

    def prompts_of(lens):
        return [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lens]

    batches = {B: lengths(B)}
    if not args.skip_points:
        batches.setdefault(1, [(PROMPT_MIN + PROMPT_MAX) // 2])     # one sequence: the mean of the range, not a draw
        batches.setdefault(64, lengths(64))
    # steps a run may take: warm-up and the regions (a second of them: some 500 steps of one sequence, 100 of 64)
    def most_steps(b):
        budget = max(K, 640 if b <= 16 else 160)
        return min(W + 2 + min(MAX_REGIONS * K, budget), cfg["max_position_embeddings"] - PROMPT_MAX - 8)
    room = max(sum((n + most_steps(len(ls)) + 8 + 63) // 64 * 64 for n in ls) for ls in batches.values())
    room = max(room, (PREFILL_TOKENS + 63) // 64 * 64)
    engine = tb.random_model(cfg, seed=0, dtype=args.dtype, max_tokens=room, max_slots=max(batches) + 1)
    sampler = Sampler(engine.device)
    greedy = tb.SampleArgs()
    dev = engine.device

    # ---- prefill of 2,048 tokens ---------------------------------------------------------------
    ptoks = prompts_of([PREFILL_TOKENS])[0]
    times = []
    for i in range(3 + 5):
        s = engine.open()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step([s], [ptoks])
        e1.record()
        torch.cuda.synchronize()
        engine.close(s)
        if i >= 3:
            times.append(e0.elapsed_time(e1))
    p_ms = statistics.median(times)
    p_flops = prefill_flops(cfg, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (p_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": p_ms,
               "frac": p_flops / (p_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}

    # ---- decode ----------------------------------------------------------------------------------
    def decode_run(lens, with_clocks):
        b = len(lens)
        prompts = prompts_of(lens)
        slots = [engine.open() for _ in range(b)]
        logits = engine.step(slots, prompts)
        ids, _ = sampler.sample(logits, greedy)
        ids = ids.clone()
        shape = [[0]] * b

        def one():
            lg = engine.step(slots, shape, device_tokens=ids)
            nxt, _ = sampler.sample(lg, greedy)
            ids.copy_(nxt)

        # which experts does a step use?  (one eager step with the recorder, outside the timing)
        chosen = []
        engine.recorder = lambda name, run, t: chosen.append(t) if name == "moe.topk_idx" else None
        engine.use_graphs = False
        one()
        engine.use_graphs = True
        engine.recorder = None
        distinct = [int(torch.unique(t).numel()) for t in chosen]
        for _ in range(W):
            one()
        torch.cuda.synchronize()
        uuid = getattr(torch.cuda.get_device_properties(dev), "uuid", None)
        clk = Clocks(uuid)
        if with_clocks:
            clk.start()
            time.sleep(0.3)
        n0 = lib.launch_count
        regions, ctx_sum, steps_left = [], 0, most_steps(b) - W - 2
        while (sum(regions) < MIN_TIMED_SECONDS * 1e3 or not regions) and len(regions) < MAX_REGIONS and steps_left >= K:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            before = sum(engine.cache.length(s) for s in slots)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(K):
                one()
            e1.record()
            torch.cuda.synchronize()
            regions.append(e0.elapsed_time(e1))
            ctx_sum += before + b * (K // 2)          # the region's mean context
            steps_left -= K
        launches = (lib.launch_count - n0) // len(regions)
        clocks = clk.stop() if with_clocks else None
        ms = statistics.median(regions)
        ctx_tokens = ctx_sum / len(regions)
        for s in slots:
            engine.close(s)
        # end to end through the public entry point: the same prompts, and as many decode steps as the device-timed
        # regions had in all (K of them would be a tenth of a second, mostly the clocks' recovery from the prompts)
        res = tb.generate(engine, prompts, max_steps=W + 1, stop_tokens=())        # warm-up
        res = tb.generate(engine, prompts, max_steps=K * len(regions) + 1, stop_tokens=())
        return {"tok_s": b * K / (ms * 1e-3), "ms_per_step": ms / K, "launches": launches, "clocks": clocks,
                "bytes": decode_bytes(cfg, distinct, ctx_tokens, 2 if args.dtype == "bfloat16" else 4),
                "distinct": sum(distinct) / max(1, len(distinct)), "ctx": ctx_tokens / b,
                "spread": [min(regions) / K, max(regions) / K], "regions": len(regions),
                "e2e": res.timing.decode_tokens / res.timing.decode_seconds,
                "h2d": int(getattr(engine, "last_h2d_bytes", 0))}

    main_run = decode_run(batches[B], True)
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            r = main_run if b == B else decode_run(batches[b], False)
            points[f"decode_b{b}"] = r["tok_s"]
            points[f"decode_b{b}_hbm_frac"] = r["bytes"] / (r["ms_per_step"] * 1e-3) / 1e9 / pk["hbm_gbs"]
            points[f"decode_b{b}_ms"] = r["ms_per_step"]
            points[f"decode_b{b}_mean_context"] = round(r["ctx"], 1)
            points[f"decode_b{b}_distinct_experts"] = round(r["distinct"], 2)
            points[f"decode_b{b}_e2e"] = r["e2e"]
    e2e_tok_s, h2d = main_run["e2e"], main_run["h2d"]

    achieved = main_run["bytes"] / (main_run["ms_per_step"] * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {B} ({'LLaMA-MoE-3.5B' if args.shape == 'llama-moe-3.5b' else args.shape} shape)",
        "value": main_run["tok_s"], "unit": "tokens/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": main_run["ms_per_step"], "higher_is_better": True,
        "spread": {"regions_of_k_steps": main_run["regions"], "ms_per_step_fastest": main_run["spread"][0],
                   "ms_per_step_slowest": main_run["spread"][1]},
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random weights ~N(0, 0.02) (counter-based, filled on the device), uniform-random token ids", "impl": "ours",
        "config": {
            "model": args.shape + "-shape", "layers": args.layers, "layers_full": full_layers,
            "width": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "experts": cfg["num_local_experts"],
            "experts_per_tok": cfg["num_experts_per_tok"], "expert_ffn": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "context": cfg["max_position_embeddings"], "global_batch": B, "prompt_len_min": PROMPT_MIN,
            "prompt_len_max": PROMPT_MAX, "mean_context": round(main_run["ctx"], 1), "seq_len": 1,
            "parallelism": "none", "l2": "every step reads all weights, far more than L2",
        },
        "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B + 4},
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"],
                     "distinct_experts_per_layer": round(main_run["distinct"], 2)},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
