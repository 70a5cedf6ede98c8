"""Tiny configurations and helpers shared by the tests.

Two configurations of the architecture that differ in every size and option: heads and groups
(GQA with 2 groups / MQA), head size, width and vocabulary (B's are no powers of two), layers,
experts and experts per token, feed-forward width, epsilon, rope base and pairing, tied head.

Weights are drawn with a standard deviation of 0.1 by default, not 0.02: at these widths 0.02
gives attention scores near 1e-3, a flat softmax, and a model that would not notice a wrong mask
or position.  The 0.02 workloads are run once as well (test_engine_gpu.py, test_published_workloads).
"""
import json
import os
import subprocess
import sys

import numpy as np
import torch

from plain import llama_moe_plain as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TINY_A = {
    "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "num_local_experts": 4,
    "num_experts_per_tok": 2, "max_position_embeddings": 128, "vocab_size": 256, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "tie_word_embeddings": False, "rope_pairing": "adjacent",
}
TINY_B = {
    "model_type": "llama", "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 80, "num_local_experts": 6,
    "num_experts_per_tok": 3, "max_position_embeddings": 256, "vocab_size": 384, "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0, "tie_word_embeddings": True, "rope_pairing": "half",
}
# A third one for the dense feed-forward and a head size that is no power of two.
TINY_DENSE = {
    "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 2,
    "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 72, "max_position_embeddings": 160,
    "vocab_size": 200, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
}
# A head size and prompt lengths that reach the tensor-core prompt kernels (attention with heads of 64,
# expert products over more than 512 (token, expert) pairs).
TINY_C = {
    "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 88, "num_local_experts": 5,
    "num_experts_per_tok": 2, "max_position_embeddings": 512, "vocab_size": 320, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "tie_word_embeddings": False,
}
CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 2), "dense": (TINY_DENSE, 5), "C": (TINY_C, 7)}

FP32_TOL = 1e-4          # absolute, on logits of order one
BF16_REL_TOL = 2.0 ** -6  # of the largest |logit| of the request


def as_bfloat16(x):
    """The rounding of the bfloat16 path where it stores an activation (``store=`` of the plain implementation)."""
    return x.bfloat16().to(x.dtype)


def make_folder(tmp, name, std=0.1, dtype="bfloat16"):
    import transformer_b200 as tb
    cfg, seed = CONFIGS[name]
    folder = os.path.join(str(tmp), f"tiny_{name}_{dtype}_{std}")
    if not os.path.isdir(folder):
        tb.write_random_model(folder, cfg, seed=seed, dtype=dtype, std=std)
    return folder


def random_prompts(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def n_moe_layers(cfg):
    return cfg["num_hidden_layers"] if cfg.get("num_local_experts", 0) else 0


def check_request(cfg, tensors, tokens, got_rows, routes, dtype, label="", store=None, logit_tol=None):
    """Compare logits of one request with the plain implementation.

    got_rows: {position: float logits row}.  routes: None, or int array [moe layers, len(tokens), k]
    of the experts the engine chose.  Where the engine's set of experts differs from the plain
    implementation's free choice, the plain gap between the k-th and (k+1)-th router logit must be
    small against the rounding of the path (top-k is discontinuous; a near-tie may fall either way
    and is then forced, not forgiven: a flip over a clear gap fails).

    The yardstick of the bfloat16 path is the plain implementation rounding to bfloat16 where the engine stores
    an activation (sums, softmax, norms and the residual stream stay exact): it predicts what a bfloat16 path
    computes up to the order of its sums, so it lies two to ten times closer to a right engine than the
    unrounded one and a wrong engine stands out the more.  The rule itself is the same for both."""
    if store is None and dtype == "bfloat16":
        store = as_bfloat16
    forced = None
    if routes is not None and len(routes):
        forced = [[[int(e) for e in routes[l][a]] for a in range(len(tokens))] for l in range(len(routes))]
    margins = []
    ref = P.forward(cfg, tensors, tokens, forced_routes=forced, margins_out=margins, store=store)
    if forced is not None:
        # the same rule as for the logits below: a number computed on the bfloat16 path may be off
        # by BF16_REL_TOL of the largest magnitude of its row; a gap is the difference of two
        for l, layer_m in enumerate(margins):
            for a, (free, gap, biggest) in enumerate(layer_m):
                if set(free) != set(forced[l][a]):
                    gap_tol = 2 * BF16_REL_TOL * biggest if dtype == "bfloat16" else 2 * FP32_TOL
                    assert gap <= gap_tol, (
                        f"{label}: layer {l} token {a}: engine chose {forced[l][a]}, plain {free}, "
                        f"over a clear gap {gap:.3e} (largest router logit {biggest:.3e})")
    tol = FP32_TOL if dtype == "float32" else BF16_REL_TOL * float(ref.abs().max())
    if logit_tol is not None:
        tol = logit_tol(float(ref.abs().max()))
    worst = 0.0
    for pos, row in sorted(got_rows.items()):
        diff = float((torch.as_tensor(row) - ref[pos]).abs().max())
        worst = max(worst, diff)
        assert diff <= tol, f"{label}: position {pos} (first wrong of the request): |diff| {diff:.3e} > {tol:.3e}"
    return worst


def check_generation(engine, cfg, tensors, prompts, tokens, batches, dtype, sample=None):
    """Check what ``generate`` produced, through the engine's own step function and the plain implementation.

    The batches are replayed teacher-forced on the generated tokens, step for step as generation ran them (prompts
    together, then one token each), eagerly so that the chosen experts can be recorded.  The replayed logits are
    the ones generation saw, bit for bit (same batch, same kernels; graphs equal eager steps), so:
      * greedy: every generated token is exactly the argmax (lowest id on ties) of the replayed logits;
      * sampled (``sample`` = (SampleArgs, {request: [u per token]})): the token is the one whose interval of the
        distribution of the replayed logits holds u;
      * the replayed logits equal the plain implementation's at every position, under the rule of the path, with the
        routing-tie protocol of :func:`check_request`.
    Every request must have generated the same number of tokens (no stop tokens)."""
    rec = []
    graphs, engine.use_graphs = engine.use_graphs, False
    engine.recorder = lambda name, run, t: rec.append(t.cpu()) if name == "moe.topk_idx" else None
    n_moe = n_moe_layers(cfg)
    try:
        for batch in batches:
            n_new = len(tokens[batch[0]])
            assert all(len(tokens[r]) == n_new for r in batch)
            slots = [engine.open() for _ in batch]
            rows = {r: {} for r in batch}
            routes = {r: {} for r in batch}
            for j in range(n_new):
                feed = [list(prompts[r]) if j == 0 else [tokens[r][j - 1]] for r in batch]
                lg = engine.step(slots, feed).cpu()
                rt = torch.stack(rec) if n_moe else None           # [layers, tokens of the step, k]
                rec.clear()
                at = 0
                for i, r in enumerate(batch):
                    pos = len(prompts[r]) + j - 1
                    rows[r][pos] = lg[i]
                    for a in range(len(feed[i])):
                        if rt is not None:
                            routes[r][pos - len(feed[i]) + 1 + a] = rt[:, at + a, :]
                    at += len(feed[i])
                    tok = tokens[r][j]
                    if sample is None or sample[0].greedy:
                        assert tok == int(torch.argmax(lg[i])), f"request {r}, token {j}: {tok} is not the argmax"
                    else:
                        args, us = sample
                        kept, probs = P.sample_distribution(lg[i], args.temperature, args.top_k, args.top_p)
                        assert tok in kept, f"request {r}, token {j}: {tok} is outside the kept set"
                        lo = sum(probs[:kept.index(tok)])
                        assert lo - 1e-4 <= us[r][j] <= lo + probs[kept.index(tok)] + 1e-4, \
                            f"request {r}, token {j}: u = {us[r][j]} misses the interval of {tok}"
            for s in slots:
                engine.close(s)
            for r in batch:
                seq = list(prompts[r]) + list(tokens[r][:-1])
                rt = None
                if n_moe:
                    rt = torch.stack([routes[r][a] for a in range(len(seq))], dim=1).numpy()
                check_request(cfg, tensors, seq, rows[r], rt, dtype, f"generation, request {r}")
    finally:
        engine.recorder = None
        engine.use_graphs = graphs


class TraceRun:
    """bin/trace_run as a child process: send a step, wait for its ``done`` line."""

    def __init__(self, model, dtype, out, max_tokens, record_routing=True):
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model, "--dtype", dtype,
               "--out", out, "--max-tokens", str(max_tokens)]
        if record_routing:
            cmd.append("--record-routing")
        self.out = out
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)

    def step(self, step, entries, end=()):
        self.proc.stdin.write(json.dumps({"step": step, "entries": entries, "end": list(end)}) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        assert line.strip() == f"done {step}", f"trace_run answered {line!r} (exit code {self.proc.poll()})"

    def logits(self, step, vocab):
        return torch.from_numpy(np.fromfile(os.path.join(self.out, f"{step}.f32"), dtype="<f4").reshape(-1, vocab).copy())

    def routes(self, step, nt, k):
        path = os.path.join(self.out, f"{step}.routes.i32")
        if not os.path.exists(path):
            return None
        return np.fromfile(path, dtype="<i4").reshape(-1, nt, k)

    def close(self):
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=120)
        assert rc == 0, f"trace_run exited with {rc}"
