#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default workload: the layer sizes of Qwen2.5-7B with random bfloat16 weights,
8 requests decoding at a context of 4,096 tokens.  A step is one decode step.
Prints ONE JSON line: ``value`` = decoded tokens per second at batch 8 (device
time over K steps), ``e2e`` = the same through the Python entry point with
host tokens in and out, ``prefill`` = one 2,048-token prompt step, ``roofline``
= bytes the decode step must read / its time against the measured copy
bandwidth, ``points`` = decode at batch 1 and 64.

The inputs of a decode step (15 GB of weights plus the live requests' cache)
are far larger than the 126 MB L2, so no separate L2 flush is done between
timed steps (``config.l2`` says so).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                v = d.get(k)
                if isinstance(v, dict):
                    v = v.get("value")
                if isinstance(v, (int, float)) and v > 0:
                    out[k] = float(v)
            return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


SIZES = {   # layer sizes of three models of the family: layers, hidden, heads, kv heads, feed-forward, vocabulary, tied
    "7b": (28, 3584, 28, 4, 18944, 152064, False),
    "3b": (36, 2048, 16, 2, 11008, 151936, True),
    "14b": (48, 5120, 40, 8, 13824, 152064, False),
}


def family_config(size: str = "7b"):
    """A config.json of the Qwen2.5-7B layer sizes (or, by name, of the 3B and 14B ones)."""
    layers, hidden, heads, kv_heads, inter, vocab, tied = SIZES[size]
    return dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=hidden, num_hidden_layers=layers,
                num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=128, intermediate_size=inter,
                vocab_size=vocab, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=tied,
                max_position_embeddings=32768, use_sliding_window=False, hidden_act="silu",
                torch_dtype="bfloat16")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                parts = [p.strip() for p in out.stdout.strip().split("\n")[0].split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except (OSError, subprocess.SubprocessError):
                pass
            self._stop.wait(0.2)

    def start(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=6)
        sm = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def reference_arm() -> int:
    """The reference as a whole cannot run here: it is a C++/CMake server that pip cannot install, and its
    forward does not compile offline (it includes llama.h of a submodule that is empty in the snapshot).  The
    line says so.  What of the reference does compile, its own attention kernels, is timed at the benchmark's
    shapes and added under "kernels" as the kernels to beat; they are no end-to-end number."""
    line = {"impl": "reference", "unavailable":
            "vjsingh1984/inferflux is a C++/CMake server with no setup.py or pyproject.toml (pip: 'Directory is not "
            "installable'), and its forward includes llama.h of an empty submodule, so it cannot be built offline"}
    try:
        import torch
        from baseline import reference_kernels
        if torch.cuda.is_available() and reference_kernels.source_root() is not None:
            from baseline.reference_kernels import yardsticks
            line["kernels"] = yardsticks.measure()
            line["kernels_note"] = ("the reference's own attention kernels (flash_attention.cu, compiled unmodified "
                                    "for sm_100a), one layer of the Qwen2.5-7B sizes; not an end-to-end figure")
    except Exception as e:                                   # the arm must still print its line
        line["kernels_error"] = f"{type(e).__name__}: {e}"[:300]
    print(json.dumps(line))
    return 0


def mixed_workload(args) -> int:
    """N requests, prompts uniform in 128..2,048 tokens, 256 greedy output tokens each, all handed to
    Engine.generate at once: the scheduler cuts prompts into portions beside the decoding requests."""
    import torch
    from inferflux_b200 import Engine, SamplingParams
    cfgd = family_config(args.size)
    if args.layers:
        cfgd["num_hidden_layers"] = args.layers
    n = args.mixed
    gen = torch.Generator().manual_seed(0)
    lens = torch.randint(128, 2049, (n,), generator=gen).tolist()
    prompts = [torch.randint(0, cfgd["vocab_size"], (k,), generator=gen).tolist() for k in lens]
    eng = Engine.from_config(cfgd, seed=0, dtype="bfloat16", kv_cache_tokens=n * 2400, max_seqs=n + 1, max_batch_size=n,
                             max_batch_tokens=4096, chunked_prefill_tokens=1024, max_model_len=4096)
    eng.generate([prompts[0][:64]], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))    # loads the kernels
    torch.cuda.synchronize()
    # Five runs, the median reported and all five listed.  The first meets every prompt step's shapes for the
    # first time, and a decode step's graph is captured when its shape has come three times (the third run); from
    # the fourth on every step is a replay.
    sampler = ClockSampler()
    sampler.start()
    runs = []
    for _ in range(5):
        steps0 = eng.stats["steps"]
        t0 = time.perf_counter()
        res = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=256, ignore_eos=True))
        torch.cuda.synchronize()
        runs.append(time.perf_counter() - t0)
        steps_run = eng.stats["steps"] - steps0
    clock_rec = sampler.stop()
    dt = sorted(runs)[2]
    out_tokens = sum(len(r.tokens) for r in res)
    st = eng.stats
    print(json.dumps({
        "metric": f"mixed workload, {n} requests (Qwen2.5-{args.size.upper()} sizes, random bf16 weights)", "impl": "ours",
        "value": round(out_tokens / dt, 1), "unit": "output tokens/s", "total_tokens_per_s": round((out_tokens + sum(lens)) / dt, 1),
        "seconds": round(dt, 3), "seconds_of_each_run": [round(v, 3) for v in runs], "n_gpus": 1, "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random token ids",
        "clocks": clock_rec,
        "config": {"model": f"Qwen2.5-{args.size.upper()} sizes", "layers": cfgd["num_hidden_layers"], "requests": n,
                   "prompt_tokens": sum(lens), "output_tokens": out_tokens, "max_batch_tokens": 4096,
                   "chunked_prefill_tokens": 1024, "steps": steps_run, "preemptions": st["preemptions"]}}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the family size (named in config)")
    ap.add_argument("--size", default="7b", choices=sorted(SIZES), help="which of the family's layer sizes (default: the 7B ones)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--e2e-steps", type=int, default=200,
                    help="steps of the end-to-end loop (at least --steps; a profiler's launch list wants few)")
    ap.add_argument("--mixed", type=int, default=0, metavar="N",
                    help="instead of the decode step: N requests with prompts of 128 to 2,048 tokens and 256 output "
                         "tokens each through Engine.generate (chunked prompts beside decoding requests)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.mixed > 0:
        return mixed_workload(args)
    warmup = max(3, args.warmup)

    import torch
    from inferflux_b200 import Engine, SamplingParams, StepEntry
    from inferflux_b200.kernels import ops

    peaks, peaks_from = load_peaks()
    cfgd = family_config(args.size)
    full_layers = cfgd["num_hidden_layers"]
    if args.layers:
        cfgd["num_hidden_layers"] = args.layers
    layers = cfgd["num_hidden_layers"]
    ctx, batch = args.context, args.batch
    max_b = batch if args.no_points else max(batch, 64)
    pool_tokens = max_b * (ctx + 64)
    eng = Engine.from_config(cfgd, seed=0, dtype="bfloat16", kv_cache_tokens=pool_tokens, max_seqs=max_b + 1,
                             max_batch_tokens=4096, max_batch_size=max_b, chunked_prefill_tokens=2048,
                             max_model_len=ctx + 64)
    runner = eng.runner
    vocab = cfgd["vocab_size"]
    gen = torch.Generator().manual_seed(0)

    h, nh, nkv, hd, inter = (cfgd[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads",
                                               "head_dim", "intermediate_size"))
    per_layer_params = (nh + 2 * nkv) * hd * h + (nh + 2 * nkv) * hd + nh * hd * h + 3 * h * inter + 2 * h
    weight_bytes = 2 * (layers * per_layer_params + vocab * h + h)          # + embedding rows (tiny)
    kv_bytes_per_token = 2 * layers * nkv * hd * 2

    def fill(rids, n_tokens):
        """Bring requests to n_tokens cached tokens by real prompt steps of up to 2,048 tokens."""
        for rid in rids:
            toks = torch.randint(0, vocab, (n_tokens,), generator=gen).tolist()
            for s in range(0, n_tokens, 2048):
                runner.step([StepEntry(rid, toks[s:s + 2048], [])])
        torch.cuda.synchronize()

    def time_decode(b, steps, warm):
        """Device time of `steps` decode steps at batch b, context ending at ctx."""
        rids = [f"b{b}_{i}" for i in range(b)]
        fill(rids, ctx - steps - warm)
        toks = torch.randint(0, vocab, (steps + warm, b), generator=gen).tolist()
        for w in range(warm):
            runner.step([StepEntry(r, [toks[w][i]], [0]) for i, r in enumerate(rids)])
        torch.cuda.synchronize()
        l0 = ops.launch_count
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        torch.cuda.synchronize()
        ev[0].record()
        for s in range(steps):
            logits = runner.step([StepEntry(r, [toks[warm + s][i]], [0]) for i, r in enumerate(rids)])
            eng.sampler.sample(logits, [greedy] * b, [0] * b, [0] * b, [[]] * b)
        ev[1].record()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[1]) / steps
        launches = ops.launch_count - l0
        for r in rids:
            runner.end(r)
        return ms, launches

    greedy = SamplingParams(temperature=0.0, max_tokens=1 << 30, ignore_eos=True)

    def clocked(fn, *a):
        """fn(*a) with the GPU's clocks and throttle reasons sampled meanwhile."""
        sampler = ClockSampler()
        sampler.start()
        res = fn(*a)
        return res, sampler.stop()

    def decode_bytes(b, steps):
        """What a decode step at batch b must read: every weight once and the live requests' cache
        (at the mean context of the timed steps)."""
        return weight_bytes + b * (ctx - steps // 2) * kv_bytes_per_token

    # ---- headline: decode at `batch`, device-timed
    (ms_step, launches), clock_rec = clocked(time_decode, batch, args.steps, warmup)
    value = batch / (ms_step / 1e3)
    step_bytes = decode_bytes(batch, args.steps)
    achieved = step_bytes / (ms_step / 1e3) / 1e9

    # ---- end to end: the Python entry point, host tokens in, host tokens out; at least 200 steps, so that
    # one stall of the host does not decide the figure
    e2e_steps = max(args.steps, args.e2e_steps)
    prompts = [torch.randint(0, vocab, (ctx - e2e_steps - warmup - 16,), generator=gen).tolist() for _ in range(batch)]
    params = SamplingParams(temperature=0.0, max_tokens=e2e_steps + warmup + 16, ignore_eos=True)
    for p in prompts:
        eng.add_request(p, params)
    while any(not r.decoding for r in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()                                   # prompt steps
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    e2e_ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    t0 = time.perf_counter()
    e2e_ev[0].record()
    n_e2e = 0
    e2e_clocks = ClockSampler()
    e2e_clocks.start()
    while eng.has_work() and n_e2e < e2e_steps:
        eng.step()                                   # plan, H2D metadata, run, sample, D2H ids
        n_e2e += 1
    e2e_ev[1].record()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / max(1, n_e2e)
    e2e_dev_ms = e2e_ev[0].elapsed_time(e2e_ev[1]) / max(1, n_e2e)
    e2e_clock_rec = e2e_clocks.stop()
    h2d = runner.slab._used * 4
    while eng.has_work():
        eng.step()
    e2e = {"value": round(batch / (e2e_ms / 1e3), 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
           "device_ms_per_step": round(e2e_dev_ms, 4), "steps": n_e2e,
           "mean_context": ctx - 16 - e2e_steps // 2, "sm_mhz": e2e_clock_rec["sm_mhz"],
           "reasons": e2e_clock_rec["reasons"],
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch}

    out = {
        "metric": f"decode tokens/s at batch {batch}, context {ctx} (Qwen2.5-{args.size.upper()} sizes, random bf16 weights)",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02), uniform random token ids",
        "impl": "ours",
        "config": {"model": f"Qwen2.5-{args.size.upper()} sizes", "layers": layers, "layers_of_family": full_layers, "hidden": h,
                   "heads": nh, "kv_heads": nkv, "head_dim": hd, "intermediate": inter, "vocab": vocab,
                   "global_batch": batch, "seq_len": ctx, "page_size": runner.page_size,
                   "parallelism": "single GPU", "l2": "inputs (weights + cache) exceed L2; no flush",
                   "peaks": peaks_from},
        "e2e": e2e, "gpu_launches": launches, "clocks": clock_rec,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "bytes_per_step": step_bytes},
    }

    if not args.no_points:
        # ---- prefill of 2,048 tokens in one step
        T = 2048
        toks = torch.randint(0, vocab, (T,), generator=gen).tolist()
        for i in range(3):
            runner.step([StepEntry(f"pw{i}", toks, [T - 1])])
            runner.end(f"pw{i}")
        torch.cuda.synchronize()
        reps = 5

        def time_prefill():
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            ev[0].record()
            for i in range(reps):
                runner.step([StepEntry(f"p{i}", toks, [T - 1])])
                runner.end(f"p{i}")
            ev[1].record()
            torch.cuda.synchronize()
            return ev[0].elapsed_time(ev[1]) / reps
        pms, pclock = clocked(time_prefill)
        lin_flops = 2 * T * layers * ((nh + 2 * nkv) * hd * h + nh * hd * h + 3 * h * inter) + 2 * vocab * h
        attn_flops = layers * 2 * 2 * nh * hd * (T * (T + 1) // 2)
        pflops = lin_flops + attn_flops
        out["prefill"] = {"value": round(T / (pms / 1e3), 1), "tokens": T, "ms": round(pms, 3),
                          "frac": round(pflops / (pms / 1e3) / 1e12 / peaks["bf16_tflops"], 4),
                          "frac_sustained": round(pflops / (pms / 1e3) / 1e12 / peaks["bf16_tflops_sustained"], 4),
                          "tflop": round(pflops / 1e12, 3), "sm_mhz": pclock["sm_mhz"], "reasons": pclock["reasons"]}
        points = {}
        for b in (1, 64):
            steps_b = min(args.steps, 32)
            (ms_b, _), bclock = clocked(time_decode, b, steps_b, 3)
            gbs = decode_bytes(b, steps_b) / (ms_b / 1e3) / 1e9
            points[f"decode_b{b}"] = round(b / (ms_b / 1e3), 2)
            points[f"decode_b{b}_ms"] = round(ms_b, 4)
            points[f"decode_b{b}_gbs"] = round(gbs, 1)
            points[f"decode_b{b}_frac"] = round(gbs / peaks["hbm_gbs"], 4)
            points[f"decode_b{b}_sm_mhz"] = bclock["sm_mhz"]
            points[f"decode_b{b}_reasons"] = ",".join(bclock["reasons"])
        out["points"] = points
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
