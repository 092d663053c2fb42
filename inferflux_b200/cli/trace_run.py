"""Trace replay: feed given token ids through a model step by step and write
the logits.  It samples nothing and has no forward pass, cache or loader of its
own: it builds the same model and :class:`StepRunner` that generation uses and
calls its step function.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
    trace_run --random CONFIG.json --seed S --dtype ... (random weights, no folder is written)

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step that wants logits, ``DIR/<step>.f32`` gets them as little-endian
float32 ``[wanted, vocab]`` in the order of the entries and of ``want``.  After
every step a line ``done <step>`` is printed and flushed.  A line
``{"stats": true}`` is no step: it is answered by one line ``stats {...}``
with the cache pools' counters (pages in all, free, handed out so far, handed
out again after an earlier use) and the steps and tokens run.

The reference's nearest tools are its first-token probe
(tests/tools/first_token_probe.cpp:191-274, one prompt, top-N logits) and its
decode-trace comparison (scripts/compare_decode_traces.py); neither replays a
schedule of steps.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", help="folder with config.json and model.safetensors")
    ap.add_argument("--random", metavar="CONFIG.json",
                    help="instead of --model: a config.json whose model gets random weights from --seed")
    ap.add_argument("--seed", type=int, default=0, help="seed of the random weights (with --random)")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each request rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import torch
    from ..config import EngineConfig, build_spec, load_config
    from ..engine import Model, StepEntry, StepRunner, torch_dtype
    from ..kernels import ops

    os.makedirs(args.out, exist_ok=True)
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is available; this engine has no CPU path", file=sys.stderr)
        return 1
    if (args.model is None) == (args.random is None):
        ap.error("give exactly one of --model and --random")
    print("trace_run: preparing kernels and model ...", file=sys.stderr, flush=True)
    if args.model is not None:
        config = load_config(args.model)
        model = Model(build_spec(config), torch_dtype(args.dtype), args.device)
        model.load_folder(args.model)
    else:
        from ..weights.random_init import random_tensors_as_loaded
        with open(args.random) as f:
            config = load_config(json.load(f))
        model = Model(build_spec(config), torch_dtype(args.dtype), args.device)
        model.load(random_tensors_as_loaded(model.weight_specs(), args.seed, torch_dtype(args.dtype), args.device))
    ecfg = EngineConfig(dtype=args.dtype, device=args.device, page_size=args.page_size,
                        kv_cache_tokens=max(args.page_size, args.max_tokens), max_seqs=64)
    runner = StepRunner(model, ecfg)
    print("trace_run: ready", file=sys.stderr, flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        if rec.get("stats"):
            pools = runner.kv.pools
            print("stats " + json.dumps({
                "pages_total": [p.num_pages for p in pools], "pages_free": [p.num_free for p in pools],
                "page_allocations": [p.allocations for p in pools], "page_reuses": [p.reuses for p in pools],
                "steps": runner.steps, "tokens": runner.tokens_run}), flush=True)
            continue
        step = rec["step"]
        entries = [StepEntry(str(e["id"]), [int(t) for t in e["tokens"]], [int(p) for p in e.get("want", [])])
                   for e in rec.get("entries", [])]
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                arr = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f"{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            else:
                torch.cuda.synchronize()
            ops.check_device_errors(args.device)          # raises if a kernel's bounded wait ran out
        for rid in rec.get("end", []):
            rid = str(rid)
            if runner.has(rid):
                runner.end(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
