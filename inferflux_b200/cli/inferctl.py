"""inferctl: the local command line, in the manner of the reference's tools.

The reference's ``inferctl`` is an HTTP client (cli/main.cpp:1598-1642:
``completion|chat|models|status ...`` with ``--prompt --model --max-tokens
--stream ...``) and its closest local tool is the first-token probe
(tests/tools/first_token_probe.cpp:21-141: ``--model --prompt|--prompt-file
--top-n --max-tokens --ctx-size --batch-size --max-parallel-sequences``, JSON
out).  There is no server here, so the same commands and option names run the
engine in-process.  There is no tokenizer either: prompts are token ids.

    inferctl completion --model DIR --prompt "5 17 3" --max-tokens 16 [--temperature 0.8 --seed 7 ...]
    inferctl completion --model DIR --prompt-file prompts.txt --max-tokens 16     (one prompt of ids per line)
    inferctl completion --random config.json --weights-seed 0 --prompt "5 17 3"   (random weights, no folder written)
    inferctl models --model DIR          the configuration and the tensors the model wants
    inferctl status                      device, kernel library
    inferctl random --config config.json --seed 0 --out DIR     write a random-weights model folder
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def _add_engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", help="folder with config.json and model.safetensors")
    p.add_argument("--random", metavar="CONFIG.json",
                   help="instead of --model: a config.json whose model gets random weights from --weights-seed")
    p.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights (with --random)")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--ctx-size", type=int, default=None, help="most tokens of one request (default: the model's)")
    p.add_argument("--batch-size", type=int, default=16384, help="most tokens of one step (max_batch_tokens)")
    p.add_argument("--max-parallel-sequences", type=int, default=32, help="most requests of one step and live")
    p.add_argument("--chunked-prefill-tokens", type=int, default=512)
    p.add_argument("--kv-cache-tokens", type=int, default=None, help="cache pool size in tokens (default: from free memory)")
    p.add_argument("--page-size", type=int, default=16)


def _engine(args):
    from .. import Engine
    options = dict(dtype=args.dtype, max_model_len=args.ctx_size, max_batch_tokens=args.batch_size,
                   max_batch_size=args.max_parallel_sequences, max_seqs=max(args.max_parallel_sequences, 1),
                   chunked_prefill_tokens=args.chunked_prefill_tokens, kv_cache_tokens=args.kv_cache_tokens,
                   page_size=args.page_size)
    if args.random is not None:
        with open(args.random) as f:
            return Engine.from_config(json.load(f), seed=args.weights_seed, as_written=True, **options)
    return Engine.from_pretrained(args.model, **options)


def cmd_completion(args) -> int:
    from .. import SamplingParams, StepEntry
    prompts: List[List[int]] = []
    if args.prompt is not None:
        prompts.append(_ids(args.prompt))
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    if not prompts:
        print("inferctl completion: give --prompt or --prompt-file (token ids)", file=sys.stderr)
        return 2
    if (args.model is None) == (args.random is None):
        print("inferctl completion: give exactly one of --model and --random", file=sys.stderr)
        return 2
    eng = _engine(args)
    params = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                            frequency_penalty=args.frequency_penalty, presence_penalty=args.presence_penalty,
                            repetition_penalty=args.repetition_penalty, seed=args.seed, max_tokens=args.max_tokens,
                            stop_token_ids=_ids(args.stop) if args.stop else [])
    out = {"model": args.model or f"random:{args.random}:{args.weights_seed}", "dtype": args.dtype}
    if args.top_n:
        # the probe's view: the top logits after the (first) prompt
        import torch
        logits = eng.run_step([StepEntry("probe", prompts[0], [len(prompts[0]) - 1])])[0]
        eng.end_request("probe")
        top = torch.topk(logits, min(args.top_n, logits.numel()))
        out["top_logits"] = [{"token": int(i), "logit": float(v)} for v, i in zip(top.values.tolist(), top.indices.tolist())]
    t0 = time.time()
    rids = [eng.add_request(p, params) for p in prompts]
    done = {}
    while eng.has_work():
        for r in eng.step():
            done[r.rid] = r
            if args.stream:
                print(json.dumps({"id": r.rid, "tokens": r.tokens, "finish_reason": r.finish_reason}), flush=True)
    dt = time.time() - t0
    out["completions"] = [{"id": rid, "prompt_tokens": done[rid].prompt_tokens, "tokens": done[rid].tokens,
                           "finish_reason": done[rid].finish_reason} for rid in rids]
    n = sum(len(done[rid].tokens) for rid in rids)
    out["usage"] = {"completion_tokens": n, "seconds": round(dt, 4), "tokens_per_second": round(n / max(dt, 1e-9), 2)}
    out["stats"] = eng.stats
    print(json.dumps(out))
    return 0


def cmd_models(args) -> int:
    import torch
    from ..config import build_spec, load_config
    from ..engine.model import Model
    cfg = load_config(args.model)
    model = Model(build_spec(cfg), torch.bfloat16, "cpu")
    specs = model.weight_specs()
    print(json.dumps({"id": args.model, "architecture": cfg.architecture, "config": cfg.to_dict(),
                      "tensors": len(specs), "parameters": sum(int(torch.tensor(s.shape).prod()) for s in specs
                                                               if s.kind != "ignored"),
                      "cache_groups": [{"streams": [{"name": s.name, "heads": s.heads, "width": s.width}
                                                    for s in n.streams], "window": n.window, "runs": r}
                                       for n, r in zip(model.kv_needs, model.runs_per_group)]}))
    return 0


def cmd_status(args) -> int:
    import torch
    from ..kernels import build
    info = {"cuda_available": torch.cuda.is_available(), "kernel_library": build.build()}
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        free, total = torch.cuda.mem_get_info()
        info.update(device=p.name, sm=f"{p.major}.{p.minor}", sms=p.multi_processor_count,
                    memory_free_gb=round(free / 2 ** 30, 1), memory_total_gb=round(total / 2 ** 30, 1))
    print(json.dumps(info))
    return 0


def cmd_random(args) -> int:
    import torch
    from ..config import load_config
    from ..weights.random_init import write_random_model
    with open(args.config) as f:
        cfg = load_config(json.load(f))
    folder = write_random_model(args.out, cfg, args.seed, torch.bfloat16,
                                torch.float32 if args.float32_vectors else None)
    print(json.dumps({"written": folder, "seed": args.seed, "architecture": cfg.architecture}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="inferctl", description="inferflux_b200 command line (token ids in, token ids out)")
    sub = ap.add_subparsers(dest="command", required=True)
    c = sub.add_parser("completion", help="generate tokens for one or more prompts")
    _add_engine_options(c)
    c.add_argument("--prompt", help="token ids separated by spaces or commas")
    c.add_argument("--prompt-file", help="one prompt of token ids per line")
    c.add_argument("--max-tokens", "--max_tokens", dest="max_tokens", type=int, default=256)
    c.add_argument("--temperature", type=float, default=1.0, help="<= 0 is greedy")
    c.add_argument("--top-p", type=float, default=1.0)
    c.add_argument("--top-k", type=int, default=0)
    c.add_argument("--min-p", type=float, default=0.0)
    c.add_argument("--frequency-penalty", type=float, default=0.0)
    c.add_argument("--presence-penalty", type=float, default=0.0)
    c.add_argument("--repetition-penalty", type=float, default=1.0)
    c.add_argument("--seed", type=int, default=None)
    c.add_argument("--stop", help="token ids that end a request")
    c.add_argument("--stream", action="store_true", help="print each request as it finishes")
    c.add_argument("--top-n", type=int, default=0, help="also print the top N logits after the first prompt")
    c.set_defaults(fn=cmd_completion)
    m = sub.add_parser("models", help="describe a model folder")
    m.add_argument("--model", required=True)
    m.set_defaults(fn=cmd_models)
    s = sub.add_parser("status", help="device and kernel library")
    s.set_defaults(fn=cmd_status)
    r = sub.add_parser("random", help="write a model folder with random weights")
    r.add_argument("--config", required=True, help="a config.json of a registered architecture")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--float32-vectors", action="store_true", help="store norm weights and biases in float32")
    r.set_defaults(fn=cmd_random)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
