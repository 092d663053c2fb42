"""Time (or just launch, for a profiler) single kernels at a model family's sizes.

    python -m inferflux_b200.cli.kernel_bench list
    python -m inferflux_b200.cli.kernel_bench time  [--rows 1 8 64] [--context 4096] [--kernels gemv attn_decode ...]
    python -m inferflux_b200.cli.kernel_bench launch KERNEL [--rows 8] [--context 4096] [--repeat 5]
    INFERFLUX_B200_TIMELINE=1 python -m inferflux_b200.cli.kernel_bench timeline [--rows 8] [--context 4096] [--layers 28]

``time`` captures each kernel 20 times into a CUDA graph and times the replay with CUDA events (so the
host's launch cost is not in the number); operands rotate between buffers larger than L2.  ``launch`` runs
a kernel (and the variants timed beside it) a few times eagerly, which is what ``ncu -k regex:... -s 2 -c 1`` wants.  Sizes default to the
Qwen2.5-7B layer sizes; ``--sizes hidden,heads,kv_heads,head_dim,intermediate,vocab`` changes them.
The library product (cuBLAS through torch) is timed beside the weight-streaming kernel for comparison.
``timeline`` needs the instrumented build that the environment variable selects (a second library, built at
first use): every kernel notes the global timer once its predecessor is complete, and the mode prints the
start-to-start intervals of one replayed decode step of a whole model, kernel by kernel within a layer.
Library kernels carry no stamp: their time counts toward the kernel before them.
"""
from __future__ import annotations

import os
import argparse
import sys

import torch

from ..kernels import ops

DEV = "cuda:0"
KERNELS = ["gemv_qkv", "gemv_o", "gemv_gate_up", "gemv_down", "gemv_lm_head", "attn_decode", "attn_decode_skewed", "attn_prefill",
           "attn_prefill_umma",
           "add_rmsnorm", "rope_kv", "swiglu", "argmax", "sample"]


PAGE_SIZE = 16      # tokens a page of the attention workloads (--page-size)


def _timeit(fn, n_rot, reps=20):
    for i in range(3):
        fn(i % n_rot)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps):
            fn(i % n_rot)
    g.replay()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record()
    g.replay()
    ev[1].record()
    torch.cuda.synchronize()
    return ev[0].elapsed_time(ev[1]) / reps * 1e3      # microseconds


class Case:
    """Builds operands for one kernel at the given sizes; ``run(i)`` launches it on buffer set i."""

    def __init__(self, name, sizes, rows, context, sweep=False):
        h, nh, nkv, hd, inter, vocab = sizes
        self.name, self.bytes, self.flops, self.extra = name, 0, 0, []
        bf = dict(device=DEV, dtype=torch.bfloat16)
        it = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        if name.startswith("gemv_"):
            n, k, sw = {"qkv": ((nh + 2 * nkv) * hd, h, False), "o": (h, nh * hd, False), "gate_up": (inter, h, True),
                        "down": (h, inter, False), "lm_head": (vocab, h, False)}[name[5:]]
            wrows = 2 * n if sw else n
            self.n_rot = max(2, int(300e6 // (wrows * k * 2)) + 1)
            ws = [torch.randn(wrows, k, **bf) * 0.02 for _ in range(self.n_rot)]
            x = torch.randn(rows, k, **bf)
            self.bytes = wrows * k * 2
            if rows <= ops.GEMV_MAX_ROWS:
                out = torch.empty(rows, n, **bf)
                self.run = lambda i: ops.gemv_bf16(x, ws[i], None, out, swiglu=sw)
                if not sw and n < 10000:
                    # projections whose consumer adds float32 partial sums run with the planned number of K parts
                    planned = ops.gemv_k_splits(n, k)
                    self.note = f"k_splits={planned} (planned)"
                    outp = torch.empty((planned, rows, n) if planned > 1 else (rows, n), device=DEV, dtype=torch.float32)
                    self.run = lambda i, outp=outp, planned=planned: ops.gemv_bf16(x, ws[i], None, outp, k_splits=planned)
                    if sweep:
                        for s in range(1, 9):
                            outs = torch.empty((s, rows, n) if s > 1 else (rows, n), device=DEV, dtype=torch.float32)
                            self.extra.append((f"k_splits={s}", lambda i, s=s, outs=outs: ops.gemv_bf16(x, ws[i], None, outs, k_splits=s)))
            else:
                self.run = None
                if rows >= 256:
                    # many rows: the tcgen05 product beside the library's (SwiGLU: against library product + SwiGLU kernel)
                    outg = torch.empty(rows, n, **bf)
                    self.flops, self.bytes = 2 * rows * wrows * k, 0
                    self.extra.append(("tcgen05", lambda i: ops.gemm_umma(x, ws[i], None, outg, swiglu=sw)))
                    if sw:
                        gu = torch.empty(rows, wrows, **bf)
                        self.extra.append(("library + swiglu", lambda i: ops.swiglu(torch.mm(x, ws[i].t(), out=gu), outg)))
                    if name == "gemv_qkv" and hd == ops.QKV_EPILOGUE_HEAD_DIM:
                        # the product with bias, rotation and cache write in its epilogue, beside library product + kernel
                        ps = PAGE_SIZE
                        pool = torch.zeros((rows + ps - 1) // ps, 1, 2, nkv, ps, hd, **bf)
                        slots = torch.randperm(pool.shape[0] * ps, device=DEV)[:rows].to(torch.int32)
                        bias = torch.randn(n, device=DEV)
                        cos, sin = torch.randn(rows, hd // 2, device=DEV), torch.randn(rows, hd // 2, device=DEV)
                        qo, qkv_lib = torch.empty(rows, nh * hd, **bf), torch.empty(rows, n, **bf)
                        kv = (pool[0, 0, 0], pool[0, 0, 1], pool.stride(0), ps)
                        self.extra.append(("tcgen05 with bias, rotation, cache write",
                                           lambda i: ops.gemm_umma_qkv(x, ws[i], bias, qo, cos, sin, slots, *kv, nh, nkv)))
                        self.extra.append(("library + bias, rotation, cache write",
                                           lambda i: ops.qkv_rope_kv_write(torch.mm(x, ws[i].t(), out=qkv_lib), bias, cos, sin,
                                                                           slots, *kv, nh, nkv, hd)))
            self.extra.append(("library", lambda i: torch.mm(x, ws[i].t())))
            if not sw and rows <= ops.SKINNY_MAX_ROWS:
                sp = ops.gemm_umma_skinny_parts(n, k)
                outs = torch.empty(sp, rows, n, device=DEV)
                self.extra.append((f"tcgen05, weights as the tiles' rows, K in {sp} parts",
                                   lambda i, outs=outs: ops.gemm_umma_skinny(x, ws[i], outs)))
        elif name in ("attn_decode", "attn_decode_skewed", "attn_prefill", "attn_prefill_umma"):
            ps = PAGE_SIZE
            decode = name.startswith("attn_decode")
            b = rows if decode else 1
            q_len = 1 if decode else rows
            ctx = context
            # skewed: the first request has the whole context, the others a thirtieth of it
            ctxs = [ctx] + [max(1, ctx // 30)] * (b - 1) if name == "attn_decode_skewed" else [ctx] * b
            nblk = (ctx + ps - 1) // ps
            pages = sum((c + ps - 1) // ps for c in ctxs)
            self.n_rot = max(2, int(300e6 // (pages * 2 * nkv * ps * hd * 2)) + 1)
            pools = [torch.randn(pages, 1, 2, nkv, ps, hd, **bf) for _ in range(self.n_rot)]
            perm, bt_host, at = torch.randperm(pages).int(), torch.full((b, nblk), -1, dtype=torch.int32), 0
            for r, c in enumerate(ctxs):
                k = (c + ps - 1) // ps
                bt_host[r, :k] = perm[at:at + k]
                at += k
            bt = bt_host.to(DEV)
            n = b * q_len
            q = torch.randn(n, (nh + 2 * nkv) * hd, **bf)
            out = torch.empty(n, nh * hd, **bf)
            qs, ql, cs = it([i * q_len for i in range(b)]), it([q_len] * b), it([c - q_len for c in ctxs])
            scale = hd ** -0.5
            if decode:
                dec = it(list(range(b)))
                splits = ops.attn_decode_splits(b, nh, nkv, hd, ctx)
                po = torch.empty(b * nh * splits * hd, device=DEV)
                pm = torch.empty(b * nh * splits * 2, device=DEV)
                self.bytes = sum(ctxs) * nkv * hd * 2 * 2
                self.note = f"splits={splits}"
                self.run = lambda i: ops.attn_decode_bf16(q, q.stride(0), out, pools[i][0, 0, 0], pools[i][0, 0, 1],
                                                          pools[i].stride(0), ps, bt, dec, b, qs, ql, cs, po, pm, nh, nkv,
                                                          hd, scale, 0, splits)
                # the variant that adds the bias, rotates and writes the cache itself (steps of single tokens)
                width = (nh + 2 * nkv) * hd
                bias, cos, sin = torch.randn(width, device=DEV), torch.rand(b, hd // 2, device=DEV), torch.rand(b, hd // 2, device=DEV)
                slots = it([int(bt_host[r, (c - 1) // ps]) * ps + (c - 1) % ps for r, c in enumerate(ctxs)])
                parts = torch.randn(4, b, width, device=DEV) if rows <= 8 else None
                self.extra.append((f"prepares q,k,v {'from 4 partial sums' if parts is not None else ''}",
                                   lambda i: ops.attn_decode_prep_bf16(
                                       q, bias, cos, sin, slots, parts, out, pools[i][0, 0, 0], pools[i][0, 0, 1],
                                       pools[i].stride(0), ps, bt, dec, b, qs, ql, cs, po, pm, nh, nkv, hd, scale, 0, splits)))
                pieces = ops.attn_decode_pieces(nh, nkv, hd, ctx)
                pe = torch.empty(b * nh * pieces * hd, device=DEV)
                pme = torch.empty(b * nh * pieces * 2, device=DEV)
                pce = torch.empty(b * nh, dtype=torch.int32, device=DEV)
                self.extra.append((f"tiles shared out evenly (pieces<={pieces})", lambda i: ops.attn_decode_even_bf16(
                    q, out, pools[i][0, 0, 0], pools[i][0, 0, 1], pools[i].stride(0), ps, bt, dec, b, qs, ql, cs, pe, pme,
                    pce, nh, nkv, hd, scale, 0, pieces)))
                if sweep:
                    for s in (1, 2, 3, 4, 5, 6, 7, 8, 10, 11, 13, 16, 22, 32):
                        if s * 64 > ctx:
                            break
                        pos = torch.empty(b * nh * s * hd, device=DEV)
                        pms = torch.empty(b * nh * s * 2, device=DEV)
                        self.extra.append((f"splits={s}", lambda i, s=s, pos=pos, pms=pms: ops.attn_decode_bf16(
                            q, q.stride(0), out, pools[i][0, 0, 0], pools[i][0, 0, 1], pools[i].stride(0), ps, bt, dec, b,
                            qs, ql, cs, pos, pms, nh, nkv, hd, scale, 0, s)))
            else:
                umma = name.endswith("umma")
                # the tile height as the attention part picks it: 128 where tiles of 256 would leave SMs idle
                full = ops.UMMA_ATTENTION_TILE
                utile = full // 2 if 2 * ((q_len + full - 1) // full) * nh <= ops.sm_count(DEV) else full
                utile = int(os.environ.get("INFERFLUX_B200_BENCH_TILE_ROWS", utile))
                tiles = [(0, q0) for q0 in range(0, q_len, utile if umma else 64)]
                te, tq = it([t[0] for t in tiles]), it([t[1] for t in tiles])
                kernel = ops.attn_prefill_umma if umma else ops.attn_prefill_bf16
                # causal: query i sees ctx - q_len + i + 1 keys
                keys = sum(ctx - q_len + i + 1 for i in range(q_len))
                self.flops = 2 * 2 * nh * hd * keys
                extra = ()
                if umma:
                    splits = ops.attn_prefill_umma_splits(len(tiles), nh, ctx)
                    self.note = f"splits={splits} tiles of {utile}"
                    extra = (splits, utile)
                self.run = lambda i: kernel(q, q.stride(0), out, pools[i][0, 0, 0], pools[i][0, 0, 1],
                                                           pools[i].stride(0), ps, bt, te, tq, len(tiles), qs, ql, cs, nh,
                                                           nkv, hd, scale, 0, *extra)
        elif name == "add_rmsnorm":
            res, delta = torch.randn(rows, h, device=DEV), torch.randn(rows, h, **bf)
            w, o = torch.ones(h, device=DEV), torch.empty(rows, h, **bf)
            self.n_rot, self.bytes = 1, rows * h * (4 + 4 + 2 + 2)
            self.run = lambda i: ops.add_rmsnorm(res, delta, w, 1e-6, o)
            if rows <= 128:                                  # as after a product that came in parts of K
                parts = torch.randn(5, rows, h, device=DEV)
                self.extra.append(("5 partial sums", lambda i: ops.add_rmsnorm(res, parts, w, 1e-6, o, n_partials=5)))
        elif name == "swiglu":
            gu, o = torch.randn(rows, 2 * inter, **bf), torch.empty(rows, inter, **bf)
            self.n_rot, self.bytes = 1, rows * inter * 6
            self.run = lambda i: ops.swiglu(gu, o)
        elif name == "rope_kv":
            ps = 16
            width = (nh + 2 * nkv) * hd
            qkv, bias = torch.randn(rows, width, **bf), torch.randn(width, device=DEV)
            cos, sin = torch.randn(rows, hd // 2, device=DEV), torch.randn(rows, hd // 2, device=DEV)
            pool = torch.zeros((rows + ps - 1) // ps + 1, 1, 2, nkv, ps, hd, **bf)
            slots = torch.arange(rows, dtype=torch.int32, device=DEV)
            self.n_rot, self.bytes = 1, rows * width * 2 * 2
            self.run = lambda i: ops.qkv_rope_kv_write(qkv, bias, cos, sin, slots, pool[0, 0, 0], pool[0, 0, 1],
                                                       pool.stride(0), ps, nh, nkv, hd)
        elif name == "argmax":
            lg, oi = torch.randn(rows, vocab, device=DEV), torch.empty(rows, dtype=torch.int32, device=DEV)
            self.n_rot, self.bytes = 1, rows * vocab * 4
            self.run = lambda i: ops.argmax(lg, oi)
        elif name == "sample":
            lg = torch.randn(rows, vocab, device=DEV) * 3.0
            oi, w = torch.empty(rows, dtype=torch.int32, device=DEV), torch.empty(rows, vocab, device=DEV)
            f32 = lambda v: torch.full((rows,), v, dtype=torch.float32, device=DEV)
            seeds = torch.arange(rows, dtype=torch.int64, device=DEV)
            ctr = torch.zeros(rows, dtype=torch.int64, device=DEV)
            self.n_rot, self.bytes = 1, rows * vocab * 4
            self.run = None
            for label, k, p, mp in (("temperature 0.8", 0, 1.0, 0.0), ("temperature 0.8, top-k 50", 50, 1.0, 0.0),
                                    ("temperature 0.8, top-p 0.9", 0, 0.9, 0.0),
                                    ("temperature 0.8, top-k 50, top-p 0.9, min-p 0.01", 50, 0.9, 0.01)):
                tk = torch.full((rows,), k, dtype=torch.int32, device=DEV)
                self.extra.append((label, lambda i, tk=tk, p=p, mp=mp: ops.sample(lg, w, f32(0.8), tk, f32(p), f32(mp),
                                                                                 seeds, ctr, oi)))
        else:
            raise SystemExit(f"unknown kernel '{name}'; one of {KERNELS}")


STAMP_FILES = ("elementwise", "rope", "gemv", "attn", "sampling")


def _read_stamps(reset: bool):
    """(time in ns, source file) of every stamp since the last reset, in order of time."""
    import ctypes
    lib = ops._lib()
    buf = (ctypes.c_ulonglong * 4096)()
    out = []
    for name in STAMP_FILES:
        fn = getattr(lib, "ifx_stamps_" + name)
        fn.argtypes, fn.restype = [ctypes.c_void_p, ctypes.c_int], ctypes.c_int
        k = fn(buf, int(reset))
        out += [(buf[i], name) for i in range(k)]
    return sorted(out)


def timeline(sizes, layers: int, batch: int, context: int) -> int:
    from ..kernels import build
    if not build.TIMELINE:
        raise SystemExit("timeline needs the instrumented build: set INFERFLUX_B200_TIMELINE=1")
    from .. import Engine, StepEntry
    hidden, heads, kv_heads, head_dim, inter, vocab = sizes
    cfg = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=hidden, num_hidden_layers=layers,
               num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter,
               vocab_size=vocab, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
               max_position_embeddings=32768, use_sliding_window=False, hidden_act="silu", torch_dtype="bfloat16")
    room = context + 128
    eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", kv_cache_tokens=batch * room, max_seqs=batch + 1,
                             max_model_len=room, max_batch_size=batch)
    runner = eng.runner
    gen = torch.Generator().manual_seed(0)
    tok = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
    for i in range(batch):
        t = tok(context - 16)
        for a in range(0, len(t), 2048):
            runner.step([StepEntry(f"r{i}", t[a:a + 2048], [])])
    decode = lambda: runner.step([StepEntry(f"r{i}", tok(1), [0]) for i in range(batch)])
    before = runner.graph_replays
    for _ in range(8):
        decode()
    torch.cuda.synchronize()
    _read_stamps(True)
    decode()
    stamps = _read_stamps(True)
    if runner.graph_replays - before < 2 or len(stamps) < 2:
        raise SystemExit("the decode step was not replayed from a captured graph")
    gaps = [(name, (t2 - t) / 1000.0) for (t, name), (t2, _) in zip(stamps, stamps[1:])]
    names = [n for n, _ in gaps]
    # the layers are the longest stretch of the list that repeats once per layer
    first, per_layer = 0, 0
    for a in range(min(16, len(names))):
        for per in range((len(names) - a) // layers, 0, -1):
            if names[a:a + per * layers] == names[a:a + per] * layers:
                first, per_layer = a, per
                break
        if per_layer:
            break
    if not per_layer:
        raise SystemExit(f"no per-layer pattern in the stamped kernels: {names[:40]}")
    print(f"one replayed decode step: batch {batch}, context {context}, {layers} layers, {len(stamps)} stamped kernels, "
          f"{(stamps[-1][0] - stamps[0][0]) / 1000.0:.1f} us from the first stamp to the last")
    print(f"kernels per layer: {per_layer}; start-to-start intervals, mean over layers (us):")
    total = 0.0
    for k in range(per_layer):
        vals = [gaps[first + l * per_layer + k][1] for l in range(layers) if first + l * per_layer + k < len(gaps)]
        mean = sum(vals) / len(vals)
        total += mean
        print(f"  {k:2d} {names[first + k]:12s} {mean:8.2f}   (min {min(vals):.2f}, max {max(vals):.2f})")
    fmt = lambda part: ", ".join(f"{n} {d:.1f}" for n, d in part) or "none"
    print(f"  layer {total:.2f} us; before the first layer: {fmt(gaps[:first])}; "
          f"after the last: {fmt(gaps[first + layers * per_layer:])} (the last stamped kernel's own time is not seen)")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kernel_bench", description=__doc__.split("\n\n")[0])
    ap.add_argument("mode", choices=["list", "time", "launch", "timeline"])
    ap.add_argument("--layers", type=int, default=28, help="timeline: layers of the model")
    ap.add_argument("kernel", nargs="?")
    ap.add_argument("--kernels", nargs="*", default=None)
    ap.add_argument("--rows", nargs="*", type=int, default=[1, 8, 64])
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--repeat", type=int, default=5)
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens a page of the attention workloads' cache")
    ap.add_argument("--sweep", action="store_true", help="time: also other numbers of K parts (small products) and of key splits (decode attention)")
    ap.add_argument("--sizes", default="3584,28,4,128,18944,152064",
                    help="hidden,heads,kv_heads,head_dim,intermediate,vocab")
    args = ap.parse_args(argv)
    globals()["PAGE_SIZE"] = args.page_size
    if args.mode == "list":
        print("\n".join(KERNELS))
        return 0
    sizes = tuple(int(v) for v in args.sizes.split(","))
    if args.mode == "timeline":
        return timeline(sizes, args.layers, args.rows[0] if len(args.rows) == 1 else 8, args.context)
    if args.mode == "launch":
        case = Case(args.kernel, sizes, args.rows[0], args.context)
        runs = ([case.run] if case.run else []) + [fn for _, fn in case.extra]     # every variant, so a profiler can pick by kernel name
        for fn in runs:
            for i in range(args.repeat):
                fn(i % case.n_rot)
        torch.cuda.synchronize()
        print(f"launched {args.kernel} {args.repeat} times at rows={args.rows[0]} context={args.context}")
        return 0
    for rows in args.rows:
        print(f"--- rows={rows} context={args.context}")
        for name in args.kernels or KERNELS:
            case = Case(name, sizes, rows, args.context, args.sweep)
            runs = ([("", case.run)] if case.run else []) + case.extra
            for label, fn in runs:
                t = _timeit(fn, case.n_rot)
                what = f"{name} {label} {getattr(case, 'note', '')}".strip()
                rate = f"{case.bytes / t / 1e3:8.0f} GB/s" if case.bytes else f"{case.flops / t / 1e6:8.1f} TFLOP/s"
                print(f"{what:34s} {t:9.1f} us {rate}")
            del case
    return 0


if __name__ == "__main__":
    sys.exit(main())
