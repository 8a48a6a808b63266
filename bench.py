"""Benchmark: decode tokens per second and prefill tokens per second of the
dense Qwen3 decoder at Qwen3-8B layer sizes, bfloat16, random weights, on one
B200.  A "step" is one decode step of a batch of 8 sequences from depth 2048
(context 4096 per sequence).  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]
    python bench.py --cpu-baseline      # the plain implementation of tests/ on the CPU, tiny configurations
    python bench.py --design tifapel    # the Tifapel decoder beside the dense decoder at equal layer sizes
    python bench.py --design voserax    # the Voserax decoder beside the Tifapel decoder's attention layers, two sizes
    python bench.py --design ninenex    # the Ninenex decoder beside the Tifapel decoder's retention and attention layers, two sizes
    python bench.py --design fusasun    # the Fusasun decoder beside the Tifapel decoder's attention layers, two sizes

``value`` is device-timed (CUDA events around K steps queued back to back);
``e2e`` is the same metric through ``Session.generate`` with host token ids in
and out, every step copying its inputs from pinned host memory and reading
the sampled tokens back, over at least 256 steps.  ``points`` has the same at
batch 1 and 64 and the prefill rate at other lengths (tokens per second);
``point_details`` has their milliseconds, roofline fractions, end-to-end rates
and the host's microseconds per step.  Weights (16 GB) and cache are far
larger than L2, so nothing is flushed between steps.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent

# The benchmark's model: Qwen3-8B layer sizes
QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960,
    use_sliding_window=False, sliding_window=None, torch_dtype="bfloat16", eos_token_id=151645,
)
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            raw = json.loads(p.read_text())
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in raw.items() if k in out and isinstance(v, (int, float))})
            return out, "measured"
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])), mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def model_numbers(cfg, n_layers):
    """Bytes a decode step must read and FLOPs a prompt step must do."""
    d, f, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = d * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * d + 3 * d * f
    weight_bytes = 2 * (n_layers * per_layer + V * d) + 4 * (n_layers * (2 * d + 2 * cfg.head_dim) + d)
    kv_bytes_per_token = n_layers * 2 * cfg.kv_dim * 2

    def prefill_flops(T):
        gemm = 2.0 * T * n_layers * per_layer + 2.0 * V * d           # the head runs on one row
        attn = n_layers * 2.0 * 2.0 * cfg.q_dim * (T * (T + 1) / 2)   # QK^T and PV over the causal half
        return gemm + attn

    return weight_bytes, kv_bytes_per_token, prefill_flops


def timeline(eng, cfg, args, rng) -> int:
    """One replayed decode step seen from inside: every kernel's first thread records when it reached its
    programmatic-launch wait and when the wait returned.  The time from one kernel's return to the next one's is
    that kernel's share of the step's critical path, measured in place (CUDA graph, overlapping launches)."""
    import ctypes
    import re
    from collections import defaultdict

    import torch
    from llmoxide_b200.csrc.build import LIBRARIES, SRC_DIR, load_library

    B, V = args.batch, cfg.vocab_size
    slots = [eng.acquire() for _ in range(B)]
    for s in slots:
        eng.step([(s, rng.integers(0, V, args.depth).tolist())], [[]])

    def step():
        eng.step([(s, [int(rng.integers(0, V))]) for s in slots])

    for _ in range(max(args.warmup, 4)):
        step()
    libs = ("elementwise", "gemm_tc", "attention_decode")

    def kernel_at(lib, line):
        src = (SRC_DIR / LIBRARIES[lib][0][0]).read_text().splitlines()
        for i in range(line - 1, -1, -1):
            m = re.search(r"^\s*(\w+_kernel)\(", src[i]) or re.search(r"__global__.*?(\w+_kernel)\(", src[i])
            if m:
                return m.group(1)
        return f"{lib}:{line}"

    def read_all():
        out = []
        for lib in libs:
            fn = load_library(lib).llmx_timeline_read
            fn.restype = ctypes.c_int
            buf = (ctypes.c_ulonglong * (3 * 65536))()
            n = fn(buf, 65536)
            if n < 0:
                raise RuntimeError(f"timeline of {lib}: CUDA error {-n}")
            out += [(buf[3 * i + 2], buf[3 * i + 1], lib, int(buf[3 * i])) for i in range(n) if buf[3 * i] < 1000000]
        return sorted(out)

    read_all()
    step()
    torch.cuda.synchronize()
    recs = read_all()
    t0 = recs[0][0]
    share = defaultdict(list)
    print(f"{'#':>4} {'kernel':34} {'resident':>10} {'ready':>10} {'to next':>9}   (us)", file=sys.stderr)
    for i, (ready, reached, lib, line) in enumerate(recs):
        name = kernel_at(lib, line)
        nxt = recs[i + 1][0] if i + 1 < len(recs) else ready
        share[name].append((nxt - ready) / 1e3)
        print(f"{i:4d} {name:34} {(reached - t0) / 1e3:10.2f} {(ready - t0) / 1e3:10.2f} {(nxt - ready) / 1e3:9.2f}",
              file=sys.stderr)
    total = (recs[-1][0] - t0) / 1e3
    summary = {k: dict(n=len(v), mean_us=round(sum(v) / len(v), 2), sum_us=round(sum(v), 1)) for k, v in share.items()}
    print(json.dumps(dict(timeline="one decode step", batch=B, depth=args.depth, layers=args.layers,
                          kernels=len(recs), step_us=round(total, 1), per_kernel=summary)))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"],
                    help="fewer layers than the configuration has, for a quick run; reported in config")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--depth", type=int, default=2048)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and batch 64 points")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--timeline", action="store_true",
                    help="instead of the benchmark: build the kernels with their in-place timers and print, for "
                         "one replayed decode step, when each kernel's dependency resolved")
    ap.add_argument("--cpu-baseline", action="store_true",
                    help="instead of the benchmark: time the plain implementation of tests/ on the CPU (tiny configurations)")
    ap.add_argument("--design", choices=["tifapel", "voserax", "ninenex", "fusasun"], default=None,
                    help="instead of the benchmark: prefill and decode rates of that design at layer sizes of a real "
                         "model (random weights), beside the dense Qwen3 decoder at equal sizes, with every kernel's "
                         "time per step (one JSON line of its own; the default workload is untouched)")
    ap.add_argument("--cuda-profiler", choices=["decode", "prefill"], default=None,
                    help="bracket that region with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "bigmah/llmoxide is a Rust workspace over wgpu; no Rust toolchain and no graphics stack "
                          "here, so pip cannot install it and its GPU path cannot run"}))
        return 0
    if args.cpu_baseline:
        return cpu_baseline()
    if args.design:
        return design_bench(args)
    if args.gpus != 1:
        print(json.dumps({"note": f"this library runs on one GPU; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2

    if args.timeline:
        import os
        os.environ["LLMX_NVCC_EXTRA"] = (os.environ.get("LLMX_NVCC_EXTRA", "") + " -DLLMX_TIMELINE").strip()

    import numpy as np
    import torch

    sys.path.insert(0, str(ROOT))
    from llmoxide_b200 import LoadOptions, Request, Sampling, Session, kernels, read_config

    raw = dict(QWEN3_8B, num_hidden_layers=args.layers)
    cfg = read_config(raw)
    pk, pk_src = peaks()
    B, K, W = args.batch, args.steps, args.warmup
    big_b = 1 if args.no_points else 64
    max_b = max(B, big_b)
    opts = LoadOptions(dtype="bfloat16", max_tokens=max_b * args.context, max_batch=max_b,
                       max_step_tokens=max(args.prefill_tokens, B * args.depth, 0 if args.no_points else 16 * 2048),
                       cuda_graphs=not args.no_graphs)
    t_load = time.time()
    session = Session.random(cfg, seed=0, options=opts)
    eng = session.engine
    torch.cuda.synchronize()
    print(f"[bench] model ready in {time.time() - t_load:.1f} s: {cfg.summary()}", file=sys.stderr)
    weight_bytes, kv_per_token, prefill_flops = model_numbers(cfg, args.layers)
    rng = np.random.default_rng(0)
    V = cfg.vocab_size

    def event_time(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    if args.timeline:
        return timeline(eng, cfg, args, rng)

    # ---- prefill: one prompt of 2,048 tokens ----------------------------------
    T = args.prefill_tokens

    def prefill_time(lengths, profile=False):
        """Median milliseconds of one prompt step over sequences of these lengths (slots taken and given back)."""
        prompts = [rng.integers(0, V, n).tolist() for n in lengths]

        def one():
            slots = [eng.acquire() for _ in prompts]
            eng.step(list(zip(slots, prompts)))
            for s in slots:
                eng.release(s)

        for _ in range(3):
            one()
        if profile:
            torch.cuda.profiler.start()
            one()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        return statistics.median(event_time(one) for _ in range(5))

    def prefill_point(lengths, profile=False):
        ms = prefill_time(lengths, profile)
        flops = sum(prefill_flops(n) for n in lengths)
        # (a short prompt step whose shape comes back is replayed as a graph by the engine: say so)
        graph = bool(eng.options.cuda_graphs and sum(lengths) <= eng.options.graph_prompt_tokens)
        return dict(value=sum(lengths) / ms * 1e3, tokens=sum(lengths), ms=ms,
                    frac=flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), tflops=flops / (ms * 1e-3) / 1e12,
                    graph=graph)

    prefill = prefill_point([T], profile=args.cuda_profiler == "prefill")
    print(f"[bench] prefill {T} tokens: {prefill['ms']:.2f} ms", file=sys.stderr)

    # ---- decode: B sequences at depth, K steps ----------------------------------
    def decode_rate(batch, steps, warmup, sampler=None, depth=None):
        depth = depth or args.depth
        slots = [eng.acquire() for _ in range(batch)]
        for s in slots:
            for lo in range(0, depth, 8192):          # deep contexts are fed in chunks
                eng.step([(s, rng.integers(0, V, min(8192, depth - lo)).tolist())], [[]])
        toks = rng.integers(0, V, (warmup + steps, batch)).tolist()
        for i in range(warmup):
            eng.step([(s, [t]) for s, t in zip(slots, toks[i])])
        launches = kernels.launch_count
        if sampler:
            sampler.start()

        def run():
            for i in range(warmup, warmup + steps):
                eng.step([(s, [t]) for s, t in zip(slots, toks[i])])

        if sampler and args.cuda_profiler == "decode":
            torch.cuda.profiler.start()
        ms = event_time(run)
        if sampler and args.cuda_profiler == "decode":
            torch.cuda.profiler.stop()
        clocks = sampler.stop() if sampler else None
        launches = kernels.launch_count - launches
        for s in slots:
            eng.release(s)
        mean_depth = depth + warmup + steps / 2
        step_bytes = weight_bytes + batch * mean_depth * kv_per_token
        gbs = step_bytes / (ms / steps * 1e-3) / 1e9
        return dict(value=batch * steps / ms * 1e3, ms_per_step=ms / steps, gb_per_s=gbs, frac=gbs / pk["hbm_gbs"],
                    launches=launches, clocks=clocks)

    main_pt = decode_rate(B, K, max(W, 3), ClockSampler())
    value, ms_per_step, launches, clocks = main_pt["value"], main_pt["ms_per_step"], main_pt["launches"], main_pt["clocks"]
    achieved = main_pt["gb_per_s"]
    print(f"[bench] decode b{B}: {ms_per_step:.3f} ms/step, {value:.0f} tok/s, {achieved:.0f} GB/s", file=sys.stderr)

    # ---- end to end through the Python entry point --------------------------------
    session.loop.stop_ids = frozenset()

    kernel_reports: list = []

    def e2e_rate(batch, steps):
        """Decoded tokens per second through Session.generate (host ids in, host ids out), and the host's own
        time per step.  A short run over the same prompts first, so that the batch's shape has its CUDA graph."""
        from llmoxide_b200.errors import KernelError

        prompts = [rng.integers(0, V, args.depth).tolist() for _ in range(batch)]
        # A prompt step of batch x depth tokens has, rarely, ended with the tcgen05 prompt attention reporting that
        # a bounded wait ran out (the loop then raises instead of using the step's results, and gives its slots
        # back).  The measurement is taken again, up to twice, and the JSON line says how often that happened.
        for attempt in range(3):
            try:
                session.generate([Request(p, max_tokens=3, sampling=Sampling.greedy(), stop_ids=()) for p in prompts])
                t0 = session.timings.decode_seconds, session.timings.decode_tokens, eng.host_seconds, eng.n_steps
                session.generate([Request(p, max_tokens=steps + 1, sampling=Sampling.greedy(), stop_ids=()) for p in prompts])
                break
            except KernelError as e:
                kernel_reports.append(str(e))
                print(f"[bench] e2e b{batch}, attempt {attempt + 1}: {e}", file=sys.stderr)
                torch.cuda.synchronize()
                if attempt == 2:
                    raise
        secs = session.timings.decode_seconds - t0[0]
        toks = session.timings.decode_tokens - t0[1]
        host_us = (eng.host_seconds - t0[2]) / max(1, eng.n_steps - t0[3] - 1) * 1e6
        return toks / secs, host_us

    e2e_steps = max(K, 256)
    e2e_value, host_us = e2e_rate(B, e2e_steps)
    lay_ints = 3 * B + (B + 1) + 2 * B + B + B * max(8, -(-((args.depth + e2e_steps + 64) // 64) // 8) * 8)
    e2e = dict(value=e2e_value, unit="tokens/s", steps=e2e_steps, h2d_bytes_per_step=4 * lay_ints,
               d2h_bytes_per_step=4 * B, host_us_per_step=host_us, kernel_reports_retried=len(kernel_reports))
    print(f"[bench] e2e decode b{B}: {e2e_value:.0f} tok/s over {e2e_steps} steps, host {host_us:.0f} us/step", file=sys.stderr)

    points, details = {}, {}
    if not args.no_points:
        for batch, steps in ((1, max(16, K // 2)), (64, max(8, K // 4))):
            pt = decode_rate(batch, steps, 3)
            rate, h_us = e2e_rate(batch, 256 if batch == 1 else 96)
            points[f"decode_b{batch}"] = pt["value"]
            details[f"decode_b{batch}"] = dict(ms_per_step=pt["ms_per_step"], gb_per_s=pt["gb_per_s"], frac=pt["frac"],
                                               e2e=rate, e2e_frac_of_device=rate / pt["value"], host_us_per_step=h_us)
        details[f"decode_b{B}"] = dict(ms_per_step=ms_per_step, gb_per_s=achieved, frac=main_pt["frac"], e2e=e2e_value,
                                       e2e_frac_of_device=e2e_value / value, host_us_per_step=host_us)
        for batch, depth in ((8, 8192), (1, 32768)):       # deeper contexts: the cache outweighs the weights
            pt = decode_rate(batch, 16, 3, depth=depth)
            points[f"decode_b{batch}_depth{depth}"] = pt["value"]
            details[f"decode_b{batch}_depth{depth}"] = dict(ms_per_step=pt["ms_per_step"], gb_per_s=pt["gb_per_s"],
                                                            frac=pt["frac"])
        lens16 = rng.integers(64, 2049, 16).tolist()       # an unequal batch: 16 prompts of 64..2048 tokens
        for name, lengths in (("prefill_512", [512]), ("prefill_8192", [8192]), ("prefill_16_unequal", lens16)):
            pp = prefill_point(lengths)
            points[name] = pp["value"]
            details[name] = dict(tokens=pp["tokens"], ms=pp["ms"], frac=pp["frac"], tflops=pp["tflops"],
                                 graph=pp["graph"])

    line = dict(
        metric="decode tok/s at batch 8 from depth 2048, Qwen3-8B layer sizes, bf16", value=value, unit="tokens/s",
        n_gpus=1, steps=K, warmup=max(W, 3), ms_per_step=ms_per_step, higher_is_better=True, scaling="weak",
        vs_baseline=None, dtype="bf16", data="synthetic: seeded uniform token ids, random weights N(0,0.02)",
        impl="ours",
        config=dict(model="Qwen3-8B layer sizes", layers=args.layers, layers_of_model=QWEN3_8B["num_hidden_layers"],
                    hidden=cfg.hidden_size, heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads,
                    head_dim=cfg.head_dim, intermediate=cfg.intermediate_size, vocab=cfg.vocab_size,
                    global_batch=B, seq_len=args.context, depth=args.depth, prefill_tokens=T,
                    parallelism="single GPU", l2="weights and cache far larger than L2; no flush",
                    cuda_graphs=not args.no_graphs, peaks=pk_src),
        prefill=prefill,
        roofline=dict(bound="hbm", achieved=achieved, peak=pk["hbm_gbs"], unit="GB/s", frac=achieved / pk["hbm_gbs"]),
        points=points, point_details=details, e2e=e2e, gpu_launches=launches, clocks=clocks,
    )
    print(json.dumps(line))
    return 0


# ---- another design beside the dense decoder ------------------------------------------------------------------

def tifapel_layers(n_layers, width, heads, kv_heads, dim, window, keep, experts, top, ff, groups):
    """Layers in the order attention, lightning, retention, attention reading the first one's keys and values."""
    moe = dict(kind="moe", expert=dict(ff=ff),
               router=dict(experts=experts, top=top, scale=1.0, groups=dict(count=groups[0], keep=groups[1])))
    decay = [1.0 - 2.0 ** -(3 + 7 * h / max(1, heads - 1)) for h in range(heads)]
    att = dict(type="attention", mlp=moe, mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim,
                                                     scale=dim ** -0.5, mask=dict(size=window, keep_first=keep)))
    out = []
    for i in range(n_layers):
        kind = i % 4
        if kind == 0:
            out.append(json.loads(json.dumps(att)))
        elif kind == 1:
            out.append(dict(type="lightning", mlp=moe, mixer=dict(heads=heads, dim=dim, vdim=dim, decay=decay)))
        elif kind == 2:
            out.append(dict(type="retention", mlp=moe, mixer=dict(heads=heads, dim=dim, vdim=dim, decay=decay,
                                                                  rot=dict(dims=dim, base=1000000.0))))
        else:
            layer = json.loads(json.dumps(att))
            layer["mixer"]["kv_from"] = i - 3
            out.append(layer)
    return out


def voserax_layers(n_layers, width, heads, kv_heads, dim, window, experts, top, ff, shared_ff):
    """Attention layers with a 4-tap convolution, rotation over half a head with scaled frequencies, mixed values;
    the first feed-forward dense, the others routed with two identity experts and a shared expert."""
    mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=dim ** -0.5, conv=4, mask=dict(size=window),
                 rot=dict(dims=dim // 2, base=10000.0, scaling=dict(factor=4.0, original=4096, fast=32.0, slow=1.0)),
                 v_mix=True)
    moe = dict(kind="moe", expert=dict(ff=ff, limit=7.0), router=dict(experts=experts, top=top, identity=2),
               shared=dict(ff=shared_ff, limit=7.0))
    return [dict(type="attention", mixer=json.loads(json.dumps(mixer)),
                 mlp=dict(kind="dense", ff=top * ff + shared_ff) if i == 0 else json.loads(json.dumps(moe)))
            for i in range(n_layers)]


def ninenex_layers(n_layers, heads, kv_heads, dim, chunk, experts, top, ff):
    """Layers in the order mLSTM (routed experts with a shared expert), attention beside retention (dense tanh-GELU
    feed-forward with biases), mLSTM on the first layer's weights, attention beside retention with routed experts."""
    moe = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top), shared=dict(ff=ff))
    mlstm = dict(type="mlstm", mixer=dict(heads=heads, dim=dim, vdim=dim, gate_cap=15.0), mlp=moe)
    half = max(1, heads // 2)
    decay = [1.0 - 2.0 ** -(3 + 7 * h / max(1, half - 1)) for h in range(half)]
    par = dict(type="parallel", mixer=dict(
        left=dict(heads=half, kv_heads=max(1, kv_heads // 2), dim=dim, vdim=dim, scale=dim ** -0.5, mask=dict(size=chunk),
                  rot=dict(dims=dim // 2, base=1000000.0)),
        right=dict(heads=half, dim=dim, vdim=dim, decay=decay), left_scale=0.8, right_scale=0.5))
    out = []
    for i in range(n_layers):
        kind = i % 4
        if kind == 0:
            out.append(json.loads(json.dumps(mlstm)))
        elif kind == 2:
            out.append(dict(json.loads(json.dumps(mlstm)), weights_of=i - 2))
        else:
            out.append(dict(json.loads(json.dumps(par)),
                            mlp=dict(kind="dense", ff=(top + 1) * ff) if kind == 1 else json.loads(json.dumps(moe))))
    return out


def fusasun_layers(n_layers, heads, kv_heads, dim, window, pool, experts, top, ff, q_rank, kv_rank):
    """Latent attention and attention over a window with pooled blocks in turn, every layer with experts named by a
    token table; a quarter of a latent head's query/key dimensions are rotated."""
    moe = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    rot = dim // 4
    latent = dict(type="latent_attention", mlp=moe, mixer=dict(
        heads=heads, dim=dim - rot, rot_dim=rot, vdim=dim, q_rank=q_rank, kv_rank=kv_rank, scale=dim ** -0.5,
        mask=dict(size=window), rot=dict(dims=rot, base=500000.0,
                                         scaling=dict(factor=4.0, original=4096, fast=32.0, slow=1.0))))
    att = dict(type="attention", mlp=moe, mixer=dict(
        heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=dim ** -0.5, mask=dict(size=window, pool=pool),
        rot=dict(dims=dim, base=10000.0, scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192))))
    return [json.loads(json.dumps(att if i % 2 else latent)) for i in range(n_layers)]


def design_bench(args) -> int:
    """``--design tifapel``: prefill and decode rates of the Tifapel decoder at layer sizes that resemble a real model's (width 2048,
    16 heads of 128 on 4 key/value heads, a window of 1024 that keeps 4 tokens, 16 experts of 1024 of which a
    token uses 2 from 2 of 4 groups), beside the dense Qwen3 decoder with the same width, heads and layer count and
    a feed-forward as wide as a token's two experts.  Device-timed with CUDA events, median of 5; weights and
    cache are larger than L2.  Then one prompt step and one decode step of each model with every kernel between
    two events of its own (no launch overlaps another), summed by kernel.

    ``--design voserax``: the same measurement of the Voserax decoder (four streams, a 4-tap convolution, a sink,
    mixed values, experts with identity and shared experts) at two sizes (width 2048 with 16 heads of 128 and 16
    experts of 1024; width 1024 with 16 heads of 64 and 8 experts of 512), beside the closest model of this package at
    equal sizes: the Tifapel decoder's attention layers with routed experts.

    ``--design ninenex``: the same measurement of the Ninenex decoder (mLSTM layers, layers with chunked attention
    beside retention, a norm before and behind every sublayer, dense feed-forwards with biases, routed experts with
    a shared expert) at the same two sizes, beside the Tifapel decoder with retention and windowed-attention layers
    in turn (every mixer with all the heads) and routed experts.

    ``--design fusasun``: the same measurement of the Fusasun decoder (latent attention and attention over a window
    with pooled blocks in turn, a 4-tap convolution before every mixer, gated results between two norms, experts
    named by a token table) at the same two sizes, beside the Tifapel decoder's attention layers with routed experts."""
    import numpy as np
    import torch

    sys.path.insert(0, str(ROOT))
    from llmoxide_b200 import Engine, LoadOptions, kernels, read_config

    L = min(args.layers, 8) if args.layers != QWEN3_8B["num_hidden_layers"] else 8
    vocab = 32768
    T, B, depth = args.prefill_tokens, args.batch, args.depth
    pk, pk_src = peaks()
    rng = np.random.default_rng(0)
    if args.design == "voserax":
        runs = []
        for width, heads, kv, dim, window, E, top, ff in ((2048, 16, 4, 128, 1024, 16, 2, 1024),
                                                          (1024, 16, 8, 64, 512, 8, 2, 512)):
            att = dict(type="attention", mixer=dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=dim ** -0.5,
                                                    mask=dict(size=window, keep_first=0)),
                       mlp=dict(kind="moe", expert=dict(ff=ff), router=dict(experts=E, top=top, scale=1.0)))
            models = {
                "voserax": dict(architecture="Voserax", vocab=vocab, width=width, norm=dict(eps=1e-6), residual_mult=0.5,
                                streams=4, max_positions=1 << 16,
                                layers=voserax_layers(L, width, heads, kv, dim, window, E, top, ff, ff)),
                "tifapel": dict(architecture="Tifapel", vocab=vocab, width=width, norm=dict(eps=1e-6),
                                layers=[json.loads(json.dumps(att)) for _ in range(L)]),
            }
            res = _design_models(args, models, vocab, T, B, depth, rng)
            runs.append(dict(sizes=dict(width=width, heads=heads, kv_heads=kv, head_dim=dim, window=window, experts=E, top=top,
                                        expert_ff=ff, shared_ff=ff, streams=4, conv=4, vocab=vocab), **res))
        print(json.dumps(dict(design="voserax", unit="tokens/s", dtype="bf16", layers=L, peaks=pk_src, hbm_gbs=pk["hbm_gbs"],
                              bf16_tflops=pk["bf16_tflops"], data="synthetic: seeded uniform token ids, random weights",
                              runs=runs)))
        return 0
    if args.design == "fusasun":
        runs = []
        for width, heads, kv, dim, window, pool, E, top, ff, rq, rkv in ((2048, 16, 4, 128, 1024, 64, 16, 2, 1024, 512, 256),
                                                                         (1024, 16, 8, 64, 512, 32, 8, 2, 512, 384, 128)):
            att = dict(type="attention", mixer=dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=dim ** -0.5,
                                                    mask=dict(size=window, keep_first=0)),
                       mlp=dict(kind="moe", expert=dict(ff=ff), router=dict(experts=E, top=top, scale=1.0)))
            models = {
                "fusasun": dict(architecture="Fusasun", vocab=vocab, width=width, norm=dict(eps=1e-6),
                                embedding=dict(scale=1.0), canon=dict(taps=4),
                                layers=fusasun_layers(L, heads, kv, dim, window, pool, E, top, ff, rq, rkv)),
                "tifapel": dict(architecture="Tifapel", vocab=vocab, width=width, norm=dict(eps=1e-6),
                                layers=[json.loads(json.dumps(att)) for _ in range(L)]),
            }
            res = _design_models(args, models, vocab, T, B, depth, rng)
            runs.append(dict(sizes=dict(width=width, heads=heads, kv_heads=kv, head_dim=dim, window=window, pool=pool,
                                        experts=E, top=top, expert_ff=ff, q_rank=rq, kv_rank=rkv, taps=4, vocab=vocab), **res))
        print(json.dumps(dict(design="fusasun", unit="tokens/s", dtype="bf16", layers=L, peaks=pk_src, hbm_gbs=pk["hbm_gbs"],
                              bf16_tflops=pk["bf16_tflops"], data="synthetic: seeded uniform token ids, random weights",
                              runs=runs)))
        return 0
    if args.design == "ninenex":
        runs = []
        for width, heads, kv, dim, window, E, top, ff in ((2048, 16, 4, 128, 1024, 16, 2, 1024),
                                                          (1024, 16, 8, 64, 512, 8, 2, 512)):
            moe = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=E, top=top, scale=1.0))
            decay = [1.0 - 2.0 ** -(3 + 7 * h / max(1, heads - 1)) for h in range(heads)]
            ret = dict(type="retention", mlp=moe, mixer=dict(heads=heads, dim=dim, vdim=dim, decay=decay))
            att = dict(type="attention", mlp=moe, mixer=dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=dim ** -0.5,
                                                             mask=dict(size=window, keep_first=0)))
            models = {
                "ninenex": dict(architecture="Ninenex", vocab=vocab, width=width, norm=dict(eps=1e-6),
                                embedding=dict(scale=1.0), logit_scale=1.0,
                                layers=ninenex_layers(L, heads, kv, dim, window, E, top, ff)),
                "tifapel": dict(architecture="Tifapel", vocab=vocab, width=width, norm=dict(eps=1e-6),
                                layers=[json.loads(json.dumps(att if i % 2 else ret)) for i in range(L)]),
            }
            res = _design_models(args, models, vocab, T, B, depth, rng)
            runs.append(dict(sizes=dict(width=width, heads=heads, kv_heads=kv, head_dim=dim, chunk=window, experts=E, top=top,
                                        expert_ff=ff, shared_ff=ff, dense_ff=(top + 1) * ff, vocab=vocab), **res))
        print(json.dumps(dict(design="ninenex", unit="tokens/s", dtype="bf16", layers=L, peaks=pk_src, hbm_gbs=pk["hbm_gbs"],
                              bf16_tflops=pk["bf16_tflops"], data="synthetic: seeded uniform token ids, random weights",
                              runs=runs)))
        return 0
    width, heads, kv, dim, window, keep, E, top, ff = 2048, 16, 4, 128, 1024, 4, 16, 2, 1024
    models = {
        "tifapel": dict(architecture="Tifapel", vocab=vocab, width=width, norm=dict(eps=1e-6),
                        layers=tifapel_layers(L, width, heads, kv, dim, window, keep, E, top, ff, (4, 2))),
        "dense": dict(QWEN3_8B, num_hidden_layers=L, hidden_size=width, num_attention_heads=heads,
                      num_key_value_heads=kv, head_dim=dim, intermediate_size=top * ff, vocab_size=vocab,
                      use_sliding_window=True, sliding_window=window, max_window_layers=0, eos_token_id=0),
    }
    result = _design_models(args, models, vocab, T, B, depth, rng)
    print(json.dumps(dict(design="tifapel", unit="tokens/s", dtype="bf16", layers=L, peaks=pk_src,
                          hbm_gbs=pk["hbm_gbs"], bf16_tflops=pk["bf16_tflops"],
                          sizes=dict(width=width, heads=heads, kv_heads=kv, head_dim=dim, window=window, keep_first=keep,
                                     experts=E, top=top, expert_ff=ff, dense_ff=top * ff, vocab=vocab),
                          data="synthetic: seeded uniform token ids, random weights", **result)))
    return 0


def _design_models(args, models, vocab, T, B, depth, rng) -> dict:
    """Per model of ``models`` (name -> raw configuration): prompt and decode times and the per-kernel lists."""
    import torch

    from llmoxide_b200 import Engine, LoadOptions, kernels, read_config

    def event_ms(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    def per_kernel(eng, entries):
        """One eager step with every launch between two events; {kernel: (launches, ms)}."""
        records, raw_fn = [], kernels._fn

        def timed_fn(lib, name, argtypes):
            f = raw_fn(lib, name, argtypes)

            def call(*a):
                tag = name.replace("llmx_", "")
                if name.startswith("llmx_gemm_tc") and len(a) > 6:
                    tag += f" N{a[5]} K{a[6]}"
                elif name == "llmx_gemm_fma":
                    tag += f" N{a[7]} K{a[8]}"
                elif name == "llmx_moe_grouped_tc":
                    tag += " gate|up" if a[13] else " down"
                elif name == "llmx_stream_mix_norm":
                    tag += " update+norm" if a[7] and a[14] else " norm" if a[14] else " update"
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                code = f(*a)
                e1.record()
                records.append((tag, e0, e1))
                return code
            return call

        kernels._fn = timed_fn
        kernels.set_overlap(False)
        graphs, eng.options.cuda_graphs = eng.options.cuda_graphs, False
        try:
            eng.step(entries)
            torch.cuda.synchronize()
        finally:
            kernels._fn = raw_fn
            kernels.set_overlap(True)
            eng.options.cuda_graphs = graphs
        out = {}
        for tag, e0, e1 in records:
            n, ms = out.get(tag, (0, 0.0))
            out[tag] = (n + 1, ms + e0.elapsed_time(e1))
        return {k: dict(launches=n, ms=round(ms, 4)) for k, (n, ms) in sorted(out.items(), key=lambda kv: -kv[1][1])}

    result = {}
    for name, raw in models.items():
        cfg = read_config(raw)
        eng = Engine.random(cfg, seed=0, options=LoadOptions(dtype="bfloat16", max_tokens=(B + 1) * (depth + 512) + T,
                                                             max_batch=B + 1, max_step_tokens=max(T, depth)))
        torch.cuda.synchronize()
        print(f"[bench] {name}: {cfg.summary()}", file=sys.stderr)

        def prefill_once():
            s = eng.acquire()
            eng.step([(s, rng.integers(0, vocab, T).tolist())])
            eng.release(s)

        for _ in range(3):
            prefill_once()
        pre_ms = statistics.median(event_ms(prefill_once) for _ in range(5))
        eng.check_status()
        s = eng.acquire()
        pre_kernels = per_kernel(eng, [(s, rng.integers(0, vocab, T).tolist())])
        eng.release(s)
        slots = [eng.acquire() for _ in range(B)]
        for sl in slots:
            eng.step([(sl, rng.integers(0, vocab, depth).tolist())], [[]])
        K, W = args.steps, max(args.warmup, 3)
        toks = rng.integers(0, vocab, (W + K + 1, B)).tolist()
        for i in range(W):
            eng.step([(sl, [t]) for sl, t in zip(slots, toks[i])])
        launches = kernels.launch_count
        dec_ms = event_ms(lambda: [eng.step([(sl, [t]) for sl, t in zip(slots, toks[i])]) for i in range(W, W + K)]) / K
        launches = (kernels.launch_count - launches) // K
        dec_kernels = per_kernel(eng, [(sl, [t]) for sl, t in zip(slots, toks[W + K])])
        eng.check_status()
        result[name] = dict(prefill_tokens=T, prefill_ms=round(pre_ms, 3), prefill_tokens_per_s=round(T / pre_ms * 1e3),
                            decode_batch=B, decode_depth=depth, decode_ms_per_step=round(dec_ms, 4),
                            decode_tokens_per_s=round(B / dec_ms * 1e3), launches_per_decode_step=launches,
                            prefill_kernels=pre_kernels, decode_kernels=dec_kernels)
        print(f"[bench] {name}: prefill {T} tokens {pre_ms:.2f} ms, decode b{B} {dec_ms:.3f} ms/step", file=sys.stderr)
        del eng
        torch.cuda.empty_cache()
    return result


def cpu_baseline() -> int:
    """Tokens per second of the plain implementation (tests/plain_qwen3.py: float32, whole sequences, no cache)
    on this machine's CPU, on the tiny configurations A and B: a prompt step over prompts of 5, 9, 13 (A) and 1, 7, 16, 31 (B) tokens and
    greedy decoding that recomputes the whole sequence for every token.  It is the oracle of the tests, timed
    for orientation; the reference's own CPU path cannot be built here."""
    import tempfile

    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import plain_qwen3 as plain
    from tiny_configs import make_folder, prompts

    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name, lengths, n_new in (("A", [5, 9, 13], 8), ("B", [1, 7, 16, 31], 12)):
            cfg, w = plain.read_model(make_folder(tmp, name, "float32"))
            ps = prompts(cfg["vocab_size"], lengths, seed=1)
            t0 = time.perf_counter()
            for p in ps:
                plain.forward(cfg, w, p)
            t_prefill = time.perf_counter() - t0
            t0 = time.perf_counter()
            for p in ps:
                plain.greedy_generate(cfg, w, p, n_new)
            t_decode = time.perf_counter() - t0 - t_prefill
            out[f"tiny_{name}"] = dict(prefill_tokens_per_s=sum(lengths) / t_prefill,
                                       decode_tokens_per_s=len(ps) * n_new / max(t_decode, 1e-9))
    print(json.dumps(dict(impl="plain implementation on the CPU (tests/plain_qwen3.py)", unit="tokens/s", **out)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
