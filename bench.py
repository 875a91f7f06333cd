"""Decode and prefill throughput of the Qwen2.5-7B shape (random weights, bfloat16) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl reference]

Prints ONE JSON line.  ``value`` is decoded tokens a second at the given batch (a step = one decode
step of the whole batch through the step function, timed on the device with CUDA events); ``e2e`` is
the same through the public engine calls (``add_request`` / ``step``) with host token ids in and
out every step; ``prefill`` is one 2,048-token prompt in one step; ``roofline`` compares the bytes a
decode step must read (every weight once, plus the cache of the live requests) with the measured
copy bandwidth; ``points`` holds decode at batch 1 and 64; ``kernels`` each dominant kernel alone at the
bench shape with its own roofline fraction.  Peaks come from MEASURED_PEAKS.json
beside this file when present.  One GPU only: for --gpus above 1 it says so and exits with 2.

``--compare fokedra`` times the Fokedra decoder (hyper-connected streams, gated chunked attention with unit-norm
heads, clamped gated feed-forward) beside the Qwen2.5 decoder at equal layer sizes: prefill and decode throughput
at three sizes, and every kernel the design adds beside the like kernel of the Qwen2.5 path with both rooflines.

``--compare sarudra`` does the same for the Sarudra decoder (state-space layers with per-request state and windowed
attention layers with query/key norms, rotated values and soft-capped scores in turn, routed experts beside a shared
one, grouped norms on the branches' outputs).

``--compare bezutar`` does the same for the Bezutar decoder (matrix-memory and gated-recurrence layers with per-request
state, latent attention over one cached row per token with sinks, a convolution over every mixer's input, an embedding
summed from three tables, hyper-connected streams, a feed-forward without a gate branch).

``--compare lakadra`` does the same for the Lakadra decoder (linear attention with a decay per head, latent attention,
windowed attention with a unit sink beside a gated linear recurrence, un-gated routed experts with groups, pass-through
experts and a gated shared expert, one norm for both branches of a layer).

``--only decode|prefill`` runs one part and prints a short line (profiling, and measurements beside the
headline): ``--only decode --batch 1 --prompt-len 32000 --context-len 32768`` is a decode step behind a long
context, ``--only prefill --chunk 512 --prefix 8192 --context-len 32768`` a prompt portion behind cached tokens.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import types
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen2.5-7B layer sizes (BASELINE.json configs[2])
SHAPE_7B = dict(vocab_size=152064, hidden_size=3584, num_hidden_layers=28, intermediate_size=18944,
                num_attention_heads=28, num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6,
                rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=8192,
                torch_dtype="bfloat16")
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

# The other measured workloads of BASELINE.json (configs[3] and configs[4]): end to end through the scheduler.
WORKLOADS = {
    "0.5b-mixed": dict(
        shape=dict(vocab_size=151936, hidden_size=896, num_hidden_layers=24, intermediate_size=4864,
                   num_attention_heads=14, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6,
                   rope_theta=1000000.0, tie_word_embeddings=True, max_position_embeddings=8192, torch_dtype="bfloat16"),
        requests=64, prompt=(16, 2048), new_tokens=128, chunk=512),
    "14b": dict(
        shape=dict(vocab_size=152064, hidden_size=5120, num_hidden_layers=48, intermediate_size=13824,
                   num_attention_heads=40, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5,
                   rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=8192, torch_dtype="bfloat16"),
        requests=32, prompt=(2048, 2048), new_tokens=256, chunk=2048),
}


def run_workload(name: str, args) -> int:
    """Generate through ``LLMEngine.generate_batch`` (scheduler, chunked prefill, continuous batching) and print
    one JSON line with the end-to-end token rates."""
    import numpy as np
    import torch

    from slipstream_b200 import CacheConfig, EngineConfig, SamplingParams, SchedulerConfig
    from slipstream_b200.engine.llm_engine import LLMEngine, Request

    w = WORKLOADS[name]
    folder = tempfile.mkdtemp(prefix=f"bench_{name}_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(w["shape"], architectures=["Qwen2ForCausalLM"], model_type="qwen2"), f)
    rng = np.random.default_rng(0)
    lo, hi = w["prompt"]
    lengths = rng.integers(lo, hi + 1, w["requests"]).tolist()
    pages = sum((n + w["new_tokens"] + 15) // 16 + 1 for n in lengths) + 64
    engine = LLMEngine(EngineConfig.for_model(
        folder, dtype="bfloat16", load_format="random", max_model_len=8192,
        cache=CacheConfig(block_size=16, num_gpu_blocks=pages),
        scheduler=SchedulerConfig(max_num_seqs=w["requests"], max_num_batched_tokens=8192, prefill_chunk_size=w["chunk"])))
    vocab = w["shape"]["vocab_size"]

    def requests(tag: str, new_tokens: int):
        return [Request(f"{tag}{i}", None, rng.integers(0, vocab, n).tolist(),
                        SamplingParams(max_tokens=new_tokens, temperature=0.0, ignore_eos=True), float(i) * 1e-6)
                for i, n in enumerate(lengths)]

    # warm-up: the same workload once, so that kernels are compiled and a graph is captured for every batch
    # bucket the run passes through while its requests finish (a capture inside the timed run costs tens of ms)
    engine.generate_batch(requests("w", w["new_tokens"]))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate_batch(requests("r", w["new_tokens"]))
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    assert all(len(o) == w["new_tokens"] for o in outs)
    generated, prompt_tokens = w["requests"] * w["new_tokens"], int(sum(lengths))
    print(json.dumps({"workload": name, "requests": w["requests"], "prompt_tokens": prompt_tokens,
                      "generated_tokens": generated, "seconds": round(seconds, 3),
                      "generated_tokens_per_s": round(generated / seconds, 1),
                      "total_tokens_per_s": round((generated + prompt_tokens) / seconds, 1),
                      "steps": engine.stats.step, "preemptions": engine.scheduler.preemptions,
                      "layers": w["shape"]["num_hidden_layers"], "dtype": "bf16", "data": "synthetic"}))
    return 0


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self) -> None:
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def __exit__(self, *exc) -> None:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(int(float(s[0])) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(float(self.samples[0][1])), "reasons": reasons,
                "samples": len(mhz)}


def reference_arm(args) -> int:
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "slipstream")):
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is not installed under baseline/_ref (pip install --no-deps --target baseline/_ref <reference>)"}))
        return 0
    from baseline.reference_bench import run_reference  # noqa: E402

    try:
        line = run_reference(args, SHAPE_7B, ref)
    except Exception as exc:  # the reference ran and failed: say so in one line instead of a traceback
        line = {"impl": "reference", "unavailable": f"the reference failed here: {type(exc).__name__}: {exc}"[:240]}
    print(json.dumps(line))
    return 0


def kernel_fractions(engine, batch: int, ctx_tokens: int, prefill_tokens: int, pk: dict) -> dict:
    """Each dominant kernel alone at the bench shape, timed with CUDA events: the decode projections and the
    decode attention against the bytes they must read (measured copy bandwidth), the prefill projections and the
    prefill attention against their flops (measured bf16 peak).  A kernel runs once per layer of the model, on that
    layer's own weights and pages, back to back as inside a step (28 x 33 MB of q/k/v weights and 28 x 17 MB of
    pages are larger than L2, so every launch reads from memory); median of five such sweeps, per launch."""
    import torch

    from slipstream_b200 import ops

    runner = engine.runner
    c = runner.config
    dev = runner.device
    blocks = runner.model.blocks
    gen = torch.Generator(device=dev).manual_seed(1)

    def rand(rows: int, cols: int) -> torch.Tensor:
        return (torch.randn(rows, cols, generator=gen, device=dev) * 0.5).to(torch.bfloat16)

    def sweep(run, layers: int | None = None) -> float:
        """Median microseconds per launch of ``run(layer)`` over ``layers`` layers (default: all).  The tensor-core
        kernels are timed as a burst, like the peak they are compared with: sweeps of a few launches, so that the
        GPU does not reach its power cap (a 2,048-token down projection takes 199 us in a burst and 238 us in
        the middle of thousands of launches)."""
        n = min(layers or len(blocks), len(blocks))
        torch.cuda.synchronize()
        if layers is not None:
            time.sleep(0.2)  # whatever ran before may have left the GPU at its power cap: let the clocks come back
        for layer in range(n):
            run(layer)
        times = []
        for _ in range(5):
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for layer in range(n):
                run(layer)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e3 / n)
        return sorted(times)[len(times) // 2]

    h, qkv_w = c.hidden_size, (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
    o_in, inter = c.num_attention_heads * c.head_dim, c.intermediate_size
    out: dict[str, dict] = {}

    def hbm(name: str, us: float, nbytes: float) -> None:
        gbs = nbytes / (us * 1e-6) / 1e9
        out[name] = {"us": round(us, 2), "gbs": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 3)}

    def tensor(name: str, us: float, flops: float) -> None:
        tf = flops / (us * 1e-6) / 1e12
        out[name] = {"us": round(us, 2), "tflops": round(tf, 1), "frac": round(tf / pk["bf16_tflops"], 3)}

    for tokens, tag in ((batch, "decode"), (prefill_tokens, "prefill")):
        x_h, x_o, x_i = rand(tokens, h), rand(tokens, o_in), rand(tokens, inter)
        shapes = {
            "qkv": (lambda i: ops.linear(x_h, blocks[i].mixer.qkv_weight, blocks[i].mixer.qkv_b), h, qkv_w),
            "o": (lambda i: ops.linear(x_o, blocks[i].mixer.o_weight, None), o_in, h),
            "gate_up": (lambda i: ops.gate_up_swiglu(x_h, blocks[i].feed_forward.gate_up, None,
                                                     blocks[i].feed_forward.block), h, 2 * inter),
            "down": (lambda i: ops.linear(x_i, blocks[i].feed_forward.down, None), inter, h),
        }
        for name, (run, k, n) in shapes.items():
            us = sweep(run, None if tag == "decode" else 8)
            if tag == "decode":
                hbm(f"decode_{name}", us, 2.0 * k * n + 2.0 * tokens * (k + n))
            else:
                tensor(f"prefill_{name}", us, 2.0 * tokens * k * n)
    # LM head: one weight, larger than L2 by itself
    x_rows = rand(batch, h)
    head = runner.model.lm_head
    us = sweep(lambda i: head.forward(x_rows))
    hbm("decode_lm_head", us, 2.0 * c.vocab_size * h + 4.0 * batch * c.vocab_size)

    # attention over the engine's own pages: `batch` requests of `ctx_tokens` cached tokens (what the pages hold
    # does not matter for the time), decode (one token each) and prefill (one request, all tokens new)
    page = runner.cache.page_size
    n_q, n_kv, d = c.num_attention_heads, c.num_key_value_heads, c.head_dim
    kv = runner.store.kv[0]

    def tables(n_req: int, tokens: int) -> torch.Tensor:
        per = (tokens + page - 1) // page
        return torch.arange(n_req * per, dtype=torch.int32, device=dev).view(n_req, per)

    qkv = rand(batch, (n_q + 2 * n_kv) * d)
    att = torch.empty(batch, n_q * d, dtype=torch.bfloat16, device=dev)
    table = tables(batch, ctx_tokens)
    q_start = torch.arange(batch + 1, dtype=torch.int32, device=dev)
    lens = torch.full((batch,), ctx_tokens, dtype=torch.int32, device=dev)
    slices = ops.decode_slices(batch, n_kv, n_q // n_kv, ctx_tokens, False, ops.sm_count(dev))
    us = sweep(lambda i: ops.paged_attention_decode(qkv, qkv.shape[1], att, kv[i], table, q_start, lens, batch, n_q, n_kv,
                                                    d, d ** -0.5, 0, slices))
    hbm("decode_attention", us, batch * ctx_tokens * 2.0 * n_kv * d * 2 + 2.0 * batch * n_q * d * 2)
    if ops.tcgen05_attention_fits(d, n_q, n_kv, page, 0):
        import numpy as np
        from slipstream_b200.engine.context import query_tiles_longest_first_host

        T, tile = prefill_tokens, 128 // (n_q // n_kv)
        qkv_p = rand(T, (n_q + 2 * n_kv) * d)
        att_p = torch.empty(T, n_q * d, dtype=torch.bfloat16, device=dev)
        req, tok0 = (torch.from_numpy(a).to(dev) for a in query_tiles_longest_first_host(
            np.asarray([T], dtype=np.int32), np.asarray([T], dtype=np.int32), tile))
        table_p = tables(1, T)
        q_start_p = torch.tensor([0, T], dtype=torch.int32, device=dev)
        lens_p = torch.tensor([T], dtype=torch.int32, device=dev)
        us = sweep(lambda i: ops.paged_attention_prefill_tcgen05(qkv_p, qkv_p.shape[1], att_p, kv[i], table_p, req, tok0,
                                                                 q_start_p, lens_p, n_q, n_kv, d, d ** -0.5, 1), 8)
        tensor("prefill_attention", us, 4.0 * n_q * d * (T * (T + 1) // 2))
    return out


def kernel_tables(which: str) -> int:
    """``--only gemm``: this package's tcgen05 products against the library product at prompt-portion sizes
    (microseconds a launch, CUDA events, weights rotated so that they come from memory).  ``--only attention``: the
    tcgen05 prefill attention at several (queries, keys), with the number of key parts the engine would choose."""
    import numpy as np
    import torch

    from slipstream_b200 import ops
    from slipstream_b200.engine.context import query_tiles_longest_first_host

    dev = torch.device("cuda:0")

    def timed(fn, n: int = 16) -> float:
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(n):
            fn(i)
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e3 / n

    if which == "gemm":
        shapes = (("7b q/k/v", 4608, 3584), ("7b o", 3584, 3584), ("7b down", 3584, 18944), ("7b gate/up", 37888, 3584),
                  ("0.5b q/k/v", 1152, 896), ("0.5b gate/up", 9728, 896), ("0.5b down", 896, 4864),
                  ("14b down", 5120, 13824), ("14b q/k/v", 7168, 5120))
        for name, features, k in shapes:
            copies = max(2, min(8, int(300e6 // (features * k * 2))))
            ws = [(torch.randn(features, k, device=dev) * 0.02).bfloat16() for _ in range(copies)]
            for tokens in (128, 256, 512, 1024, 2048, 4096):
                x = torch.randn(tokens, k, device=dev).bfloat16()
                row = {"library": timed(lambda i: torch.mm(x, ws[i % copies].t()))}
                for width in (64, 128, 256):
                    if width <= features and tokens <= 1024:
                        row[f"one-SM {width}"] = timed(lambda i: ops.gemm_tcgen05(x, ws[i % copies], plan=(False, width, 1)))
                row["two-SM"] = timed(lambda i: ops.gemm_tcgen05_many(x, ws[i % copies]))
                print(json.dumps({"shape": name, "features": features, "k": k, "tokens": tokens,
                                  **{key: round(v, 1) for key, v in row.items()}}), flush=True)
        ops.check_errors(dev)
        return 0

    n_q, n_kv, d, page = SHAPE_7B["num_attention_heads"], SHAPE_7B["num_key_value_heads"], SHAPE_7B["head_dim"], 16
    tile = 128 // (n_q // n_kv)
    for queries, keys in ((2048, 2048), (2048, 8192), (8192, 8192), (1024, 1024), (512, 4096), (64, 4096)):
        pages = keys // page + 4
        copies = max(2, min(16, int(300e6 // (pages * 2 * n_kv * page * d * 2))))
        kvs = [torch.randn(pages, 2, n_kv, page, d, device=dev).bfloat16() for _ in range(copies)]
        qkv = torch.randn(queries, (n_q + 2 * n_kv) * d, device=dev).bfloat16()
        out = torch.empty(queries, n_q * d, device=dev, dtype=torch.bfloat16)
        q_lens, seq_lens = np.asarray([queries], dtype=np.int32), np.asarray([keys], dtype=np.int32)
        req, tok0 = (torch.from_numpy(a).to(dev) for a in query_tiles_longest_first_host(q_lens, seq_lens, tile))
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1)
        q_start = torch.tensor([0, queries], dtype=torch.int32, device=dev)
        lens = torch.tensor([keys], dtype=torch.int32, device=dev)
        parts = ops.prefill_key_parts(q_lens, seq_lens, tile, n_kv)
        us = timed(lambda i: ops.paged_attention_prefill_tcgen05(qkv, qkv.shape[1], out, kvs[i % copies], table, req, tok0,
                                                                 q_start, lens, n_q, n_kv, d, d ** -0.5, parts), 20)
        flops = 4.0 * n_q * d * sum(min(keys, keys - queries + t + 1) for t in range(queries))
        print(json.dumps({"queries": queries, "keys": keys, "key_parts": parts, "us": round(us, 1),
                          "tflops": round(flops / us / 1e6, 1)}), flush=True)
    ops.check_errors(dev)
    return 0


# Layer sizes of the comparison (those of Qwen2.5-0.5B, -7B and -14B), with few layers: the per-layer times are what
# is compared, and the weights of either model are still larger than L2.
COMPARE_SIZES = {
    "0.5b": dict(vocab=151936, width=896, heads=14, kv_heads=2, dim=64, ff=4864, layers=8),
    "7b": dict(vocab=152064, width=3584, heads=28, kv_heads=4, dim=128, ff=18944, layers=8),
    "14b": dict(vocab=152064, width=5120, heads=40, kv_heads=8, dim=128, ff=13824, layers=6),
}


def compare_configs(z: dict, chunk: int, streams: int, share_kv: bool) -> tuple[dict, dict]:
    """config.json of the Qwen2.5 decoder and of the Fokedra decoder at the sizes ``z``."""
    qwen = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=z["vocab"], hidden_size=z["width"],
                num_hidden_layers=z["layers"], intermediate_size=z["ff"], num_attention_heads=z["heads"],
                num_key_value_heads=z["kv_heads"], head_dim=z["dim"], rms_norm_eps=1e-6, rope_theta=1000000.0,
                tie_word_embeddings=False, max_position_embeddings=8192, torch_dtype="bfloat16")
    layers = []
    for i in range(z["layers"]):
        mixer = dict(dim=z["dim"], vdim=z["dim"], heads=z["heads"], kv_heads=z["kv_heads"], scale=z["dim"] ** -0.5,
                     mask=dict(size=chunk),
                     rot=dict(base=1000000.0, dims=z["dim"], scaling=dict(factor=4.0, original=2048, fast=32.0, slow=1.0)))
        if share_kv and i % 2:
            mixer["kv_from"] = i - 1
        layers.append(dict(type="attention", mixer=mixer, mlp=dict(kind="dense", ff=z["ff"], limit=7.0)))
    fokedra = dict(architecture="Fokedra", vocab=z["vocab"], width=z["width"], streams=streams, norm=dict(eps=1e-6),
                   embedding=dict(scale=1.0), layers=layers, max_position_embeddings=8192)
    return qwen, fokedra


def measure_model(config: dict, args, pk: dict, rng) -> dict:
    """Prefill of one prompt of ``args.chunk`` tokens in one step (median of five, each by itself) and decode of
    ``args.batch`` requests behind ``args.prompt_len`` cached tokens, for the model ``config`` with random weights."""
    import torch

    from slipstream_b200 import ops
    from slipstream_b200.engine.runner import ModelRunner, StepEntry

    batch, ctx_tokens, T, page = args.batch, args.prompt_len, args.chunk, 16
    folder = tempfile.mkdtemp(prefix="bench_compare_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    pages = (batch * (ctx_tokens + args.steps + args.warmup + 16) + 2 * T) // page + 64
    runner = ModelRunner(folder, dtype="bfloat16", page_size=page, num_pages=pages, max_num_seqs=max(batch, 4),
                         max_model_len=8192, load_format="random", use_cuda_graphs=not args.no_graphs)
    vocab = runner.config.vocab_size
    # prefill: one prompt of T tokens in one step, as the captured graph a running engine replays; median of five
    times = []
    for w in range(getattr(runner, "mixed_graph_after", 0) + 2 + 5):
        toks = rng.integers(0, vocab, T).tolist()
        torch.cuda.synchronize()
        time.sleep(0.2)  # a step by itself, as the burst peak it is compared with
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry(f"p{w}", toks, [T - 1])])
        stop.record()
        torch.cuda.synchronize()
        runner.release(f"p{w}")
        times.append(start.elapsed_time(stop))
    prefill_ms = sorted(times[-5:])[2]
    print(f"[bench]   prefill {prefill_ms:.3f} ms", file=sys.stderr, flush=True)
    # decode: `batch` requests behind `ctx_tokens` cached tokens each
    ids = [f"d{i}" for i in range(batch)]
    per_step = max(1, 4096 // ctx_tokens)
    for i in range(0, batch, per_step):
        runner.step([StepEntry(r, rng.integers(0, vocab, ctx_tokens).tolist(), []) for r in ids[i:i + per_step]])
    feeds = rng.integers(0, vocab, (args.steps + args.warmup, batch)).tolist()
    for w in range(args.warmup):
        runner.step([StepEntry(r, [feeds[w][j]], [0]) for j, r in enumerate(ids)])
    torch.cuda.synchronize()
    launches0 = ops.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for s in range(args.steps):
        runner.step([StepEntry(r, [feeds[args.warmup + s][j]], [0]) for j, r in enumerate(ids)])
    stop.record()
    torch.cuda.synchronize()
    decode_ms = start.elapsed_time(stop) / args.steps
    launches = (ops.launch_count() - launches0) // args.steps
    nbytes = runner.weight_bytes_per_step() + batch * (ctx_tokens + args.warmup + args.steps / 2) * runner.kv_bytes_per_token()
    # what a design with routed experts and recurrent state reads besides: the experts a batch touches beyond one
    # token's (at most all of them), and every request's state, read and written
    for block in runner.model.blocks:
        ffn = getattr(block, "feed_forward", None)
        if hasattr(ffn, "experts"):
            first = ffn.gate_up if getattr(ffn, "gated", True) else ffn.up
            per_expert = (first[0].numel() + ffn.down[0].numel()) * ffn.down.element_size()
            nbytes += (min(ffn.experts, batch * ffn.top) - ffn.top) * per_expert
    for entry, state in zip(runner.model.order, runner.store.state):
        nbytes += 2 * batch * sum(t[0].numel() * t.element_size() for t in state.values())
    out = {"prefill_ms": round(prefill_ms, 3), "prefill_tok_s": round(T * 1000.0 / prefill_ms, 1),
           "decode_ms": round(decode_ms, 4), "decode_tok_s": round(batch * 1000.0 / decode_ms, 1),
           "decode_launches": int(launches), "decode_bytes_mb": round(nbytes / 1e6, 1),
           "decode_hbm_frac": round(nbytes / (decode_ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)}
    runner.check()
    del runner
    torch.cuda.empty_cache()
    return out



def run_compare(args) -> int:
    import numpy as np
    import torch

    from slipstream_b200 import ops
    from slipstream_b200.engine.context import query_tiles_host, query_tiles_longest_first_host
    from slipstream_b200.engine.runner import ModelRunner, StepEntry

    pk, pk_kind = peaks()
    rng = np.random.default_rng(0)
    dev = torch.device("cuda:0")
    batch, ctx_tokens, T, page = args.batch, args.prompt_len, args.chunk, 16
    result: dict = {"compare": "fokedra", "peaks": pk_kind, "batch": batch, "context": ctx_tokens, "prefill_tokens": T,
                    "mask_chunk": args.mask_chunk, "streams": args.streams, "share_kv": bool(args.share_kv), "sizes": {}}

    def measure(config: dict) -> dict:
        return measure_model(config, args, pk, rng)

    for name in (args.sizes.split(",") if args.sizes else COMPARE_SIZES):
        qwen, fokedra = compare_configs(COMPARE_SIZES[name], args.mask_chunk, args.streams, args.share_kv)
        result["sizes"][name] = {}
        for which, config in (("qwen2", qwen), ("fokedra", fokedra)):
            if which == "qwen2" and args.skip_qwen2:
                continue
            print(f"[bench] {name} {which} ...", file=sys.stderr, flush=True)
            result["sizes"][name][which] = measure(config)
            print(f"[bench] {name} {which}: {result['sizes'][name][which]}", file=sys.stderr, flush=True)

    # ---- every kernel the design adds, beside the like kernel of the Qwen2.5 path, at the 7B layer sizes
    print("[bench] single kernels ...", file=sys.stderr, flush=True)
    z = COMPARE_SIZES["7b"]
    h, n_q, n_kv, d, inter, S = z["width"], z["heads"], z["kv_heads"], z["dim"], z["ff"], args.streams
    gen = torch.Generator(device=dev).manual_seed(1)
    COPIES = 12  # operands of each timed launch rotate through this many copies: more than L2 holds

    def rand(*shape, dtype=torch.bfloat16):
        return (torch.randn(*shape, generator=gen, device=dev) * 0.5).to(dtype)

    def sweep(run) -> float:
        for i in range(COPIES):
            run(i)
        times = []
        for _ in range(5):
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(COPIES):
                run(i)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e3 / COPIES)
        return sorted(times)[2]

    kernels: dict = {}

    def hbm(name: str, us: float, nbytes: float) -> None:
        gbs = nbytes / (us * 1e-6) / 1e9
        kernels[name] = {"us": round(us, 2), "gbs": round(gbs, 1), "hbm_frac": round(gbs / pk["hbm_gbs"], 3)}

    def tensor(name: str, us: float, flops: float) -> None:
        tf = flops / (us * 1e-6) / 1e12
        kernels[name] = {"us": round(us, 2), "tflops": round(tf, 1), "bf16_frac": round(tf / pk["bf16_tflops"], 3)}

    w_norm = rand(h)
    mix, w_out, w_in = rand(S, S, dtype=torch.float32), rand(S, dtype=torch.float32), rand(S, dtype=torch.float32)
    for tokens, tag in ((T, "prefill"), (batch, "decode")):
        res = [rand(tokens, h, dtype=torch.float32) for _ in range(COPIES)]
        streams = [rand(tokens, S, h, dtype=torch.float32) for _ in range(COPIES)]
        ys = [rand(tokens, h) for _ in range(COPIES)]
        us = sweep(lambda i: ops.add_rmsnorm(res[i], ys[i], w_norm, 1e-6, torch.bfloat16))
        hbm(f"{tag}_add_rmsnorm (qwen2)", us, tokens * h * (4 + 4 + 2 + 2))
        us = sweep(lambda i: ops.hc_norm(streams[i], ys[i], mix, w_out, w_in, w_norm, 1e-6, torch.bfloat16))
        hbm(f"{tag}_hyper_connection_norm", us, tokens * h * (8 * S + 2 + 2))
        # rotation and page write
        width = (n_q + 2 * n_kv) * d
        rows = [rand(tokens, width + n_q * d) for _ in range(COPIES)]
        plain_rows = [rand(tokens, width) for _ in range(COPIES)]
        kvs = [torch.zeros((tokens + page - 1) // page + 1, 2, n_kv, page, d, dtype=torch.bfloat16, device=dev) for _ in range(COPIES)]
        positions = torch.arange(tokens, dtype=torch.int32, device=dev)
        inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev)
        us = sweep(lambda i: ops.rope_and_cache(plain_rows[i], positions, positions, inv_freq, kvs[i], n_q, n_kv, d, d))
        moved = tokens * d * 2.0 * (2 * n_q + 4 * n_kv)
        hbm(f"{tag}_rope_and_cache (qwen2)", us, moved)
        us = sweep(lambda i: ops.rope_norm_cache(rows[i], positions, positions, inv_freq, kvs[i], n_q, n_kv, d, d,
                                                 interleaved=True, mscale=1.1, norm_dim=d, eps=1e-6))
        hbm(f"{tag}_rope_norm_cache", us, moved)
    gu = [rand(T, 2 * inter) for _ in range(4)]
    COPIES_SAVED, COPIES = COPIES, 4
    us = sweep(lambda i: ops.swiglu(gu[i], block=64))
    hbm("prefill_swiglu (qwen2, unfused form)", us, T * inter * 6.0)
    us = sweep(lambda i: ops.glu_limited(gu[i], 64, 1.702, 7.0, 1.0))
    hbm("prefill_glu_limited (unfused form)", us, T * inter * 6.0)
    del gu
    x_h = rand(T, h)
    w_gu = [rand(2 * inter, h) for _ in range(4)]
    us = sweep(lambda i: ops.gate_up_swiglu(x_h, w_gu[i], None, 64))
    tensor("prefill_gate_up_swiglu (qwen2)", us, 4.0 * T * h * inter)
    us = sweep(lambda i: ops.gate_up_glu(x_h, w_gu[i], None, 64, 1.702, 7.0, 1.0))
    tensor("prefill_gate_up_glu", us, 4.0 * T * h * inter)
    x_b = rand(batch, h)
    us = sweep(lambda i: ops.gate_up_swiglu(x_b, w_gu[i], None, 64))
    hbm("decode_gate_up_swiglu (qwen2)", us, 4.0 * h * inter)
    us = sweep(lambda i: ops.gate_up_glu(x_b, w_gu[i], None, 64, 1.702, 7.0, 1.0))
    hbm("decode_gate_up_glu", us, 4.0 * h * inter)
    del w_gu
    COPIES = COPIES_SAVED

    # attention: the chunk as long as the context, so that both designs do the same work
    def tables(n_req: int, tokens: int) -> torch.Tensor:
        per = (tokens + page - 1) // page
        return torch.arange(n_req * per, dtype=torch.int32, device=dev).view(n_req, per)

    kv_pages = [rand(batch * ((ctx_tokens + page - 1) // page) + 1, 2, n_kv, page, d) for _ in range(COPIES)]
    width = (n_q + 2 * n_kv) * d
    qkv = rand(batch, width + n_q * d)
    att = torch.empty(batch, n_q * d, dtype=torch.bfloat16, device=dev)
    table = tables(batch, ctx_tokens)
    q_start = torch.arange(batch + 1, dtype=torch.int32, device=dev)
    lens = torch.full((batch,), ctx_tokens, dtype=torch.int32, device=dev)
    slices = ops.decode_slices(batch, n_kv, n_q // n_kv, ctx_tokens, False, ops.sm_count(dev))
    nbytes = batch * ctx_tokens * 2.0 * n_kv * d * 2 + 2.0 * batch * n_q * d * 2
    us = sweep(lambda i: ops.paged_attention_decode(qkv, qkv.shape[1], att, kv_pages[i], table, q_start, lens, batch, n_q,
                                                    n_kv, d, d ** -0.5, 0, slices, stages=ops.functions.DECODE_RING_STAGES))
    hbm("decode_attention (qwen2: rotation outside here)", us, nbytes)
    us = sweep(lambda i: ops.paged_attention_decode(qkv, qkv.shape[1], att, kv_pages[i], table, q_start, lens, batch, n_q,
                                                    n_kv, d, d ** -0.5, 0, slices, stages=ops.functions.DECODE_RING_STAGES,
                                                    chunk=args.mask_chunk, gate=qkv[:, width:]))
    hbm("decode_attention chunked + gate", us, nbytes + batch * n_q * d * 2.0)
    qkv_p = rand(T, width + n_q * d)
    att_p = torch.empty(T, n_q * d, dtype=torch.bfloat16, device=dev)
    table_p, q_start_p = tables(1, T), torch.tensor([0, T], dtype=torch.int32, device=dev)
    lens_p = torch.tensor([T], dtype=torch.int32, device=dev)
    req, tok0 = (torch.from_numpy(a).to(dev) for a in query_tiles_longest_first_host(
        np.asarray([T], dtype=np.int32), np.asarray([T], dtype=np.int32), 128 // (n_q // n_kv)))
    flops = 4.0 * n_q * d * (T * (T + 1) // 2)
    us = sweep(lambda i: ops.paged_attention_prefill_tcgen05(qkv_p, qkv_p.shape[1], att_p, kv_pages[i], table_p, req, tok0,
                                                             q_start_p, lens_p, n_q, n_kv, d, d ** -0.5, 1))
    tensor("prefill_attention tcgen05 (qwen2)", us, flops)
    req2, row0 = (torch.from_numpy(a).to(dev) for a in query_tiles_host(np.asarray([T * (n_q // n_kv)], dtype=np.int32), 64))
    us = sweep(lambda i: ops.paged_attention_prefill(qkv_p, qkv_p.shape[1], att_p, kv_pages[i], table_p, req2, row0, q_start_p,
                                                     lens_p, n_q, n_kv, d, d ** -0.5, 0))
    tensor("prefill_attention mma.sync, no mask (qwen2 with a window takes this kernel)", us, flops)
    us = sweep(lambda i: ops.paged_attention_prefill(qkv_p, qkv_p.shape[1], att_p, kv_pages[i], table_p, req2, row0, q_start_p,
                                                     lens_p, n_q, n_kv, d, d ** -0.5, 0, chunk=args.mask_chunk,
                                                     gate=qkv_p[:, width:]))
    tensor("prefill_attention mma.sync chunked + gate", us, flops)
    result["kernels_7b"] = kernels
    print(json.dumps(result))
    return 0


def sarudra_config(z: dict, window: int) -> dict:
    """config.json of a Sarudra decoder at the layer sizes ``z``: state-space layers and windowed attention layers in
    turn; every feed-forward routed, two of eight experts of a quarter of the dense size beside a shared expert of
    half of it, so that a token's feed-forward does the dense layer's work."""
    heads = 2 * z["width"] // 64  # the state-space layers' inner width is twice the model's
    groups = 8 if heads % 8 == 0 else 4
    layers = []
    for i in range(z["layers"]):
        if i % 2 == 0:
            kind, mixer = "mamba2", dict(heads=heads, vdim=64, state=128, groups=groups, conv=4, norm_groups=groups)
        else:
            kind, mixer = "attention", dict(dim=z["dim"], vdim=z["dim"], heads=z["heads"], kv_heads=z["kv_heads"],
                                            scale=z["dim"] ** -0.5, softcap=50.0, mask=dict(size=window),
                                            rot=dict(base=1000000.0, dims=z["dim"]))
        mlp = dict(kind="moe", expert=dict(ff=z["ff"] // 4), router=dict(experts=8, top=2), shared=dict(ff=z["ff"] // 2))
        layers.append(dict(type=kind, mixer=mixer, mlp=mlp))
    return dict(architecture="Sarudra", vocab=z["vocab"], width=z["width"], norm=dict(eps=1e-6, groups=4),
                embedding=dict(scale=1.0), logit_softcap=30.0, layers=layers, max_position_embeddings=8192)


def run_compare_sarudra(args) -> int:
    """The Sarudra decoder beside the Qwen2.5 decoder at equal layer sizes (whole steps), then every kernel the design
    adds, alone at the 7B layer sizes, beside its nearest relative of the Qwen2.5 path."""
    import numpy as np
    import torch

    from slipstream_b200 import ops
    from slipstream_b200.engine.context import query_tiles_longest_first_host

    pk, pk_kind = peaks()
    rng = np.random.default_rng(0)
    dev = torch.device("cuda:0")
    batch, ctx_tokens, T, page = args.batch, args.prompt_len, args.chunk, 16
    result: dict = {"compare": "sarudra", "peaks": pk_kind, "batch": batch, "context": ctx_tokens, "prefill_tokens": T,
                    "window": args.window, "sizes": {}}
    for name in (args.sizes.split(",") if args.sizes else COMPARE_SIZES):
        qwen, _ = compare_configs(COMPARE_SIZES[name], 8192, 1, False)
        result["sizes"][name] = {}
        for which, config in (("qwen2", qwen), ("sarudra", sarudra_config(COMPARE_SIZES[name], args.window))):
            if which == "qwen2" and args.skip_qwen2:
                continue
            print(f"[bench] {name} {which} ...", file=sys.stderr, flush=True)
            result["sizes"][name][which] = measure_model(config, args, pk, rng)
            print(f"[bench] {name} {which}: {result['sizes'][name][which]}", file=sys.stderr, flush=True)

    print("[bench] single kernels ...", file=sys.stderr, flush=True)
    z = COMPARE_SIZES["7b"]
    h, n_q, n_kv, d, inter = z["width"], z["heads"], z["kv_heads"], z["dim"], z["ff"]
    m = sarudra_config(z, args.window)["layers"][0]["mixer"]
    s_heads, s_p, s_n, s_g, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner, chans = s_heads * s_p, s_heads * s_p + 2 * s_g * s_n
    experts, top, e_ff = 8, 2, inter // 4
    gen = torch.Generator(device=dev).manual_seed(1)
    COPIES = 6  # operands of each timed launch rotate through this many copies

    def rand(*shape, dtype=torch.bfloat16, std=0.5):
        return (torch.randn(*shape, generator=gen, device=dev) * std).to(dtype)

    def sweep(run, copies=COPIES) -> float:
        for i in range(copies):
            run(i)
        times = []
        for _ in range(5):
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(copies):
                run(i)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e3 / copies)
        return sorted(times)[2]

    kernels: dict = {}

    def hbm(name: str, us: float, nbytes: float) -> None:
        gbs = nbytes / (us * 1e-6) / 1e9
        kernels[name] = {"us": round(us, 2), "gbs": round(gbs, 1), "hbm_frac": round(gbs / pk["hbm_gbs"], 3)}

    def tensor(name: str, us: float, flops: float, peak_key: str = "bf16_tflops") -> None:
        tf = flops / (us * 1e-6) / 1e12
        kernels[name] = {"us": round(us, 2), "tflops": round(tf, 1), "bf16_frac": round(tf / pk[peak_key], 3)}

    def step(q_lens, seq_lens):
        starts = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
        as_dev = lambda v: torch.tensor(np.asarray(v), dtype=torch.int32, device=dev)  # noqa: E731
        return types.SimpleNamespace(q_start=as_dev(starts), seq_lens=as_dev(seq_lens), state_slots=as_dev(np.arange(len(q_lens))),
                                     num_requests=len(q_lens), is_decode_only=all(n == 1 for n in q_lens))

    w_norm = rand(h, dtype=torch.float32)
    w_norm_bf = w_norm.bfloat16()
    for tokens, tag, ctx in ((T, "prefill", step([T], [T])), (batch, "decode", step([1] * batch, [ctx_tokens] * batch))):
        res = [rand(tokens, h, dtype=torch.float32) for _ in range(COPIES)]
        ys = [rand(tokens, h) for _ in range(COPIES)]
        us = sweep(lambda i: ops.add_rmsnorm(res[i], ys[i], w_norm_bf, 1e-6, torch.bfloat16))
        hbm(f"{tag}_add_rmsnorm (qwen2)", us, tokens * h * (4 + 4 + 2 + 2))
        us = sweep(lambda i: ops.group_norm(ys[i], w_norm, 4, 1e-6, torch.bfloat16, residual=res[i]))
        hbm(f"{tag}_group_norm_add", us, tokens * h * (4 + 4 + 2 + 2))
        # the sum over the chosen experts and the shared expert inside the same kernel
        terms = [rand(tokens, top, h, dtype=torch.float32) for _ in range(COPIES)]
        us = sweep(lambda i: ops.group_norm(terms[i], w_norm, 4, 1e-6, torch.bfloat16, residual=res[i], terms=top, extra=ys[i]))
        hbm(f"{tag}_group_norm_add of expert sum", us, tokens * h * (4 * top + 2 + 4 + 4 + 2))
        del terms
        width = (n_q + 2 * n_kv) * d
        rows = [rand(tokens, width) for _ in range(COPIES)]
        kvs = [torch.zeros((tokens + page - 1) // page + 1, 2, n_kv, page, d, dtype=torch.bfloat16, device=dev) for _ in range(COPIES)]
        positions = torch.arange(tokens, dtype=torch.int32, device=dev)
        inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev)
        qw = rand(d, dtype=torch.float32)
        moved = tokens * d * 2.0 * (2 * n_q + 4 * n_kv)
        us = sweep(lambda i: ops.rope_and_cache(rows[i], positions, positions, inv_freq, kvs[i], n_q, n_kv, d, d))
        hbm(f"{tag}_rope_and_cache (qwen2)", us, moved)
        us = sweep(lambda i: ops.norm_rope_cache(rows[i], positions, positions, kvs[i], n_q, n_kv, d, inv_freq=inv_freq, rotary_dim=d,
                                                 value_inv_freq=inv_freq, value_rotary_dim=d, q_weight=qw, k_weight=qw, norm_dim=d, eps=1e-6))
        hbm(f"{tag}_norm_rope_cache (q/k norm, rotated values)", us, moved)
        outs = [rand(tokens, n_q * d) for _ in range(COPIES)]
        us = sweep(lambda i: ops.turn_heads(outs[i], positions, inv_freq, n_q, d, d))
        hbm(f"{tag}_turn_heads", us, tokens * n_q * d * 4.0)
        del rows, kvs, outs
        # state-space mixer
        proj_w = 2 * inner + 2 * s_g * s_n + s_heads
        projs = [rand(tokens, proj_w) for _ in range(COPIES)]
        w_taps, b_taps = rand(chans, taps, dtype=torch.float32), rand(chans, dtype=torch.float32)
        conv_state = torch.zeros(ctx.num_requests, taps - 1, chans, device=dev)
        us = sweep(lambda i: ops.conv_silu(projs[i], inner, chans, w_taps, b_taps, conv_state, ctx))
        hbm(f"{tag}_conv_silu", us, tokens * chans * 4.0 + ctx.num_requests * (taps - 1) * chans * 8.0)
        xbcs = [rand(tokens, chans) for _ in range(COPIES)]
        dt_bias, a_log, d_skip = (rand(s_heads, dtype=torch.float32) for _ in range(3))
        states = [torch.zeros(ctx.num_requests, s_heads, s_p, s_n, device=dev) for _ in range(COPIES)]
        us = sweep(lambda i: ops.ssm_scan(xbcs[i], projs[i][:, inner + chans:], dt_bias, a_log, d_skip, states[i], ctx, s_heads, s_g, s_p, s_n))
        state_bytes = ctx.num_requests * s_heads * s_p * s_n * 8.0
        hbm(f"{tag}_ssm_scan", us, state_bytes + tokens * (chans * 2.0 + inner * 4.0))
        kernels[f"{tag}_ssm_scan"]["fp32_tflops"] = round(6.0 * tokens * s_heads * s_p * s_n / us / 1e6, 2)
        ysc = [rand(tokens, inner, dtype=torch.float32) for _ in range(COPIES)]
        w_in = rand(inner, dtype=torch.float32)
        us = sweep(lambda i: ops.group_norm(ysc[i], w_in, s_g, 1e-6, torch.bfloat16, gate=projs[i][:, :inner]))
        hbm(f"{tag}_gated_group_norm", us, tokens * inner * 8.0)
        del projs, xbcs, states, ysc
        # routed experts: router, plan + gather + both grouped products; beside the dense gate/up + down of equal work
        xs = [rand(tokens, h) for _ in range(COPIES)]
        w_router = rand(experts, h, std=0.05)
        us = sweep(lambda i: ops.router(xs[i], w_router, top))
        kernels[f"{tag}_router"] = {"us": round(us, 2)}
        ids, scores = ops.router(xs[0], w_router, top)
        gate_up = [rand(experts, 2 * e_ff, h, std=0.02) for _ in range(2)]
        down = [rand(experts, h, e_ff, std=0.02) for _ in range(2)]
        before = ops.launch_count()
        us = sweep(lambda i: ops.moe_experts(xs[i], ids, scores, gate_up[i % 2], down[i % 2], run=64), copies=4)
        touched = len(set(ids.flatten().tolist()))
        if tag == "prefill":
            tensor("prefill_routed_experts (plan, gather, up, down)", us, 6.0 * tokens * top * h * e_ff)
        else:
            hbm("decode_routed_experts (plan, gather, up, down)", us, touched * 3.0 * h * e_ff * 2)
            kernels["decode_routed_experts (plan, gather, up, down)"]["experts_touched"] = touched
        w_gu, w_d = [rand(2 * top * e_ff, h, std=0.02) for _ in range(2)], [rand(h, top * e_ff, std=0.02) for _ in range(2)]
        us = sweep(lambda i: ops.linear(ops.gate_up_swiglu(xs[i], w_gu[i % 2], None, 64), w_d[i % 2]), copies=4)
        if tag == "prefill":
            tensor("prefill_dense gate/up + down of equal work (qwen2)", us, 6.0 * tokens * top * h * e_ff)
        else:
            hbm("decode_dense gate/up + down of equal work (qwen2)", us, 3.0 * h * top * e_ff * 2)
        del gate_up, down, w_gu, w_d, xs

    # attention: a window as long as the context, so that both designs do the same work
    def tables(n_req: int, tokens: int) -> torch.Tensor:
        per = (tokens + page - 1) // page
        return torch.arange(n_req * per, dtype=torch.int32, device=dev).view(n_req, per)

    kv_pages = [rand(batch * ((max(ctx_tokens, T) + page - 1) // page) + 1, 2, n_kv, page, d) for _ in range(COPIES)]
    width = (n_q + 2 * n_kv) * d
    qkv = rand(batch, width)
    att = torch.empty(batch, n_q * d, dtype=torch.bfloat16, device=dev)
    table = tables(batch, ctx_tokens)
    q_start = torch.arange(batch + 1, dtype=torch.int32, device=dev)
    lens = torch.full((batch,), ctx_tokens, dtype=torch.int32, device=dev)
    slices = ops.decode_slices(batch, n_kv, n_q // n_kv, ctx_tokens, False, ops.sm_count(dev))
    nbytes = batch * ctx_tokens * 2.0 * n_kv * d * 2 + 2.0 * batch * n_q * d * 2
    stages = ops.functions.DECODE_RING_STAGES
    us = sweep(lambda i: ops.paged_attention_decode(qkv, qkv.shape[1], att, kv_pages[i], table, q_start, lens, batch, n_q,
                                                    n_kv, d, d ** -0.5, 0, slices, stages=stages))
    hbm("decode_attention (qwen2: rotation outside here)", us, nbytes)
    us = sweep(lambda i: ops.paged_attention_decode(qkv, qkv.shape[1], att, kv_pages[i], table, q_start, lens, batch, n_q,
                                                    n_kv, d, d ** -0.5, ctx_tokens, slices, stages=stages, softcap=50.0))
    hbm("decode_attention window + soft cap", us, nbytes)
    qkv_p = rand(T, width)
    att_p = torch.empty(T, n_q * d, dtype=torch.bfloat16, device=dev)
    table_p, q_start_p = tables(1, T), torch.tensor([0, T], dtype=torch.int32, device=dev)
    lens_p = torch.tensor([T], dtype=torch.int32, device=dev)
    req, tok0 = (torch.from_numpy(a).to(dev) for a in query_tiles_longest_first_host(
        np.asarray([T], dtype=np.int32), np.asarray([T], dtype=np.int32), 128 // (n_q // n_kv)))
    flops = 4.0 * n_q * d * (T * (T + 1) // 2)
    us = sweep(lambda i: ops.paged_attention_prefill_tcgen05(qkv_p, qkv_p.shape[1], att_p, kv_pages[i], table_p, req, tok0,
                                                             q_start_p, lens_p, n_q, n_kv, d, d ** -0.5, 1))
    tensor("prefill_attention tcgen05 (qwen2)", us, flops)
    us = sweep(lambda i: ops.paged_attention_prefill_tcgen05(qkv_p, qkv_p.shape[1], att_p, kv_pages[i], table_p, req, tok0,
                                                             q_start_p, lens_p, n_q, n_kv, d, d ** -0.5, 1, window=T, softcap=50.0))
    tensor("prefill_attention tcgen05 window + soft cap", us, flops)
    half = T // 4
    flops_w = 4.0 * n_q * d * sum(min(t + 1, half) for t in range(T))
    us = sweep(lambda i: ops.paged_attention_prefill_tcgen05(qkv_p, qkv_p.shape[1], att_p, kv_pages[i], table_p, req, tok0,
                                                             q_start_p, lens_p, n_q, n_kv, d, d ** -0.5, 1, window=half, softcap=50.0))
    tensor(f"prefill_attention tcgen05 window of {half} + soft cap", us, flops_w)
    ops.check_errors(dev)
    result["kernels_7b"] = kernels
    print(json.dumps(result))
    return 0


def bezutar_config(z: dict, streams: int) -> dict:
    """config.json of a Bezutar decoder at the layer sizes ``z``: a matrix-memory layer, a latent-attention layer, a
    gated-recurrence layer and a latent-attention layer that reads the rows of the one before, in turn.  The matrix memory
    has the attention's heads and head size; latent attention caches 96 + 32 elements a token (rows of 128, the size the
    tcgen05 attention kernels take); the feed-forward without a gate branch is half again as wide as the gated one, so
    that a token's feed-forward does the same work."""
    rot = dict(base=1000000.0, dims=32, scaling=dict(factor=4.0, original=2048, fast=32.0, slow=1.0))
    layers = []
    for i in range(z["layers"]):
        if i % 4 == 0:
            kind, mixer = "mlstm", dict(heads=z["heads"], dim=z["dim"], vdim=z["dim"], gate_cap=15.0)
        elif i % 4 == 2:
            kind, mixer = "mingru", dict(width=z["width"])
        else:
            kind = "latent_attention"
            mixer = dict(heads=z["heads"], dim=z["dim"], rot_dim=32, vdim=z["dim"], q_rank=max(z["width"] // 4, 256) // 64 * 64,
                         kv_rank=96, scale=(z["dim"] + 32) ** -0.5, rot=rot)
            if i % 4 == 3:
                mixer["kv_from"] = i - 2
        layers.append(dict(type=kind, mixer=mixer, mlp=dict(kind="dense", ff=z["ff"] * 3 // 2)))
    return dict(architecture="Bezutar", vocab=z["vocab"], width=z["width"], streams=streams, norm=dict(eps=1e-6),
                canon=dict(taps=4), embedding=dict(bigram=dict(buckets=65521, mul_prev=1000003, mul_cur=31)),
                max_positions=8192, layers=layers)


def run_compare_bezutar(args) -> int:
    """The Bezutar decoder beside the Qwen2.5 decoder at equal layer sizes (whole steps), then every kernel the design
    adds, alone at the 7B layer sizes, beside its nearest relative among the kernels of the other decoders."""
    import numpy as np
    import torch

    from slipstream_b200 import ops
    from slipstream_b200.engine.context import query_tiles_longest_first_host

    pk, pk_kind = peaks()
    rng = np.random.default_rng(0)
    dev = torch.device("cuda:0")
    batch, ctx_tokens, T, page = args.batch, args.prompt_len, args.chunk, 16
    result: dict = {"compare": "bezutar", "peaks": pk_kind, "batch": batch, "context": ctx_tokens, "prefill_tokens": T,
                    "streams": args.streams, "sizes": {}}
    for name in (args.sizes.split(",") if args.sizes else COMPARE_SIZES):
        qwen, _ = compare_configs(COMPARE_SIZES[name], 8192, 1, False)
        result["sizes"][name] = {}
        for which, config in (("qwen2", qwen), ("bezutar", bezutar_config(COMPARE_SIZES[name], args.streams))):
            if which == "qwen2" and args.skip_qwen2:
                continue
            print(f"[bench] {name} {which} ...", file=sys.stderr, flush=True)
            result["sizes"][name][which] = measure_model(config, args, pk, rng)
            print(f"[bench] {name} {which}: {result['sizes'][name][which]}", file=sys.stderr, flush=True)
    if args.no_kernels:
        print(json.dumps(result))
        return 0

    print("[bench] single kernels ...", file=sys.stderr, flush=True)
    z = COMPARE_SIZES["7b"]
    h, n_q, n_kv, d, inter = z["width"], z["heads"], z["kv_heads"], z["dim"], z["ff"]
    lat = bezutar_config(z, args.streams)["layers"][1]["mixer"]
    q_rank, kv_rank, rot_dim = lat["q_rank"], lat["kv_rank"], lat["rot_dim"]
    row = kv_rank + rot_dim
    ff = inter * 3 // 2
    gen = torch.Generator(device=dev).manual_seed(1)
    COPIES = 6  # operands of each timed launch rotate through this many copies

    def rand(*shape, dtype=torch.bfloat16, std=0.5):
        return (torch.randn(*shape, generator=gen, device=dev) * std).to(dtype)

    def sweep(run, copies=COPIES) -> float:
        for i in range(copies):
            run(i)
        times = []
        for _ in range(5):
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(copies):
                run(i)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e3 / copies)
        return sorted(times)[2]

    kernels: dict = {}

    def hbm(name: str, us: float, nbytes: float, **more) -> None:
        gbs = nbytes / (us * 1e-6) / 1e9
        kernels[name] = {"us": round(us, 2), "gbs": round(gbs, 1), "hbm_frac": round(gbs / pk["hbm_gbs"], 3), **more}

    def tensor(name: str, us: float, flops: float) -> None:
        tf = flops / (us * 1e-6) / 1e12
        kernels[name] = {"us": round(us, 2), "tflops": round(tf, 1), "bf16_frac": round(tf / pk["bf16_tflops"], 3)}

    def step(q_lens, seq_lens):
        starts = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
        as_dev = lambda v: torch.tensor(np.asarray(v), dtype=torch.int32, device=dev)  # noqa: E731
        positions = np.concatenate([np.arange(s - n, s) for n, s in zip(q_lens, seq_lens)])
        return types.SimpleNamespace(q_start=as_dev(starts), seq_lens=as_dev(seq_lens), state_slots=as_dev(np.arange(len(q_lens))),
                                     positions=as_dev(positions), num_requests=len(q_lens),
                                     is_decode_only=all(n == 1 for n in q_lens))

    table_rows = 65536  # rows of each embedding table here: rows are gathered, the tables' size does not matter
    tables3 = [rand(table_rows, h) for _ in range(3)]
    for tokens, tag, ctx in ((T, "prefill", step([T], [T])), (batch, "decode", step([1] * batch, [ctx_tokens] * batch))):
        R = ctx.num_requests
        # embedding
        ids = torch.randint(0, table_rows, (tokens,), generator=gen, device=dev, dtype=torch.int32)
        last = torch.zeros(R, dtype=torch.int32, device=dev)
        us = sweep(lambda i: ops.embedding(ids, tables3[0]))
        hbm(f"{tag}_embedding (qwen2)", us, tokens * h * (2 + 4))
        us = sweep(lambda i: ops.embed_sum(ids, tables3[0], ctx, pair_table=tables3[1][:65522], pair_hash=(65521, 1000003, 31),
                                           last_token=last, position_table=tables3[2][:8192], copies=args.streams))
        hbm(f"{tag}_embed_sum (3 rows into {args.streams} streams)", us, tokens * h * (3 * 2 + 4 * args.streams))
        # the convolution over a mixer's input, beside the state-space layers' convolution over as many channels
        xs = [rand(tokens, h) for _ in range(COPIES)]
        w_taps = rand(h, 4, dtype=torch.float32)
        conv_state = torch.zeros(R, 3, h, device=dev)
        us = sweep(lambda i: ops.conv_silu(xs[i], 0, h, w_taps, None, conv_state, ctx))
        hbm(f"{tag}_conv_silu (sarudra)", us, tokens * h * 4.0 + R * 3 * h * 8.0)
        us = sweep(lambda i: ops.conv_silu(xs[i], 0, h, w_taps, None, conv_state, ctx, plus_input=True))
        hbm(f"{tag}_input + convolution", us, tokens * h * 4.0 + R * 3 * h * 8.0)
        # matrix memory: the cell and its output norm, beside the state-space scan of equal state (heads x 128 x 128)
        qkvg = [rand(tokens, n_q * 4 * d) for _ in range(COPIES)]
        gates = [rand(tokens, 2 * n_q, dtype=torch.float32, std=3.0) for _ in range(COPIES)]
        bias = rand(n_q, dtype=torch.float32)
        memory = [torch.zeros(R, n_q, d + 1, d, device=dev) for _ in range(COPIES)]
        peak = torch.zeros(R, n_q, device=dev)
        us = sweep(lambda i: ops.matrix_cell(qkvg[i], gates[i], bias, bias, 15.0, d ** -0.5, memory[i], peak, ctx, n_q, d, d))
        state_bytes = R * n_q * (d + 1) * d * 8.0
        hbm(f"{tag}_matrix_cell", us, state_bytes + tokens * n_q * d * (3 * 2.0 + 4.0),
            fp32_tflops=round(6.0 * tokens * n_q * (d + 1) * d / us / 1e6, 2))
        num, nq, peaks_t = ops.matrix_cell(qkvg[0], gates[0], bias, bias, 15.0, d ** -0.5, memory[0], peak, ctx, n_q, d, d)
        w_cell = rand(n_q * d, dtype=torch.float32)
        us = sweep(lambda i: ops.cell_output(num, nq, peaks_t, w_cell, qkvg[i][:, 3 * n_q * d:], n_q, d, 1e-6, torch.bfloat16))
        hbm(f"{tag}_cell_output (head norm, gate)", us, tokens * n_q * d * (4.0 + 2.0 + 2.0))
        s_heads, s_p, s_n, s_g = n_q, d, d, 4
        chans = s_heads * s_p + 2 * s_g * s_n
        xbcs = [rand(tokens, chans) for _ in range(COPIES)]
        dts = [rand(tokens, s_heads) for _ in range(COPIES)]
        dt_bias, a_log, d_skip = (rand(s_heads, dtype=torch.float32) for _ in range(3))
        states = [torch.zeros(R, s_heads, s_p, s_n, device=dev) for _ in range(COPIES)]
        us = sweep(lambda i: ops.ssm_scan(xbcs[i], dts[i], dt_bias, a_log, d_skip, states[i], ctx, s_heads, s_g, s_p, s_n))
        hbm(f"{tag}_ssm_scan of equal state (sarudra)", us, R * s_heads * s_p * s_n * 8.0 + tokens * (chans * 2.0 + s_heads * s_p * 4.0),
            fp32_tflops=round(6.0 * tokens * s_heads * s_p * s_n / us / 1e6, 2))
        del qkvg, gates, memory, xbcs, dts, states, num
        # gated recurrence
        projs = [rand(tokens, 3 * h) for _ in range(COPIES)]
        cell = torch.zeros(R, h, device=dev)
        bias2 = rand(2 * h, dtype=torch.float32)
        us = sweep(lambda i: ops.gated_recurrence(projs[i], h, cell, ctx, bias=bias2))
        hbm(f"{tag}_gated_recurrence", us, tokens * h * (3 * 2.0 + 2.0) + R * h * 8.0)
        del projs
        # feed-forward activation
        ups = [rand(tokens, ff) for _ in range(COPIES)]
        us = sweep(lambda i: ops.xielu(ups[i], 0.7, 1.2))
        hbm(f"{tag}_xielu (in place)", us, tokens * ff * 4.0)
        gus = [rand(tokens, 2 * inter) for _ in range(COPIES)]
        us = sweep(lambda i: ops.swiglu(gus[i], block=64))
        hbm(f"{tag}_swiglu by itself (qwen2)", us, tokens * inter * 6.0)
        del ups, gus
        # latent attention: latents, rotation and page write; the products per head
        positions = ctx.positions
        slots = torch.arange(tokens, dtype=torch.int32, device=dev)
        downs = [rand(tokens, (q_rank + row + n_q + 7) // 8 * 8) for _ in range(COPIES)]
        kvs = [torch.zeros((tokens + page - 1) // page + 1, 2, 1, page, row, dtype=torch.bfloat16, device=dev) for _ in range(COPIES)]
        inv_freq = (1.0 / (1e6 ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))).to(dev)
        qw, kw = rand(q_rank, dtype=torch.float32), rand(kv_rank, dtype=torch.float32)
        us = sweep(lambda i: ops.latent_rows(downs[i], positions, slots, kvs[i], qw, kw, inv_freq, 1.1, q_rank, kv_rank, rot_dim, 1e-6))
        hbm(f"{tag}_latent_rows (two norms, rotation, page write)", us, tokens * 2.0 * (2 * q_rank + row + 2 * row))
        width = (n_q + 2 * n_kv) * d
        rows = [rand(tokens, width) for _ in range(COPIES)]
        kvq = [torch.zeros((tokens + page - 1) // page + 1, 2, n_kv, page, d, dtype=torch.bfloat16, device=dev) for _ in range(COPIES)]
        inv_d = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev)
        us = sweep(lambda i: ops.rope_and_cache(rows[i], positions, slots, inv_d, kvq[i], n_q, n_kv, d, d))
        hbm(f"{tag}_rope_and_cache (qwen2)", us, tokens * d * 2.0 * (2 * n_q + 4 * n_kv))
        del rows, kvq, kvs
        qs = [rand(tokens, n_q * (d + rot_dim)) for _ in range(COPIES)]
        to_latent, to_value = rand(n_q, d, kv_rank, std=0.1), rand(n_q, kv_rank, d, std=0.1)
        q_lat = torch.empty(tokens, n_q * row, dtype=torch.bfloat16, device=dev)
        us = sweep(lambda i: ops.head_product(qs[i], d + rot_dim, to_latent, q_lat, row, turn=rot_dim, pad_to=row, positions=positions,
                                              inv_freq=inv_freq, mscale=1.1))
        flops = 2.0 * tokens * n_q * d * kv_rank
        moved = tokens * n_q * (d + rot_dim + row) * 2.0 + n_q * d * kv_rank * 2.0
        kernels[f"{tag}_head_product into the latent space (+ rotation)"] = {
            "us": round(us, 2), "tflops": round(flops / us / 1e6, 2), "gbs": round(moved / us / 1e3, 1),
            "hbm_frac": round(moved / us / 1e3 / pk["hbm_gbs"], 3)}
        vals = torch.empty(tokens, n_q * d, dtype=torch.bfloat16, device=dev)
        mixed = [rand(tokens, n_q * row) for _ in range(COPIES)]
        us = sweep(lambda i: ops.head_product(mixed[i], row, to_value, vals, d, gates=downs[i][:, q_rank + row: q_rank + row + n_q]))
        moved = tokens * n_q * (row + d) * 2.0 + n_q * d * kv_rank * 2.0
        kernels[f"{tag}_head_product up to values (+ gate)"] = {
            "us": round(us, 2), "tflops": round(flops / us / 1e6, 2), "gbs": round(moved / us / 1e3, 1),
            "hbm_frac": round(moved / us / 1e3 / pk["hbm_gbs"], 3)}
        del qs, mixed, downs

    # attention: every design's own kernel over the same number of cached tokens
    def tables(n_req: int, tokens: int) -> torch.Tensor:
        per = (tokens + page - 1) // page
        return torch.arange(n_req * per, dtype=torch.int32, device=dev).view(n_req, per)

    n_pages = batch * ((max(ctx_tokens, T) + page - 1) // page) + 1
    sinks = rand(n_q, dtype=torch.float32)
    q_start = torch.arange(batch + 1, dtype=torch.int32, device=dev)
    lens = torch.full((batch,), ctx_tokens, dtype=torch.int32, device=dev)
    table = tables(batch, ctx_tokens)
    stages = ops.functions.DECODE_RING_STAGES
    kv_pages = [rand(n_pages, 2, n_kv, page, d) for _ in range(COPIES)]
    qkv = rand(batch, (n_q + 2 * n_kv) * d)
    att = torch.empty(batch, n_q * d, dtype=torch.bfloat16, device=dev)
    slices = ops.decode_slices(batch, n_kv, n_q // n_kv, ctx_tokens, False, ops.sm_count(dev))
    us = sweep(lambda i: ops.paged_attention_decode(qkv, qkv.shape[1], att, kv_pages[i], table, q_start, lens, batch, n_q,
                                                    n_kv, d, d ** -0.5, 0, slices, stages=stages))
    hbm(f"decode_attention (qwen2: {n_q} heads on {n_kv} cached heads of {d})", us, batch * ctx_tokens * 2.0 * n_kv * d * 2 + 2.0 * batch * n_q * d * 2)
    qkv_p = rand(T, (n_q + 2 * n_kv) * d)
    att_p = torch.empty(T, n_q * d, dtype=torch.bfloat16, device=dev)
    table_p, q_start_p = tables(1, T), torch.tensor([0, T], dtype=torch.int32, device=dev)
    lens_p = torch.tensor([T], dtype=torch.int32, device=dev)
    req, tok0 = (torch.from_numpy(a).to(dev) for a in query_tiles_longest_first_host(
        np.asarray([T], dtype=np.int32), np.asarray([T], dtype=np.int32), 128 // (n_q // n_kv)))
    us = sweep(lambda i: ops.paged_attention_prefill_tcgen05(qkv_p, qkv_p.shape[1], att_p, kv_pages[i], table_p, req, tok0,
                                                             q_start_p, lens_p, n_q, n_kv, d, d ** -0.5, 1))
    tensor("prefill_attention tcgen05 (qwen2)", us, 4.0 * n_q * d * (T * (T + 1) // 2))
    del kv_pages
    lat_pages = [rand(n_pages, 2, 1, page, row) for _ in range(COPIES)]
    q_lat = rand(batch, n_q * row)
    att_l = torch.empty(batch, n_q * row, dtype=torch.bfloat16, device=dev)
    slices = ops.decode_slices(batch, 1, n_q, ctx_tokens, False, ops.sm_count(dev))
    us = sweep(lambda i: ops.paged_attention_decode(q_lat, q_lat.shape[1], att_l, lat_pages[i], table, q_start, lens, batch, n_q,
                                                    1, row, 0.08, 0, slices, stages=stages, sinks=sinks))
    hbm(f"decode_attention with sinks ({n_q} heads on one cached row of {row})", us, batch * ctx_tokens * 2.0 * row * 2 + 2.0 * batch * n_q * row * 2)
    q_lat_p = rand(T, n_q * row)
    att_lp = torch.empty(T, n_q * row, dtype=torch.bfloat16, device=dev)
    if ops.tcgen05_prefill_fits(row, n_q, 1, page):
        req, tok0 = (torch.from_numpy(a).to(dev) for a in query_tiles_longest_first_host(
            np.asarray([T], dtype=np.int32), np.asarray([T], dtype=np.int32), 128 // n_q))
        parts = ops.prefill_key_parts(np.asarray([T], dtype=np.int32), np.asarray([T], dtype=np.int32), 128 // n_q, 1)
        us = sweep(lambda i: ops.paged_attention_prefill_tcgen05(q_lat_p, q_lat_p.shape[1], att_lp, lat_pages[i], table_p, req, tok0,
                                                                 q_start_p, lens_p, n_q, 1, row, 0.08, parts, sinks=sinks))
        tensor(f"prefill_attention tcgen05 with sinks ({n_q} heads on one cached row of {row})", us, 4.0 * n_q * row * (T * (T + 1) // 2))
    ops.check_errors(dev)
    result["kernels_7b"] = kernels
    print(json.dumps(result))
    return 0


def lakadra_config(z: dict, window: int) -> dict:
    """config.json of a Lakadra decoder at the layer sizes ``z``: a decayed linear-attention layer, a latent-attention
    layer, a pair of windowed attention and gated linear recurrence, and a latent-attention layer that reads the rows of
    the other, in turn.  Linear attention has the attention's heads and head size; latent attention caches 96 + 32
    elements a token; the recurrence has the model's width in blocks of 256.  Every feed-forward is routed: two of eight
    un-gated experts (and two pass-through experts) in five groups of which three are kept, beside a shared expert,
    sized so that a token's feed-forward does the work of the dense gated one."""
    rot = dict(base=1000000.0, dims=32)
    ff_e, ff_s = z["ff"] * 3 // 8 // 64 * 64, z["ff"] * 3 // 4 // 64 * 64
    mlp = dict(kind="moe", expert=dict(ff=ff_e), shared=dict(ff=ff_s),
               router=dict(experts=8, identity=2, top=2, groups=dict(count=5, keep=3)))
    layers = []
    for i in range(z["layers"]):
        if i % 4 == 0:
            kind = "lightning"
            mixer = dict(heads=z["heads"], dim=z["dim"], vdim=z["dim"], decay=[1.0 - 2.0 ** -(2 + 6 * h / z["heads"]) for h in range(z["heads"])])
        elif i % 4 == 2:
            kind = "parallel"
            mixer = dict(left=dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=z["dim"], vdim=z["dim"], scale=z["dim"] ** -0.5,
                                   mask=dict(size=window), rot=dict(base=1000000.0, dims=z["dim"] // 2, scaling=dict(factor=8.0))),
                         right=dict(width=z["width"], blocks=z["width"] // 256 if z["width"] % 256 == 0 else z["width"] // 128, conv=4),
                         left_scale=1.2, right_scale=0.9)
        else:
            kind = "latent_attention"
            mixer = dict(heads=z["heads"], dim=z["dim"], rot_dim=32, vdim=z["dim"], q_rank=max(z["width"] // 4, 256) // 64 * 64,
                         kv_rank=96, scale=(z["dim"] + 32) ** -0.5, rot=rot)
            if i % 4 == 3:
                mixer["kv_from"] = i - 2
        layers.append(dict(type=kind, mixer=mixer, mlp=mlp))
    return dict(architecture="Lakadra", vocab=z["vocab"], width=z["width"], norm=dict(eps=1e-6), logit_scale=2.0,
                logit_softcap=30.0, layers=layers, max_position_embeddings=8192)


def run_compare_lakadra(args) -> int:
    """The Lakadra decoder beside the Qwen2.5 decoder at equal layer sizes (whole steps), then every kernel the design
    adds, alone at the 7B layer sizes, beside its nearest relative among the kernels of the other decoders."""
    import numpy as np
    import torch

    from slipstream_b200 import ops

    pk, pk_kind = peaks()
    rng = np.random.default_rng(0)
    dev = torch.device("cuda:0")
    batch, ctx_tokens, T = args.batch, args.prompt_len, args.chunk
    result: dict = {"compare": "lakadra", "peaks": pk_kind, "batch": batch, "context": ctx_tokens, "prefill_tokens": T,
                    "window": args.window, "sizes": {}}
    for name in (args.sizes.split(",") if args.sizes else COMPARE_SIZES):
        qwen, _ = compare_configs(COMPARE_SIZES[name], 8192, 1, False)
        result["sizes"][name] = {}
        for which, config in (("qwen2", qwen), ("lakadra", lakadra_config(COMPARE_SIZES[name], args.window))):
            if which == "qwen2" and args.skip_qwen2:
                continue
            print(f"[bench] {name} {which} ...", file=sys.stderr, flush=True)
            result["sizes"][name][which] = measure_model(config, args, pk, rng)
            print(f"[bench] {name} {which}: {result['sizes'][name][which]}", file=sys.stderr, flush=True)
    if args.no_kernels:
        print(json.dumps(result))
        return 0

    print("[bench] single kernels ...", file=sys.stderr, flush=True)
    z = COMPARE_SIZES["7b"]
    h, n_q, d, inter = z["width"], z["heads"], z["dim"], z["ff"]
    cfg = lakadra_config(z, args.window)
    ff_e, ff_s = cfg["layers"][0]["mlp"]["expert"]["ff"], cfg["layers"][0]["mlp"]["shared"]["ff"]
    blocks = cfg["layers"][2]["mixer"]["right"]["blocks"]
    bs = h // blocks
    gen = torch.Generator(device=dev).manual_seed(1)
    COPIES = 6  # operands of each timed launch rotate through this many copies

    def rand(*shape, dtype=torch.bfloat16, std=0.5):
        return (torch.randn(*shape, generator=gen, device=dev) * std).to(dtype)

    def sweep(run, copies=COPIES) -> float:
        for i in range(copies):
            run(i)
        times = []
        for _ in range(5):
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(copies):
                run(i)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e3 / copies)
        return sorted(times)[2]

    kernels: dict = {}

    def hbm(name: str, us: float, nbytes: float, **more) -> None:
        gbs = nbytes / (us * 1e-6) / 1e9
        kernels[name] = {"us": round(us, 2), "gbs": round(gbs, 1), "hbm_frac": round(gbs / pk["hbm_gbs"], 3), **more}

    def tensor(name: str, us: float, flops: float) -> None:
        tf = flops / (us * 1e-6) / 1e12
        kernels[name] = {"us": round(us, 2), "tflops": round(tf, 1), "bf16_frac": round(tf / pk["bf16_tflops"], 3)}

    def step(q_lens, seq_lens):
        starts = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
        as_dev = lambda v: torch.tensor(np.asarray(v), dtype=torch.int32, device=dev)  # noqa: E731
        positions = np.concatenate([np.arange(s - n, s) for n, s in zip(q_lens, seq_lens)])
        return types.SimpleNamespace(q_start=as_dev(starts), seq_lens=as_dev(seq_lens), state_slots=as_dev(np.arange(len(q_lens))),
                                     positions=as_dev(positions), num_requests=len(q_lens),
                                     is_decode_only=all(n == 1 for n in q_lens))

    one = torch.ones(1, device=dev)
    for tokens, tag, ctx in ((T, "prefill", step([T], [T])), (batch, "decode", step([1] * batch, [ctx_tokens] * batch))):
        R = ctx.num_requests
        # the norm in front of a layer, which adds the two outputs of the layer before; beside the add + norm of one
        streams = [rand(tokens, 1, h, dtype=torch.float32) for _ in range(COPIES)]
        ys, y2s = [rand(tokens, h) for _ in range(COPIES)], [rand(tokens, h) for _ in range(COPIES)]
        w_norm = rand(h, dtype=torch.float32)
        us = sweep(lambda i: ops.add_rmsnorm(streams[i][:, 0], ys[i], w_norm, 1e-6, torch.bfloat16))
        hbm(f"{tag}_add_rmsnorm (qwen2)", us, tokens * h * (4 + 4 + 2 + 2))
        us = sweep(lambda i: ops.hc_norm(streams[i], ys[i], one.view(1, 1), one, None, w_norm, 1e-6, torch.bfloat16, y2=y2s[i]))
        hbm(f"{tag}_norm that adds two outputs", us, tokens * h * (4 + 4 + 2 + 2 + 2))
        del streams, y2s
        # linear attention with a decay per head and its gated norm, beside the matrix memory of equal state
        qkvg = [rand(tokens, n_q * 4 * d) for _ in range(COPIES)]
        decay = torch.full((n_q,), 0.99, device=dev)
        memory = [torch.zeros(R, n_q, d, d, device=dev) for _ in range(COPIES)]
        us = sweep(lambda i: ops.decay_attention(qkvg[i], decay, memory[i], ctx, n_q, d, d))
        hbm(f"{tag}_decay_attention", us, R * n_q * d * d * 8.0 + tokens * n_q * d * (3 * 2.0 + 4.0),
            fp32_tflops=round(4.0 * tokens * n_q * d * d / us / 1e6, 2))
        gates = [rand(tokens, 2 * n_q, dtype=torch.float32, std=3.0) for _ in range(COPIES)]
        bias = rand(n_q, dtype=torch.float32)
        memory1 = [torch.zeros(R, n_q, d + 1, d, device=dev) for _ in range(COPIES)]
        peak = torch.zeros(R, n_q, device=dev)
        us = sweep(lambda i: ops.matrix_cell(qkvg[i], gates[i], bias, bias, 15.0, d ** -0.5, memory1[i], peak, ctx, n_q, d, d))
        hbm(f"{tag}_matrix_cell of equal state (bezutar)", us, R * n_q * (d + 1) * d * 8.0 + tokens * n_q * d * (3 * 2.0 + 4.0),
            fp32_tflops=round(6.0 * tokens * n_q * (d + 1) * d / us / 1e6, 2))
        num, nq, peaks_t = ops.matrix_cell(qkvg[0], gates[0], bias, bias, 15.0, d ** -0.5, memory1[0], peak, ctx, n_q, d, d)
        w_cell = rand(n_q * d, dtype=torch.float32)
        us = sweep(lambda i: ops.cell_output(num, nq, peaks_t, w_cell, qkvg[i][:, 3 * n_q * d:], n_q, d, 1e-6, torch.bfloat16))
        hbm(f"{tag}_cell_output (bezutar: head norm, gate)", us, tokens * n_q * d * (4.0 + 2.0 + 2.0))
        mixed = ops.decay_attention(qkvg[0], decay, memory[0], ctx, n_q, d, d)
        us = sweep(lambda i: ops.gated_rmsnorm(mixed, qkvg[i][:, 3 * n_q * d:], w_cell, 1e-6, torch.bfloat16))
        hbm(f"{tag}_gated_rmsnorm (norm over all heads, gate)", us, tokens * n_q * d * (4.0 + 2.0 + 2.0))
        del qkvg, gates, memory, memory1, num, mixed
        # the gated linear recurrence: convolution, gates from square blocks, the recurrence; beside the gated recurrence
        # per channel of the Bezutar decoder
        projs = [rand(tokens, 2 * h) for _ in range(COPIES)]
        w_taps, b_taps = rand(h, 4, dtype=torch.float32), rand(h, dtype=torch.float32)
        conv_state = torch.zeros(R, 3, h, device=dev)
        us = sweep(lambda i: ops.conv_silu(projs[i], h, h, w_taps, b_taps, conv_state, ctx, activation=False))
        hbm(f"{tag}_convolution (no activation)", us, tokens * h * 4.0 + R * 3 * h * 8.0)
        us = sweep(lambda i: ops.conv_silu(projs[i], h, h, w_taps, b_taps, conv_state, ctx))
        hbm(f"{tag}_conv_silu (sarudra)", us, tokens * h * 4.0 + R * 3 * h * 8.0)
        us_ = [rand(tokens, h) for _ in range(COPIES)]
        gate_w = rand(blocks, 2 * bs, bs, std=0.05)
        us = sweep(lambda i: ops.block_gates(us_[i], gate_w))
        flops = 4.0 * tokens * h * bs
        moved = tokens * h * (2.0 + 8.0) + gate_w.numel() * 2.0
        kernels[f"{tag}_block_gates ({blocks} blocks of {bs})"] = {
            "us": round(us, 2), "tflops": round(flops / us / 1e6, 2), "bf16_frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3),
            "gbs": round(moved / us / 1e3, 1), "hbm_frac": round(moved / us / 1e3 / pk["hbm_gbs"], 3)}
        pre = ops.block_gates(us_[0], gate_w)
        gate_b, lam = rand(blocks, 2 * bs, dtype=torch.float32), rand(h, dtype=torch.float32)
        cell = torch.zeros(R, h, device=dev)
        us = sweep(lambda i: ops.gated_linear_recurrence(pre, gate_b, us_[i], projs[i][:, :h], lam, 8.0, cell, ctx))
        hbm(f"{tag}_gated_linear_recurrence", us, tokens * h * (8.0 + 3 * 2.0) + R * h * 8.0)
        projs3 = [rand(tokens, 3 * h) for _ in range(COPIES)]
        bias2 = rand(2 * h, dtype=torch.float32)
        us = sweep(lambda i: ops.gated_recurrence(projs3[i], h, cell, ctx, bias=bias2))
        hbm(f"{tag}_gated_recurrence (bezutar)", us, tokens * h * (3 * 2.0 + 2.0) + R * h * 8.0)
        del projs, projs3, us_, pre
        # small kernels around the attention of a pair of mixers
        outs = [rand(tokens, n_q * d) for _ in range(COPIES)]
        hg = rand(tokens, 32)
        us = sweep(lambda i: ops.head_gate(outs[i], hg[:, :n_q], n_q, d))
        hbm(f"{tag}_head_gate (in place)", us, tokens * n_q * d * 4.0)
        us = sweep(lambda i: ops.sigmoid_gate(outs[i], outs[(i + 1) % COPIES]))
        hbm(f"{tag}_sigmoid_gate (fokedra, in place)", us, tokens * n_q * d * 6.0)
        us = sweep(lambda i: ops.scaled_sum(ys[i], 1.2, ys[(i + 1) % COPIES], 0.9))
        hbm(f"{tag}_scaled_sum of two mixers", us, tokens * h * 6.0)
        del outs
        # the routed feed-forward: router, experts, weighted sum; beside the gated experts of the Sarudra decoder of
        # equal work (two of eight, expert size a quarter of the dense one)
        xs = [rand(tokens, h) for _ in range(COPIES)]
        w_router = rand(11, h, std=0.05)
        corr = rand(10, dtype=torch.float32, std=0.05)
        us = sweep(lambda i: ops.router(xs[i], w_router, 2, softmax=True, correction=corr, groups=5, keep=3, extra=1))
        kernels[f"{tag}_router (softmax, correction, groups, a gate's row)"] = {"us": round(us, 2)}
        w8 = w_router[:8].contiguous()
        us = sweep(lambda i: ops.router(xs[i], w8, 2))
        kernels[f"{tag}_router (sarudra: sigmoid)"] = {"us": round(us, 2)}
        ids, scores, sg = ops.router(xs[0], w_router, 2, softmax=True, correction=corr, groups=5, keep=3, extra=1)
        up, down = rand(8, ff_e, h, std=0.02), rand(8, h, ff_e, std=0.02)
        us = sweep(lambda i: ops.moe_experts_single(xs[i], ids, up, down, 10))
        touched = int(torch.unique(ids[ids < 8]).numel())
        flops = 4.0 * int((ids < 8).sum()) * h * ff_e
        moved = touched * 2 * ff_e * h * 2.0
        kernels[f"{tag}_un-gated experts (plan, gather, up, down)"] = {
            "us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "bf16_frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3),
            "gbs": round(moved / us / 1e3, 1), "hbm_frac": round(moved / us / 1e3 / pk["hbm_gbs"], 3), "experts_touched": touched}
        ff_g = inter // 4 // 64 * 64
        gate_up, down_g = rand(8, 2 * ff_g, h, std=0.02), rand(8, h, ff_g, std=0.02)
        ids8, scores8 = ops.router(xs[0], w8, 2)
        us = sweep(lambda i: ops.moe_experts(xs[i], ids8, scores8, gate_up, down_g, 64))
        touched8 = int(torch.unique(ids8).numel())
        flops = 6.0 * tokens * 2 * h * ff_g
        moved = touched8 * 3 * ff_g * h * 2.0
        kernels[f"{tag}_gated experts of equal work (sarudra)"] = {
            "us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "bf16_frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3),
            "gbs": round(moved / us / 1e3, 1), "hbm_frac": round(moved / us / 1e3 / pk["hbm_gbs"], 3), "experts_touched": touched8}
        y, term_rows = ops.moe_experts_single(xs[0], ids, up, down, 10)
        shared = rand(tokens, h)
        us = sweep(lambda i: ops.moe_mix(y, term_rows, ids, scores, 8, xs[i], shared, sg))
        hbm(f"{tag}_moe_mix (weights, pass-through, gated shared expert)", us, tokens * h * (2 * (2.0 if term_rows is not None else 4.0) + 6.0))
        y8, rows8 = ops.moe_experts(xs[0], ids8, scores8, gate_up, down_g, 64)
        us = sweep(lambda i: ops.moe_combine(y8, shared, torch.bfloat16, rows8, 2))
        hbm(f"{tag}_moe_combine (sarudra)", us, tokens * h * (2 * (2.0 if rows8 is not None else 4.0) + 4.0))
        ups = [rand(tokens, ff_s) for _ in range(COPIES)]
        us = sweep(lambda i: ops.relu_square(ups[i]))
        hbm(f"{tag}_relu_square", us, tokens * ff_s * 4.0)
        us = sweep(lambda i: ops.xielu(ups[i], 0.7, 1.2))
        hbm(f"{tag}_xielu (bezutar)", us, tokens * ff_s * 4.0)
        del xs, ups, y, y8, up, down, gate_up, down_g, ys
    ops.check_errors(dev)
    result["kernels_7b"] = kernels
    print(json.dumps(result))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=SHAPE_7B["num_hidden_layers"])
    ap.add_argument("--context-len", type=int, default=SHAPE_7B["max_position_embeddings"],
                    help="positions of the model (with --only: measurements at longer contexts)")
    ap.add_argument("--chunk", type=int, default=2048, help="--only prefill: tokens of the timed prompt portion")
    ap.add_argument("--prefix", type=int, default=0, help="--only prefill: tokens already cached in front of it")
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel timings")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=None,
                    help="run another measured workload end to end through the scheduler instead")
    ap.add_argument("--window", type=int, default=4096, help="--compare sarudra: positions of the sliding window")
    ap.add_argument("--compare", choices=["fokedra", "sarudra", "bezutar", "lakadra"], default=None,
                    help="time another decoder design beside the Qwen2.5 decoder at equal layer sizes instead")
    ap.add_argument("--sizes", default="", help="--compare: which of 0.5b,7b,14b (default: all)")
    ap.add_argument("--mask-chunk", type=int, default=8192, help="--compare: positions per attention chunk")
    ap.add_argument("--streams", type=int, default=2, help="--compare: residual streams")
    ap.add_argument("--skip-qwen2", action="store_true", help="--compare: time the other design only")
    ap.add_argument("--share-kv", action="store_true", help="--compare: every second layer reads the pages of the layer before")
    ap.add_argument("--only", choices=["decode", "prefill", "gemm", "attention"], default=None,
                    help="run just this part and print a short line (for profiling); gemm / attention: tables of "
                         "single kernels at several sizes")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (this engine uses a single device); got --gpus {args.gpus}")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.compare:
        if args.steps == 256:
            args.steps = 64
        args.warmup = max(args.warmup, 3)
        if args.compare == "bezutar":
            return run_compare_bezutar(args)
        if args.compare == "lakadra":
            return run_compare_lakadra(args)
        return run_compare_sarudra(args) if args.compare == "sarudra" else run_compare(args)
    if args.workload:
        return run_workload(args.workload, args)
    if args.only in ("gemm", "attention"):
        return kernel_tables(args.only)
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch

    from slipstream_b200 import CacheConfig, EngineConfig, SamplingParams, SchedulerConfig, ops
    from slipstream_b200.engine.llm_engine import LLMEngine, Request
    from slipstream_b200.engine.runner import StepEntry

    pk, pk_kind = peaks()
    shape = dict(SHAPE_7B, num_hidden_layers=args.layers, max_position_embeddings=args.context_len)
    folder = tempfile.mkdtemp(prefix="bench_qwen7b_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(shape, architectures=["Qwen2ForCausalLM"], model_type="qwen2"), f)
    ctx_len, page = shape["max_position_embeddings"], 16
    max_batch = max(64, args.batch)
    pages = max_batch * (args.prompt_len + args.steps + args.warmup + 2 * max_batch + 96) // page + 4096 // page + 64
    if args.only:  # one batch, or one prompt behind a prefix: the pool need not hold 64 requests
        pages = (max(args.batch * (args.prompt_len + args.steps + args.warmup + 16), args.prefix + args.chunk) + 4096) // page + 64
    engine = LLMEngine(EngineConfig.for_model(
        folder, dtype="bfloat16", load_format="random", max_model_len=ctx_len,
        cache=CacheConfig(block_size=page, num_gpu_blocks=pages),
        scheduler=SchedulerConfig(max_num_seqs=max_batch, max_num_batched_tokens=8192, prefill_chunk_size=2048),
        seed=0, use_cuda_graphs=not args.no_graphs))
    runner = engine.runner
    vocab = shape["vocab_size"]
    rng = np.random.default_rng(0)
    torch.cuda.synchronize()

    def fill(batch: int, tag: str) -> list[str]:
        """Prefill ``batch`` requests of prompt_len random tokens (untimed)."""
        ids = [f"{tag}{i}" for i in range(batch)]
        if args.prompt_len > 4096:  # long prompts go in portions of 2,048 tokens
            for r in ids:
                for at in range(0, args.prompt_len, 2048):
                    runner.step([StepEntry(r, rng.integers(0, vocab, min(2048, args.prompt_len - at)).tolist(), [])])
            return ids
        per_step = max(1, 4096 // args.prompt_len)
        for i in range(0, batch, per_step):
            runner.step([StepEntry(r, rng.integers(0, vocab, args.prompt_len).tolist(), [])
                         for r in ids[i:i + per_step]])
        return ids

    def decode_device(batch: int, steps: int, warmup: int, tag: str) -> tuple[float, float, int]:
        """(tokens/s, ms per step, own kernel launches) of ``steps`` decode steps timed on the device."""
        ids = fill(batch, tag)
        feeds = rng.integers(0, vocab, (steps + warmup, batch)).tolist()
        for w in range(warmup):
            engine.sampler.greedy(runner.step([StepEntry(r, [feeds[w][j]], [0]) for j, r in enumerate(ids)]))
        torch.cuda.synchronize()
        launches0 = ops.launch_count()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for s in range(steps):
            engine.sampler.greedy(runner.step([StepEntry(r, [feeds[warmup + s][j]], [0]) for j, r in enumerate(ids)]))
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        launches = ops.launch_count() - launches0
        for r in ids:
            runner.release(r)
        return batch * 1000.0 / ms, ms, launches

    def decode_bytes(batch: int, steps: int, warmup: int) -> float:
        mean_ctx = args.prompt_len + warmup + (steps + 1) / 2
        return runner.weight_bytes_per_step() + batch * mean_ctx * runner.kv_bytes_per_token()

    if args.only == "decode":
        value, ms_step, launches = decode_device(args.batch, args.steps, args.warmup, "d")
        print(json.dumps({"only": "decode", "batch": args.batch, "tokens_per_s": round(value, 1),
                          "ms_per_step": round(ms_step, 4), "gpu_launches": launches}))
        return 0
    if args.only == "prefill":
        T = args.chunk
        all_ms = []
        for w in range(args.warmup + args.steps):
            for at in range(0, args.prefix, 2048):  # untimed: the tokens in front of the timed portion
                runner.step([StepEntry(f"p{w}", rng.integers(0, vocab, min(2048, args.prefix - at)).tolist(), [])])
            toks = rng.integers(0, vocab, T).tolist()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.step([StepEntry(f"p{w}", toks, [T - 1])])
            stop.record()
            torch.cuda.synchronize()
            runner.release(f"p{w}")
            all_ms.append(round(start.elapsed_time(stop), 3))
        print(json.dumps({"only": "prefill", "tokens": T, "prefix": args.prefix, "ms_last": all_ms[-1], "ms_each": all_ms}))
        return 0

    # ---- prefill of one 2,048-token prompt in one step (median of five).  It is the one phase that runs at the
    # power cap: single runs of the same step vary between 21.4 and 24.8 ms with the power management's state
    T = 2048
    # warm-up until the step of this shape has been captured as a graph (the runner does that once a shape has
    # come up `mixed_graph_after` times), so that the timed steps are what a running engine repeats
    for w in range(max(3, getattr(runner, "mixed_graph_after", 0) + 2)):
        runner.step([StepEntry(f"pw{w}", rng.integers(0, vocab, T).tolist(), [T - 1])])
        runner.release(f"pw{w}")
    torch.cuda.synchronize()

    def timed_prefill(tag: str, pause: float) -> list[float]:
        out = []
        for w in range(5):
            toks = rng.integers(0, vocab, T).tolist()
            if pause:
                time.sleep(pause)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.step([StepEntry(f"{tag}{w}", toks, [T - 1])])
            stop.record()
            torch.cuda.synchronize()
            out.append(start.elapsed_time(stop))
            runner.release(f"{tag}{w}")
        return out

    # A step of 2,048 prompt tokens draws the full 1,000 W: back to back, the second or third step already runs at
    # the clock the power cap sustains (1.3 to 1.5 GHz instead of 1.97).  Both figures are taken, each against the
    # peak that was measured the same way: a step by itself after a pause (median of five) against the burst
    # rate of the matmul, and five steps back to back (median) against the rate sustained under the cap.
    times = timed_prefill("p", 0.3)
    sustained = timed_prefill("q", 0.0)
    prefill_ms = sorted(times)[len(times) // 2]
    sustained_ms = sorted(sustained)[len(sustained) // 2]
    c = runner.config
    per_token_matmul = sum(e for e in [
        2 * c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim,
        2 * c.num_attention_heads * c.head_dim * c.hidden_size,
        2 * c.hidden_size * 2 * c.intermediate_size,
        2 * c.intermediate_size * c.hidden_size]) * c.num_hidden_layers
    attn_flops = 4 * c.num_attention_heads * c.head_dim * (T * (T + 1) // 2) * c.num_hidden_layers
    flops = T * per_token_matmul + attn_flops + 2 * c.hidden_size * c.vocab_size
    prefill = {"value": round(T * 1000.0 / prefill_ms, 1), "tokens": T, "ms": round(prefill_ms, 3),
               "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "tflops": round(flops / (prefill_ms * 1e-3) / 1e12, 1), "peak_tflops": pk["bf16_tflops"],
               "ms_each": [round(t, 2) for t in times],
               "sustained": {"ms": round(sustained_ms, 3), "value": round(T * 1000.0 / sustained_ms, 1),
                             "frac": round(flops / (sustained_ms * 1e-3) / (pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) * 1e12), 4),
                             "peak_tflops": pk.get("bf16_tflops_sustained", pk["bf16_tflops"]),
                             "ms_each": [round(t, 2) for t in sustained]}}

    # ---- headline: decode at --batch, device-timed, with clocks sampled
    with ClockSampler() as clocks:
        value, ms_step, launches = decode_device(args.batch, args.steps, args.warmup, "d")
    clock_summary = clocks.summary()
    achieved = decode_bytes(args.batch, args.steps, args.warmup) / (ms_step * 1e-3) / 1e9

    # ---- end to end through the public engine calls: host tokens in, host tokens out, every step
    for j in range(args.batch):
        engine.add_request(Request(f"e{j}", None, rng.integers(0, vocab, args.prompt_len).tolist(),
                                   # room for the steps during which later prompts are still being admitted: no
                                   # request may finish (and no smaller batch bucket appear) inside the timed loop
                                   SamplingParams(max_tokens=args.steps + args.warmup + 2 * args.batch + 16,
                                                  temperature=0.0, ignore_eos=True), float(j)))
    while any(s.num_output_tokens == 0 for s in engine.scheduler.running) or engine.scheduler.waiting:
        engine.step()
    # The prompts of all requests went in as one step of 8,192 tokens, which runs at the GPU's power cap; for some
    # tens of milliseconds afterwards the SM clock stays at 1.3 to 1.7 GHz and a decode step takes 3.5 ms instead
    # of 2.9.  The device-timed figure above is taken at full clocks, so this one waits until they are back.
    engine.drain()
    torch.cuda.synchronize()
    time.sleep(0.5)
    for _ in range(args.warmup):
        engine.step()
    engine.drain()  # the engine launches a decode step before it has read the tokens of the step before:
    torch.cuda.synchronize()  # nothing is in flight when the clock starts, and none when it stops
    t0 = time.perf_counter()
    for _ in range(args.steps):
        engine.step()
    engine.drain()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    h2d = engine.runner.last_h2d_bytes
    while engine.scheduler.has_work():
        engine.step()

    points = {}
    if not args.no_points:
        pts_steps = max(16, args.steps // 2)
        points["decode_b1"] = round(decode_device(1, pts_steps, 3, "a")[0], 1)
        points["decode_b64"] = round(decode_device(64, pts_steps, 3, "b")[0], 1)

    kernels = {} if args.no_kernels else kernel_fractions(engine, args.batch, args.prompt_len, 2048, pk)

    line = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2048 tokens (Qwen2.5-7B bf16)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random token ids, random-init weights N(0, 0.02)",
        "config": {"model": "Qwen2.5-7B shape", "global_batch": args.batch, "seq_len": args.prompt_len,
                   "context_len": ctx_len, "parallelism": "single GPU", "layers": c.num_hidden_layers,
                   "layers_of_model": SHAPE_7B["num_hidden_layers"], "hidden": c.hidden_size,
                   "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
                   "intermediate": c.intermediate_size, "vocab": c.vocab_size, "kv_block": page,
                   "l2": "inputs larger than L2 (weights read every step)", "cuda_graphs": not args.no_graphs,
                   "order": "prefill first, then decode", "peaks": pk_kind,
                   "prefill_timing": "each step by itself after 0.3 s idle, against the burst peak; sustained: five back to back, against the sustained peak",
                   "e2e_settle": "0.5 s idle between the prompt phase and the timed decode steps"},
        "e2e": {"value": round(args.batch * 1000.0 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "kernels": kernels,
        "clocks": clock_summary,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
